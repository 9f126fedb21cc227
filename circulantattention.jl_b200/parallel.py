"""Multi-GPU plumbing: one process per GPU, `torch.distributed` for the only
exchange the path has.

Two ways to shard, neither of which exists in the reference (it is a
single-device package):

* batch x head units are independent in every kernel, so `shard_units` hands
  each rank a contiguous range of units and nothing is communicated;
* for images too large for one GPU the slow spatial axis W is cut into bands
  (`BandPlan`).  A rank then needs `p = (ws-1)/2` columns of the key-side
  tensors from its two neighbours `r-1` and `r+1` (mod R: the modulo is the
  circular wrap of the window); `exchange_halos` does that with point-to-point
  sends (NCCL over NVLink on GPUs, gloo on CPU ranks): all tensors of one
  exchange travel as one message per neighbour, land in the rank's own staging
  buffer first, and the kernels run in band mode on the extended slabs, every
  thread block reading local memory only.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

from . import jl, ops


def shard_units(units: int, world: int, rank: int) -> Tuple[int, int]:
    """(first unit, number of units) of `rank`: contiguous, the first `units % world`
    ranks hold one more; ranks beyond `units` hold none."""
    if units < 0 or world < 1 or not 0 <= rank < world:
        raise ValueError(f"bad sharding request: units={units} world={world} rank={rank}")
    base, extra = divmod(units, world)
    count = base + (1 if rank < extra else 0)
    start = rank * base + min(rank, extra)
    return start, count


def take_units(x: torch.Tensor, world: int, rank: int) -> torch.Tensor:
    """The shard of a head-split (spatial..., c, units) tensor that `rank` owns: a view,
    because a unit is a contiguous block of the column-major array."""
    start, count = shard_units(x.shape[-1], world, rank)
    return x.narrow(x.ndim - 1, start, count)


@dataclass(frozen=True)
class BandPlan:
    """Bands of columns of a (H, W, ...) image over `world` ranks for window `ws`."""
    W: int
    world: int
    ws: int

    def __post_init__(self):
        if self.ws % 2 != 1:
            raise AssertionError(f"filter size M={self.ws} must be odd.")
        if self.world < 1:
            raise ValueError("world must be positive")
        if min(self.widths()) < max(self.p, 1):
            raise ValueError(f"a band of {min(self.widths())} columns is narrower than the halo ({self.p}): "
                             f"W={self.W} cannot be split over {self.world} ranks for window {self.ws}")

    @property
    def p(self) -> int:
        return (self.ws - 1) // 2

    def widths(self) -> List[int]:
        return [shard_units(self.W, self.world, r)[1] for r in range(self.world)]

    def band(self, rank: int) -> Tuple[int, int]:
        """(first column, number of columns) of `rank`."""
        return shard_units(self.W, self.world, rank)

    def neighbours(self, rank: int) -> Tuple[int, int]:
        """(left, right) = ranks holding the columns before / after this band, circularly."""
        return (rank - 1) % self.world, (rank + 1) % self.world

    def take(self, x: torch.Tensor, rank: int) -> torch.Tensor:
        """Band of a (H, W, ...) tensor (column-major copy)."""
        start, width = self.band(rank)
        return jl.colmajor(x.narrow(1, start, width).clone())


def _cview(x: torch.Tensor) -> torch.Tensor:
    """C-contiguous view (..., W, H) of a column-major (H, W, ...) tensor."""
    x = jl.colmajor(x)
    return x.permute(tuple(range(x.ndim - 1, -1, -1)))


# Staging buffers of the exchange, kept per (direction, size, dtype, device): the halos of all tensors of
# one exchange travel as ONE message per neighbour, so the buffers are reused step after step.
_STAGING = {}


def _staging(tag, numel, dtype, device):
    key = (tag, numel, dtype, str(device))
    buf = _STAGING.get(key)
    if buf is None:
        buf = torch.empty(numel, dtype=dtype, device=device)
        _STAGING[key] = buf
    return buf


class Ring:
    """The ring of bands through the library's own NCCL binding (ca_comm_* / ca_halo_exchange of the C ABI):
    the path a host without torch.distributed (the Julia package) uses.  Rank 0 creates the 128-byte id with
    `Ring.unique_id()` and hands it to the other ranks by any means; every rank then constructs
    `Ring(rank, world, id)` with its GPU current."""

    def __init__(self, rank: int, world: int, unique_id: bytes = None):
        import ctypes
        self.rank, self.world = int(rank), int(world)
        self._h = ctypes.c_void_p()
        buf = ctypes.create_string_buffer(bytes(unique_id), 128) if unique_id is not None else None
        ops.check(ops.lib.ca_comm_init(self.rank, self.world, buf, ctypes.byref(self._h)))

    @staticmethod
    def unique_id() -> bytes:
        import ctypes
        buf = ctypes.create_string_buffer(128)
        ops.check(ops.lib.ca_comm_unique_id(buf))
        return buf.raw

    def exchange(self, send_left, send_right, recv_left, recv_right):
        """Contiguous device buffers of equal size; ordered on torch's current stream."""
        n = send_left.numel() * send_left.element_size()
        ops.check(ops.lib.ca_halo_exchange(self._h, ops.ptr(send_left), ops.ptr(send_right), ops.ptr(recv_left),
                                           ops.ptr(recv_right), n, ops._stream()))

    def close(self):
        if self._h:
            ops.check(ops.lib.ca_comm_destroy(self._h))
            self._h = None


def exchange_halos(xs, p: int, group=None, ring: "Ring" = None):
    """Extended slabs (H, Wb + 2p, ...) of the band-local (H, Wb, ...) tensors `xs` (same dtype and device):
    `p` columns from the left neighbour, the band, `p` columns from the right neighbour.

    All tensors of the call share one exchange: their outgoing halos are gathered into one contiguous
    message per neighbour (two sends and two receives in one grouped point-to-point call, whatever the
    number of tensors), and the incoming ones are scattered into the slabs.  Without an initialised
    process group (or world size 1) the band is the whole image and the halos are its own wrapped
    columns."""
    xs = list(xs)
    if not xs:
        return []
    ts, exts = [], []
    on_gpu = xs[0].is_cuda
    for x in xs:
        if x.ndim < 2:
            raise ValueError("expected a (H, W, ...) tensor")
        Wb = x.shape[1]
        if p < 1 or Wb < p:
            raise ValueError(f"band of {Wb} columns cannot supply a halo of {p}")
        if x.dtype != xs[0].dtype or x.device != xs[0].device:
            raise TypeError("tensors of one exchange must share dtype and device")
        t = _cview(x)                                        # (..., Wb, H)
        ext = torch.empty(t.shape[:-2] + (Wb + 2 * p, t.shape[-1]), dtype=t.dtype, device=t.device)
        if not on_gpu:
            ext.narrow(-2, p, Wb).copy_(t)
        ts.append(t)
        exts.append(ext)
    if ring is not None:
        world = ring.world
    else:
        world = dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1
    dtype, device = ts[0].dtype, ts[0].device
    esize = ts[0].element_size()
    sizes = [t.numel() // t.shape[-2] * p for t in ts]
    total = sum(sizes)

    def geometry(t):
        """(trailing index count, bytes of one column, band columns) of a (..., Wb, H) view."""
        Wb, H = t.shape[-2], t.shape[-1]
        return t.numel() // (Wb * H), H * esize, Wb

    if world == 1:
        if on_gpu:
            # one launch: the bands into their slabs, and the wrapped columns into the halos
            jobs = []
            for t, ext in zip(ts, exts):
                outer, col, Wb = geometry(t)
                src, dst, ss, ds = t.data_ptr(), ext.data_ptr(), Wb * col, (Wb + 2 * p) * col
                jobs.append((src, dst + p * col, Wb * col, outer, ss, ds))
                jobs.append((src + (Wb - p) * col, dst, p * col, outer, ss, ds))
                jobs.append((src, dst + (p + Wb) * col, p * col, outer, ss, ds))
            with ops._on_device(device, "circatt.halo"):
                ops.copy_chunks(jobs)
        else:
            for t, ext in zip(ts, exts):
                Wb = t.shape[-2]
                ext.narrow(-2, 0, p).copy_(t.narrow(-2, Wb - p, p))
                ext.narrow(-2, p + Wb, p).copy_(t.narrow(-2, 0, p))
    else:
        to_right, to_left = _staging("to_right", total, dtype, device), _staging("to_left", total, dtype, device)
        from_left, from_right = _staging("from_left", total, dtype, device), _staging("from_right", total, dtype, device)
        if on_gpu:
            # one launch gathers the outgoing columns of every tensor into the two messages and copies the
            # bands into their slabs; one more scatters the incoming columns
            jobs, off = [], 0
            for t, ext, n in zip(ts, exts, sizes):
                outer, col, Wb = geometry(t)
                src, ss = t.data_ptr(), Wb * col
                jobs.append((src, ext.data_ptr() + p * col, Wb * col, outer, ss, (Wb + 2 * p) * col))
                jobs.append((src + (Wb - p) * col, to_right.data_ptr() + off * esize, p * col, outer, ss, p * col))
                jobs.append((src, to_left.data_ptr() + off * esize, p * col, outer, ss, p * col))
                off += n
            with ops._on_device(device, "circatt.halo"):
                ops.copy_chunks(jobs)
        else:
            off = 0
            for t, n in zip(ts, sizes):
                Wb = t.shape[-2]
                shape = t.shape[:-2] + (p, t.shape[-1])
                to_right[off:off + n].view(shape).copy_(t.narrow(-2, Wb - p, p))   # the right neighbour's left halo
                to_left[off:off + n].view(shape).copy_(t.narrow(-2, 0, p))         # the left neighbour's right halo
                off += n
        if ring is not None:
            ring.exchange(to_left, to_right, from_left, from_right)
        else:
            rank = dist.get_rank(group)
            left, right = (rank - 1) % world, (rank + 1) % world
            peer = lambda r: dist.get_global_rank(group, r) if group is not None else r
            reqs = dist.batch_isend_irecv([
                dist.P2POp(dist.isend, to_right, peer(right), group, tag=0),
                dist.P2POp(dist.isend, to_left, peer(left), group, tag=1),
                dist.P2POp(dist.irecv, from_left, peer(left), group, tag=0),
                dist.P2POp(dist.irecv, from_right, peer(right), group, tag=1),
            ])
            for r in reqs:
                r.wait()
        if on_gpu:
            jobs, off = [], 0
            for t, ext, n in zip(ts, exts, sizes):
                outer, col, Wb = geometry(t)
                ds = (Wb + 2 * p) * col
                jobs.append((from_left.data_ptr() + off * esize, ext.data_ptr(), p * col, outer, p * col, ds))
                jobs.append((from_right.data_ptr() + off * esize, ext.data_ptr() + (p + Wb) * col, p * col, outer, p * col, ds))
                off += n
            with ops._on_device(device, "circatt.halo"):
                ops.copy_chunks(jobs)
        else:
            off = 0
            for t, ext, n in zip(ts, exts, sizes):
                Wb = t.shape[-2]
                shape = t.shape[:-2] + (p, t.shape[-1])
                ext.narrow(-2, 0, p).copy_(from_left[off:off + n].view(shape))
                ext.narrow(-2, p + Wb, p).copy_(from_right[off:off + n].view(shape))
                off += n
    return [ext.permute(tuple(range(ext.ndim - 1, -1, -1))) for ext in exts]


_SIDE = {}


def _side_stream(device):
    """One helper stream per device for the exchange that overlaps the dq sweep."""
    s = _SIDE.get(device.index)
    if s is None:
        s = torch.cuda.Stream(device=device)
        _SIDE[device.index] = s
    return s


def exchange_halo(x: torch.Tensor, p: int, group=None) -> torch.Tensor:
    """Extended slab of one tensor (see exchange_halos)."""
    return exchange_halos([x], p, group)[0]


def band_attention_fwd(kind, q, k, v, ws, group=None, normalizer=0, ring=None):
    """Forward on this rank's band of head-split (H, Wb, c, units) tensors: one exchange (k and v
    together), one kernel call.  Returns (y, stats, k_ext, v_ext); the extended slabs are reused by
    the backward."""
    p = (ws - 1) // 2
    k_ext, v_ext = exchange_halos([k, v], p, group, ring)
    y, _, stats = ops.attention_fwd(kind, normalizer, q, k_ext, v_ext, ws, False, band=(k_ext.shape[1], p))
    return y, stats, k_ext, v_ext


def band_attention_bwd(kind, q, k, v, y, dy, stats, k_ext, v_ext, ws, group=None, normalizer=0, ring=None):
    """Backward on this rank's band.  One more exchange: q, dy, stats and D of the neighbouring columns
    (one message per neighbour) feed the key-owned dk/dv sweep.  The dq sweep needs nothing from the
    neighbours beyond the forward's k and v slabs, so it is queued before the exchange is waited for."""
    p = (ws - 1) // 2
    Wb = q.shape[1]
    H, units = q.shape[0], q.shape[-1]
    D = ops.attention_bwd_pre(kind, normalizer, q, k, v, y, dy, stats, ws)

    def second_exchange():
        if q.dtype == torch.float32:
            # the two scalar planes ride in the same message as q and dy
            return exchange_halos([q, dy, jl.reshape(stats, (H, Wb, units)), jl.reshape(D, (H, Wb, units))], p, group, ring)
        return (exchange_halos([q, dy], p, group, ring) +
                exchange_halos([jl.reshape(stats, (H, Wb, units)), jl.reshape(D, (H, Wb, units))], p, group, ring))

    if q.is_cuda:
        # the exchange runs on a side stream next to the dq sweep (which needs nothing from the neighbours
        # beyond the forward's slabs); the dk/dv sweep waits for both
        main, side = torch.cuda.current_stream(q.device), _side_stream(q.device)
        ready = torch.cuda.Event()
        ready.record(main)                                   # q, dy, stats, D are final here
        dq = ops.attention_bwd_dq(kind, normalizer, q, k_ext, v_ext, dy, stats, D, ws, band=(Wb + 2 * p, p))
        with torch.cuda.stream(side):
            side.wait_event(ready)
            q_ext, dy_ext, stats_ext, D_ext = second_exchange()
            done = torch.cuda.Event()
            done.record(side)
        for t in (q_ext, dy_ext, stats_ext, D_ext):
            t.record_stream(main)                            # allocated on the side stream, read on the main one
        main.wait_event(done)
    else:
        dq = ops.attention_bwd_dq(kind, normalizer, q, k_ext, v_ext, dy, stats, D, ws, band=(Wb + 2 * p, p))
        q_ext, dy_ext, stats_ext, D_ext = second_exchange()
    dk, dv = ops.attention_bwd_dkdv(kind, normalizer, q_ext, k, v, dy_ext,
                                    jl.reshape(stats_ext, (H * (Wb + 2 * p), units)),
                                    jl.reshape(D_ext, (H * (Wb + 2 * p), units)), ws, band=(Wb + 2 * p, p))
    return dq, dk, dv
