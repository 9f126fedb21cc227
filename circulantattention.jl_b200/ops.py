"""Thin tensor-level wrappers over the C ABI: shape bookkeeping, output
allocation (the caller owns every buffer, as CUDA.jl's pool does on the Julia
side) and the ctypes calls.  No arithmetic happens here."""
from __future__ import annotations

import math
import threading
from dataclasses import dataclass

import torch

from . import _lib, jl
from ._lib import CA_BF16, CA_C64, CA_F32, ca_desc, check, lib, ptr  # noqa: F401  (re-exported: parallel.py uses ops.lib / ops.check)


@dataclass(frozen=True)
class Meta:
    """What a windowed kernel needs to know about a (spatial..., c, units) tensor."""
    spatial: tuple
    channels: int
    units: int
    ws: int
    cplx: bool
    bf16: bool = False      # bfloat16 storage (fused attention only)

    @property
    def ndim(self):
        return len(self.spatial)

    @property
    def H(self):
        return self.spatial[0]

    @property
    def W(self):
        return self.spatial[1] if len(self.spatial) == 2 else 1

    @property
    def Np(self):
        return self.H * self.W

    @property
    def K(self):
        return self.ws ** self.ndim

    def desc(self, similarity=0, normalizer=0, scale=1.0, Wk=0, wk_off=0, units=None, W=None):
        return ca_desc(self.H, self.W if W is None else W, self.ndim, self.channels,
                       self.units if units is None else units, self.ws,
                       CA_C64 if self.cplx else (CA_BF16 if self.bf16 else CA_F32), similarity, normalizer, Wk, wk_off,
                       float(scale))


def meta_of(x: torch.Tensor, ws: int) -> Meta:
    if x.ndim not in (3, 4):
        raise AssertionError(f"expected a (spatial..., channels, batch) array with 1 or 2 spatial dims, got {tuple(x.shape)}")
    return Meta(tuple(x.shape[:-2]), x.shape[-2], x.shape[-1], int(ws), x.is_complex(), x.dtype == torch.bfloat16)


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream():
    """Handle (cudaStream_t as an integer) of torch's current stream on the current device."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


_NVTX = [False]


def enable_nvtx(flag: bool = True) -> bool:
    """NVTX ranges ("circatt.fwd", "circatt.bwd", "circatt.halo") around the library's calls, for timeline
    profilers; off by default (a range costs two host calls).  Returns the previous setting."""
    old, _NVTX[0] = _NVTX[0], bool(flag)
    return old


class _on_device:
    """`with _on_device(t.device)`: makes that device current for the C ABI calls inside, without the cost of
    a device switch when it already is (the common case).  With a `name` and NVTX enabled the block is also
    an NVTX range."""
    __slots__ = ("index", "prev", "name")

    def __init__(self, device, name=None):
        self.index = device.index if device.index is not None else torch.cuda.current_device()
        self.prev = None
        self.name = name if (name and _NVTX[0]) else None

    def __enter__(self):
        cur = torch.cuda.current_device()
        if cur != self.index:
            self.prev = cur
            torch.cuda.set_device(self.index)
        if self.name:
            torch.cuda.nvtx.range_push(self.name)

    def __exit__(self, *exc):
        if self.name:
            torch.cuda.nvtx.range_pop()
        if self.prev is not None:
            torch.cuda.set_device(self.prev)
        return False


def require_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise RuntimeError("CirculantAttention is only CUDA compatible (no CPU path): got a tensor on " + str(t.device))


def _dense_ok(t, cplx=None):
    want = (torch.float32, torch.complex64, torch.bfloat16)
    if t.dtype not in want:
        raise TypeError(f"only Float32, ComplexF32 and (fused attention) BFloat16 are supported, got {t.dtype}")
    return jl.colmajor(t)


def structure(spatial, ws, batch, device):
    """rowPtr (Np+1, batch...) and colVal (Np*K, batch...) Int32, 1-based."""
    spatial = tuple(spatial)
    H, W = spatial[0], (spatial[1] if len(spatial) == 2 else 1)
    Np, K = H * W, ws ** len(spatial)
    nb = int(math.prod(batch)) if batch else 1
    rowptr = jl.empty((Np + 1,) + tuple(batch), torch.int32, device)
    colval = jl.empty((Np * K,) + tuple(batch), torch.int32, device)
    with _on_device(rowptr.device):
        check(lib.ca_structure(H, W, len(spatial), ws, nb, ptr(rowptr), ptr(colval), _stream()))
    return rowptr, colval


def _operator_workspace(d, device):
    """Scratch of ca_operator_workspace() bytes, or None when the shape runs on the generic kernels."""
    n = lib.ca_operator_workspace(d)
    return torch.empty(n, dtype=torch.uint8, device=device) if n else None


def similarity(kind, x, y, ws, scale=1.0):
    require_cuda(x, y)
    x, y = _dense_ok(x), _dense_ok(y)
    m = meta_of(x, ws)
    nz = jl.empty((m.Np * m.K, m.units), torch.float32, x.device)
    d = m.desc(similarity=kind, scale=scale)
    with _on_device(x.device):
        ws_buf = _operator_workspace(d, x.device)
        check(lib.ca_similarity(d, ptr(x), ptr(y), ptr(nz), ptr(ws_buf), _stream()))
    return nz


def similarity_bwd(kind, x, y, ws, dS, scale=1.0):
    x, y = _dense_ok(x), _dense_ok(y)
    dS = jl.colmajor(dS)
    m = meta_of(x, ws)
    dx, dy = jl.empty(x.shape, x.dtype, x.device), jl.empty(y.shape, y.dtype, y.device)
    d = m.desc(similarity=kind, scale=scale)
    with _on_device(x.device):
        ws_buf = _operator_workspace(d, x.device)
        check(lib.ca_similarity_bwd(d, ptr(x), ptr(y), ptr(dS), ptr(dx), ptr(dy), ptr(ws_buf), _stream()))
    return dx, dy


def _nz_meta(spatial, ws, units):
    return Meta(tuple(spatial), 1, int(units), int(ws), False)


def row_normalize(nz, spatial, ws, normalizer, out=None, want_stats=False):
    require_cuda(nz)
    nz = jl.colmajor(nz)
    units = nz.numel() // nz.shape[0]
    m = _nz_meta(spatial, ws, units)
    out = jl.empty(nz.shape, torch.float32, nz.device) if out is None else out
    stats = jl.empty((m.Np, units), torch.float32, nz.device) if want_stats else None
    with _on_device(nz.device):
        check(lib.ca_row_normalize(m.desc(normalizer=normalizer), ptr(nz), ptr(out), ptr(stats), _stream()))
    return (out, stats) if want_stats else out


def row_normalize_bwd(p, dp, spatial, ws, normalizer):
    p, dp = jl.colmajor(p), jl.colmajor(dp)
    units = p.numel() // p.shape[0]
    m = _nz_meta(spatial, ws, units)
    ds = jl.empty(p.shape, torch.float32, p.device)
    with _on_device(p.device):
        check(lib.ca_row_normalize_bwd(m.desc(normalizer=normalizer), ptr(p), ptr(dp), ptr(ds), _stream()))
    return ds


def apply(nz, v, ws, transpose=False, out=None):
    """A (x) v or A^T (x) v.  nz: (Np*K, ua); v: (spatial..., c, uv); ua, uv broadcast."""
    require_cuda(nz, v)
    nz, v = jl.colmajor(nz), _dense_ok(v)
    m = meta_of(v, ws)
    ua = nz.numel() // nz.shape[0]
    units = max(ua, m.units)
    if ua not in (1, units) or m.units not in (1, units):
        raise AssertionError(f"batch dims of A ({ua}) and of x ({m.units}) do not broadcast")
    if nz.shape[0] != m.Np * m.K:
        raise AssertionError(f"A has {nz.shape[0]} stored entries per batch, x needs {m.Np * m.K}")
    if out is None:
        out = jl.empty(tuple(v.shape[:-1]) + (units,), v.dtype, v.device)
    d = m.desc(units=units)
    with _on_device(v.device):
        ws_buf = _operator_workspace(d, v.device)
        check(lib.ca_apply(d, ptr(nz), ptr(v), ptr(out), int(transpose), int(ua == 1 and units > 1),
                           int(m.units == 1 and units > 1), ptr(ws_buf), _stream()))
    return out


# Transient scratch per (device, stream, purpose): grown on demand and reused by later calls on the
# same stream, which is safe because work on one stream is ordered.  Buffers that must outlive the
# call (the forward workspace kept for the backward) are never taken from here.
_SCRATCH = {}


def _scratch(purpose, nbytes, device):
    if not nbytes:
        return None
    key = (device.index, _stream(), purpose)
    buf = _SCRATCH.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(nbytes, dtype=torch.uint8, device=device)
        _SCRATCH[key] = buf
    return buf


def release_scratch():
    """Drops the cached transient workspaces (they are re-created on demand)."""
    _SCRATCH.clear()


# ------------------------------------------------------------------ device-side failure reporting
_STATUS = {}
_REGISTERED = threading.local()


def _status_word(device):
    """The int32 on `device` in which kernels flag a wait that ran out; registered with the library for
    the calling host thread (the registration is per thread, so it is redone when the thread last
    registered another device's word)."""
    w = _STATUS.get(device.index)
    if w is None:
        w = torch.zeros(1, dtype=torch.int32, device=device)
        _STATUS[device.index] = w
    if getattr(_REGISTERED, "index", None) != device.index:
        check(lib.ca_status_word(ptr(w)))
        _REGISTERED.index = device.index
    return w


def check_status(device=None):
    """Synchronising check: raises if a kernel of this library gave up a bounded device-side wait since the
    last check on `device` (its tile then holds NaN).  Call it where the program synchronises anyway."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    w = _STATUS.get(device.index)
    if w is None:
        return
    flag = int(w.item())
    if flag:
        w.zero_()
        raise _lib.CircAttError("a circatt_b200 kernel gave up a bounded wait for a shared-memory stage copy; "
                                "the outputs of that call hold NaN")


def attention_fwd(kind, normalizer, q, k, v, ws, want_nz, scale=None, band=None, keep_workspace=False):
    """Fused forward on (spatial..., c, units) tensors.  Returns (y, nz | None, stats), plus the workspace
    tensor when `keep_workspace` (hand it to attention_bwd as `fwd_workspace`).
    `band=(Wk, wk_off)` selects band mode: k, v then have Wk columns."""
    require_cuda(q, k, v)
    q, k, v = _dense_ok(q), _dense_ok(k), _dense_ok(v)
    m = meta_of(q, ws)
    scale = 1.0 / math.sqrt(m.channels) if scale is None else scale
    Wk, wk_off = band if band else (0, 0)
    d = m.desc(similarity=kind, normalizer=normalizer, scale=scale, Wk=Wk, wk_off=wk_off)
    y = jl.empty(q.shape, q.dtype, q.device)
    nz = jl.empty((m.Np * m.K, m.units), torch.float32, q.device) if want_nz else None
    stats = jl.empty((m.Np, m.units), torch.float32, q.device)
    nbytes = lib.ca_attention_fwd_workspace(d, int(want_nz))
    with _on_device(q.device, "circatt.fwd"):
        _status_word(q.device)
        if keep_workspace:
            wsb = torch.empty(nbytes, dtype=torch.uint8, device=q.device) if nbytes else None
        else:
            wsb = _scratch("fwd", nbytes, q.device)
        check(lib.ca_attention_fwd(d, ptr(q), ptr(k), ptr(v), ptr(y), ptr(nz), ptr(stats), ptr(wsb), _stream()))
    return (y, nz, stats, wsb) if keep_workspace else (y, nz, stats)


def attention_bwd(kind, normalizer, q, k, v, y, dy, stats, ws, nz=None, dA=None, scale=None, fwd_workspace=None):
    """Fused backward.  Returns (dq, dk, dv).  `fwd_workspace`: the workspace kept from the matching
    attention_fwd(keep_workspace=True) call, untouched since (spares packing k and v again)."""
    q, k, v, y, dy = (_dense_ok(t) for t in (q, k, v, y, dy))
    m = meta_of(q, ws)
    scale = 1.0 / math.sqrt(m.channels) if scale is None else scale
    d = m.desc(similarity=kind, normalizer=normalizer, scale=scale)
    dq, dk, dv = (jl.empty(q.shape, q.dtype, q.device) for _ in range(3))
    if dA is not None:
        dA = jl.colmajor(dA)
    with _on_device(q.device, "circatt.bwd"):
        _status_word(q.device)
        wsb = _scratch("bwd", lib.ca_attention_bwd_workspace(d, int(dA is not None)), q.device)
        check(lib.ca_attention_bwd(d, ptr(q), ptr(k), ptr(v), ptr(y), ptr(dy), ptr(stats), ptr(nz), ptr(dA),
                                   ptr(dq), ptr(dk), ptr(dv), ptr(wsb), ptr(fwd_workspace), _stream()))
    return dq, dk, dv


def copy_chunks(jobs):
    """Several strided device copies in one launch (ca_copy_chunks).  `jobs`: tuples
    (src_ptr, dst_ptr, chunk_bytes, nchunks, src_stride_bytes, dst_stride_bytes) with integer addresses;
    longer lists are split into launches of CA_MAX_CHUNK_JOBS."""
    for i in range(0, len(jobs), _lib.CA_MAX_CHUNK_JOBS):
        part = jobs[i:i + _lib.CA_MAX_CHUNK_JOBS]
        arr = (_lib.ca_chunk_job * len(part))(*[_lib.ca_chunk_job(*j) for j in part])
        check(lib.ca_copy_chunks(arr, len(part), _stream()))


def entmax_scratch_limit(nbytes: int = -1) -> int:
    """Largest A-sized scratch (bytes) the flash-mode entmax forward may use before it switches to the
    scratch-free sweeps; sets it when `nbytes` >= 0.  Returns the previous limit."""
    return int(lib.ca_entmax_scratch_limit(int(nbytes)))


# ------------------------------------------------------------------ algebra
def axpby(alpha, x, beta=0.0, y=None):
    require_cuda(x, y)
    x = jl.colmajor(x)
    y = jl.colmajor(y) if y is not None else None
    out = jl.empty(x.shape, torch.float32, x.device)
    with _on_device(x.device):
        check(lib.ca_axpby(x.numel(), float(alpha), ptr(x), float(beta), ptr(y), ptr(out), _stream()))
    return out


def _b12(batch):
    batch = tuple(batch)
    if len(batch) > 2:
        raise NotImplementedError("at most two batch dims (heads, batch) are supported")
    return (batch + (1, 1))[:2]


def scale_batch(c, nz):
    """nz (inner, a...) times c (c...) with Julia-style extent-1 broadcasting."""
    require_cuda(c, nz)
    c, nz = jl.colmajor(c), jl.colmajor(nz)
    a1, a2 = _b12(nz.shape[1:])
    c1, c2 = _b12(c.shape)
    o1, o2 = max(a1, c1), max(a2, c2)
    nb = max(nz.ndim - 1, c.ndim)
    out = jl.empty((nz.shape[0],) + (o1, o2)[:nb], torch.float32, nz.device)
    with _on_device(nz.device):
        check(lib.ca_scale_batch(nz.shape[0], o1, o2, ptr(nz), a1, a2, ptr(c), c1, c2, ptr(out), _stream()))
    return out


def dot_batch(x, y=None):
    """per-slice sum_n x*y (y None: sum of x); x, y: (inner, b...) broadcasting -> (b...)"""
    require_cuda(x, y)
    x = jl.colmajor(x)
    x1, x2 = _b12(x.shape[1:])
    if y is not None:
        y = jl.colmajor(y)
        y1, y2 = _b12(y.shape[1:])
    else:
        y1 = y2 = 1
    o1, o2 = max(x1, y1), max(x2, y2)
    nb = max(x.ndim, y.ndim if y is not None else 0) - 1
    out = jl.empty((o1, o2)[:nb] if nb else (1,), torch.float32, x.device)
    with _on_device(x.device):
        check(lib.ca_dot_batch(x.shape[0], o1, o2, ptr(x), x1, x2, ptr(y), y1, y2, ptr(out), _stream()))
    return out


def sum_batch(nz, sum1, sum2):
    require_cuda(nz)
    nz = jl.colmajor(nz)
    b1, b2 = _b12(nz.shape[1:])
    o = (1 if sum1 else b1, 1 if sum2 else b2)[:nz.ndim - 1]
    out = jl.empty((nz.shape[0],) + o, torch.float32, nz.device)
    with _on_device(nz.device):
        check(lib.ca_sum_batch(nz.shape[0], b1, b2, int(sum1), int(sum2), ptr(nz), ptr(out), _stream()))
    return out


def sum_rows(nz, spatial, ws):
    require_cuda(nz)
    nz = jl.colmajor(nz)
    units = nz.numel() // nz.shape[0]
    m = _nz_meta(spatial, ws, units)
    out = jl.empty((m.Np, 1) + tuple(nz.shape[1:]), torch.float32, nz.device)
    with _on_device(nz.device):
        check(lib.ca_sum_rows(m.desc(), ptr(nz), ptr(out), _stream()))
    return out


def sum_cols(nz, spatial, ws):
    require_cuda(nz)
    nz = jl.colmajor(nz)
    units = nz.numel() // nz.shape[0]
    m = _nz_meta(spatial, ws, units)
    out = jl.empty((1, m.Np) + tuple(nz.shape[1:]), torch.float32, nz.device)
    with _on_device(nz.device):
        check(lib.ca_sum_cols(m.desc(), ptr(nz), ptr(out), _stream()))
    return out


# ------------------------------------------------------------------ backward stages (band split)
def _stage_ws(d, device):
    n = lib.ca_attention_bwd_stage_workspace(d)
    return torch.empty(max(n, 16), dtype=torch.uint8, device=device) if n else None


def attention_bwd_pre(kind, normalizer, q, k, v, y, dy, stats, ws, scale=None):
    """D of ca_attention_bwd_pre for band-local tensors (no A cotangent)."""
    q, k, v, y, dy = (_dense_ok(t) for t in (q, k, v, y, dy))
    m = meta_of(q, ws)
    scale = 1.0 / math.sqrt(m.channels) if scale is None else scale
    d = m.desc(similarity=kind, normalizer=normalizer, scale=scale)
    D = jl.empty((m.Np, m.units), torch.float32, q.device)
    with _on_device(q.device):
        check(lib.ca_attention_bwd_pre(d, ptr(q), ptr(k), ptr(v), ptr(y), ptr(dy), ptr(stats), None, None, ptr(D),
                                       _stream()))
    return D


def attention_bwd_dq(kind, normalizer, q, k, v, dy, stats, D, ws, scale=None, band=None):
    """dq stage; in band mode k, v carry Wk = W + 2p columns."""
    q, k, v, dy = (_dense_ok(t) for t in (q, k, v, dy))
    m = meta_of(q, ws)
    scale = 1.0 / math.sqrt(m.channels) if scale is None else scale
    Wk, wk_off = band if band else (0, 0)
    d = m.desc(similarity=kind, normalizer=normalizer, scale=scale, Wk=Wk, wk_off=wk_off)
    dq = jl.empty(q.shape, q.dtype, q.device)
    wsb = _stage_ws(d, q.device)
    with _on_device(q.device):
        check(lib.ca_attention_bwd_dq(d, ptr(q), ptr(k), ptr(v), ptr(dy), ptr(stats), ptr(D), None, ptr(dq),
                                      ptr(wsb), _stream()))
    return dq


def attention_bwd_dkdv(kind, normalizer, q, k, v, dy, stats, D, ws, scale=None, band=None):
    """dk/dv stage; in band mode q, dy, stats, D carry Wk = W + 2p columns and k, v are band-local."""
    q, k, v, dy = (_dense_ok(t) for t in (q, k, v, dy))
    m = meta_of(k, ws)
    scale = 1.0 / math.sqrt(m.channels) if scale is None else scale
    Wk, wk_off = band if band else (0, 0)
    d = m.desc(similarity=kind, normalizer=normalizer, scale=scale, Wk=Wk, wk_off=wk_off)
    dk, dv = jl.empty(k.shape, k.dtype, k.device), jl.empty(k.shape, k.dtype, k.device)
    wsb = _stage_ws(d, k.device)
    with _on_device(k.device):
        check(lib.ca_attention_bwd_dkdv(d, ptr(q), ptr(k), ptr(v), ptr(dy), ptr(stats), ptr(D), None, ptr(dk),
                                        ptr(dv), ptr(wsb), _stream()))
    return dk, dv
