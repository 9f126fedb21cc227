"""Band split across real GPUs: one process per GPU, NCCL point-to-point halo
exchange (including the circular wrap between the last and the first rank), results
gathered through files and compared with the oracle.  Skipped with fewer than 2 GPUs."""
import os
import socket
import tempfile

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import circatt_oracle as orc
from tests.helpers import TOL, randn, rel_err, up

pytestmark = pytest.mark.gpu

SHAPE, WS, NHEADS = (64, 48, 32, 2), 7, 2


def _ring_worker(rank, world, tmp):
    """The same band split with the exchange done by the library's own NCCL binding (no torch.distributed):
    the unique id travels through a file, as a Julia launcher would pass it."""
    import sys, time
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, root)
    from __graft_entry__ import load_package
    ca = load_package()
    torch.cuda.set_device(rank)
    idfile = os.path.join(tmp, "nccl_id.bin")
    if rank == 0:
        uid = ca.parallel.Ring.unique_id()
        with open(idfile + ".tmp", "wb") as f:
            f.write(uid)
        os.replace(idfile + ".tmp", idfile)
    else:
        for _ in range(600):
            if os.path.exists(idfile):
                break
            time.sleep(0.05)
        uid = open(idfile, "rb").read()
    ring = ca.parallel.Ring(rank, world, uid)
    try:
        rng = np.random.default_rng(0)
        full = [orc.splitheads(randn(rng, SHAPE), NHEADS) for _ in range(4)]
        plan = ca.parallel.BandPlan(SHAPE[1], world, WS)
        start, width = plan.band(rank)
        q, k, v, dy = (ca.jl.from_numpy(np.asfortranarray(t[:, start:start + width]), f"cuda:{rank}") for t in full)
        y, stats, k_ext, v_ext = ca.parallel.band_attention_fwd(0, q, k, v, WS, ring=ring)
        dq, dk, dv = ca.parallel.band_attention_bwd(0, q, k, v, y, dy, stats, k_ext, v_ext, WS, ring=ring)
        torch.cuda.synchronize()
        np.savez(os.path.join(tmp, f"rank{rank}.npz"), **{n: ca.jl.to_numpy(t) for n, t in
                                                           (("y", y), ("dq", dq), ("dk", dk), ("dv", dv))})
    finally:
        ring.close()


def _worker(rank, world, port, tmp):
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, root)
    from __graft_entry__ import load_package
    ca = load_package()
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        rng = np.random.default_rng(0)                       # every rank draws the same full image
        full = [orc.splitheads(randn(rng, SHAPE), NHEADS) for _ in range(4)]
        plan = ca.parallel.BandPlan(SHAPE[1], world, WS)
        start, width = plan.band(rank)
        q, k, v, dy = (ca.jl.from_numpy(np.asfortranarray(t[:, start:start + width]), f"cuda:{rank}") for t in full)
        y, stats, k_ext, v_ext = ca.parallel.band_attention_fwd(0, q, k, v, WS)
        dq, dk, dv = ca.parallel.band_attention_bwd(0, q, k, v, y, dy, stats, k_ext, v_ext, WS)
        torch.cuda.synchronize()
        np.savez(os.path.join(tmp, f"rank{rank}.npz"), **{n: ca.jl.to_numpy(t) for n, t in
                                                           (("y", y), ("dq", dq), ("dk", dk), ("dv", dv))})
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least 2 GPUs")
def test_band_split_over_nccl_ranks():
    world = min(torch.cuda.device_count(), 4)
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    with tempfile.TemporaryDirectory() as tmp:
        mp.spawn(_worker, args=(world, port, tmp), nprocs=world, join=True)
        parts = [np.load(os.path.join(tmp, f"rank{r}.npz")) for r in range(world)]
        got = {n: np.concatenate([p[n] for p in parts], axis=1).reshape(SHAPE, order="F") for n in ("y", "dq", "dk", "dv")}
    rng = np.random.default_rng(0)
    qn, kn, vn, rn = (randn(rng, SHAPE) for _ in range(4))
    yo, _ = orc.mh_attention(orc.DOT, up(qn), up(kn), up(vn), WS, NHEADS)
    dqo, dko, dvo = orc.mh_attention_pullback(orc.DOT, up(qn), up(kn), up(vn), WS, NHEADS, up(rn))
    for name, want in (("y", yo), ("dq", dqo), ("dk", dko), ("dv", dvo)):
        assert rel_err(got[name], want) < TOL, name


def _check_parts(tmp, world):
    parts = [np.load(os.path.join(tmp, f"rank{r}.npz")) for r in range(world)]
    got = {n: np.concatenate([p[n] for p in parts], axis=1).reshape(SHAPE, order="F") for n in ("y", "dq", "dk", "dv")}
    rng = np.random.default_rng(0)
    qn, kn, vn, rn = (randn(rng, SHAPE) for _ in range(4))
    yo, _ = orc.mh_attention(orc.DOT, up(qn), up(kn), up(vn), WS, NHEADS)
    dqo, dko, dvo = orc.mh_attention_pullback(orc.DOT, up(qn), up(kn), up(vn), WS, NHEADS, up(rn))
    for name, want in (("y", yo), ("dq", dqo), ("dk", dko), ("dv", dvo)):
        assert rel_err(got[name], want) < TOL, name


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least 2 GPUs")
def test_band_split_with_the_c_abi_ring():
    """ca_comm_init / ca_halo_exchange between real GPUs (world 2: both neighbours are the same peer)."""
    world = min(torch.cuda.device_count(), 4)
    with tempfile.TemporaryDirectory() as tmp:
        mp.spawn(_ring_worker, args=(world, tmp), nprocs=world, join=True)
        _check_parts(tmp, world)


def test_c_abi_ring_single_rank_wraps(ca):
    """world == 1 needs no NCCL: the halos are the band's own wrapped columns."""
    ring = ca.parallel.Ring(0, 1)
    try:
        rng = np.random.default_rng(3)
        x = ca.jl.from_numpy(randn(rng, (6, 9, 3, 2)))
        ext = ca.jl.to_numpy(ca.parallel.exchange_halos([x], 2, ring=ring)[0])
        xn = ca.jl.to_numpy(x)
        assert np.array_equal(ext, np.concatenate([xn[:, -2:], xn, xn[:, :2]], axis=1))
    finally:
        ring.close()
