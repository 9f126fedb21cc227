"""Host-side logic of the multi-GPU path on CPU ranks: shard plans (uneven
splits, more ranks than units), wrap neighbours, and the halo exchange itself
run as two gloo processes (no GPU involved; the tensors stand in for device
slabs)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def test_shard_units_plans(ca):
    su = ca.parallel.shard_units
    assert [su(128, 8, r) for r in range(8)] == [(16 * r, 16) for r in range(8)]
    assert [su(10, 4, r) for r in range(4)] == [(0, 3), (3, 3), (6, 2), (8, 2)]
    assert [su(2, 4, r) for r in range(4)] == [(0, 1), (1, 1), (2, 0), (2, 0)]      # more ranks than units
    for units, world in [(7, 3), (128, 5), (1, 1), (0, 2)]:
        parts = [su(units, world, r) for r in range(world)]
        assert sum(c for _, c in parts) == units
        assert all(parts[i][0] + parts[i][1] == parts[i + 1][0] for i in range(world - 1))
    with pytest.raises(ValueError):
        su(4, 2, 2)


def test_take_units_is_a_view(ca):
    x = ca.jl.randn(6, 5, 4, 8, device="cpu")
    s = ca.parallel.take_units(x, 4, 2)
    assert tuple(s.shape) == (6, 5, 4, 2) and s.data_ptr() == x[..., 4:].data_ptr()
    assert ca.jl.is_colmajor(s)


def test_band_plan(ca):
    plan = ca.parallel.BandPlan(1024, 8, 21)
    assert plan.p == 10 and plan.widths() == [128] * 8
    assert plan.neighbours(0) == (7, 1) and plan.neighbours(7) == (6, 0)           # circular wrap
    assert ca.parallel.BandPlan(100, 3, 7).widths() == [34, 33, 33]
    assert ca.parallel.BandPlan(96, 1, 15).neighbours(0) == (0, 0)
    with pytest.raises(ValueError, match="narrower than the halo"):
        ca.parallel.BandPlan(40, 8, 15)                                            # bands of 5 < halo 7
    with pytest.raises(AssertionError, match="must be odd"):
        ca.parallel.BandPlan(96, 2, 4)


def test_exchange_halo_single_rank_wraps(ca):
    x = ca.jl.from_numpy(np.asfortranarray(np.arange(5 * 6 * 2, dtype=np.float32).reshape((5, 6, 2), order="F")), "cpu")
    ext = ca.jl.to_numpy(ca.parallel.exchange_halo(x, 2))
    want = np.concatenate([ca.jl.to_numpy(x)[:, -2:], ca.jl.to_numpy(x), ca.jl.to_numpy(x)[:, :2]], axis=1)
    assert np.array_equal(ext, want)
    with pytest.raises(ValueError, match="cannot supply a halo"):
        ca.parallel.exchange_halo(x, 7)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, W, p, out):
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, root)
    from __graft_entry__ import load_package
    ca = load_package()
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        full = np.asfortranarray(np.arange(4 * W * 3 * 2, dtype=np.float32).reshape((4, W, 3, 2), order="F"))
        plan = ca.parallel.BandPlan(W, world, 2 * p + 1)
        start, width = plan.band(rank)
        band = ca.jl.from_numpy(np.asfortranarray(full[:, start:start + width]), "cpu")
        ext = ca.jl.to_numpy(ca.parallel.exchange_halo(band, p))
        cols = [(c % W) for c in range(start - p, start + width + p)]
        ok = np.array_equal(ext, full[:, cols])
        # several tensors of different trailing shapes in ONE exchange (one message per neighbour),
        # twice, so that the reused staging buffers are exercised
        full2 = np.asfortranarray(-np.arange(4 * W * 5, dtype=np.float32).reshape((4, W, 5), order="F"))
        band2 = ca.jl.from_numpy(np.asfortranarray(full2[:, start:start + width]), "cpu")
        for _ in range(2):
            e1, e2 = ca.parallel.exchange_halos([band, band2], p)
            ok = ok and np.array_equal(ca.jl.to_numpy(e1), full[:, cols]) and np.array_equal(ca.jl.to_numpy(e2), full2[:, cols])
        out[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,W,p", [(2, 12, 3), (2, 9, 2), (3, 15, 2)])
def test_exchange_halo_between_gloo_ranks(world, W, p):
    """Each rank's extended slab equals the circularly indexed full image (uneven bands,
    and world 2 where the left and right neighbour are the same rank)."""
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), W, p, out), nprocs=world, join=True)
    assert dict(out) == {r: True for r in range(world)}
