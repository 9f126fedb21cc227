"""Band mode of the kernels (spatial split along W with neighbour halos), checked on
one GPU by emulating the ranks: each band gets its halo columns sliced from the
circularly indexed full image, exactly what `exchange_halo` delivers between ranks."""
import numpy as np
import pytest
import torch

from oracle import circatt_oracle as orc
from tests.helpers import KIND, TOL, randn, rel_err, up

pytestmark = pytest.mark.gpu


def ext_cols(x, start, width, p):
    W = x.shape[1]
    cols = [(c % W) for c in range(start - p, start + width + p)]
    return np.asfortranarray(x[:, cols])


@pytest.mark.parametrize("simname", ["dot", "distance"])
@pytest.mark.parametrize("shape,ws,nheads,world", [((40, 36, 32, 1), 7, 2, 3),     # tiled kernels (16 ch/head)
                                                   ((24, 30, 12, 2), 5, 2, 2),     # generic kernels
                                                   ((33, 28, 16, 1), 9, 1, 2),
                                                   ((32, 24, 16, 1), 15, 1, 3),    # bands of 8 columns: halo 7 <= band < window 15
                                                   ((24, 18, 6, 1), 9, 1, 3)])     # the same on the generic kernels (bands of 6, halo 4)
def test_band_split_equals_full_circular_attention(ca, shape, ws, nheads, world, simname):
    rng = np.random.default_rng(0)
    p = ws // 2
    qn, kn, vn, rn = (randn(rng, shape) for _ in range(4))
    kind = KIND[simname]
    yo, _ = orc.mh_attention(kind, up(qn), up(kn), up(vn), ws, nheads)
    dqo, dko, dvo = orc.mh_attention_pullback(kind, up(qn), up(kn), up(vn), ws, nheads, up(rn))
    qs, ks, vs, rs = (orc.splitheads(t, nheads) for t in (qn, kn, vn, rn))          # (H, W, c, units)
    plan = ca.parallel.BandPlan(shape[1], world, ws)
    outs = {n: [] for n in ("y", "dq", "dk", "dv")}
    ops, jl = ca.ops, ca.jl
    for rank in range(world):
        start, width = plan.band(rank)
        band = lambda t: jl.from_numpy(np.asfortranarray(t[:, start:start + width]))
        ext = lambda t: jl.from_numpy(ext_cols(t, start, width, p))
        q, k, v, dy = band(qs), band(ks), band(vs), band(rs)
        k_ext, v_ext = ext(ks), ext(vs)
        y, _, stats = ops.attention_fwd(kind, 0, q, k_ext, v_ext, ws, False, band=(width + 2 * p, p))
        D = ops.attention_bwd_pre(kind, 0, q, k, v, y, dy, stats, ws)
        dq = ops.attention_bwd_dq(kind, 0, q, k_ext, v_ext, dy, stats, D, ws, band=(width + 2 * p, p))
        outs["y"].append(jl.to_numpy(y)); outs["dq"].append(jl.to_numpy(dq))
        outs.setdefault("stats", []).append(jl.to_numpy(stats).reshape((shape[0], width, -1), order="F"))
        outs.setdefault("D", []).append(jl.to_numpy(D).reshape((shape[0], width, -1), order="F"))
    stats_full = np.concatenate(outs["stats"], axis=1)
    D_full = np.concatenate(outs["D"], axis=1)
    for rank in range(world):
        start, width = plan.band(rank)
        band = lambda t: jl.from_numpy(np.asfortranarray(t[:, start:start + width]))
        ext = lambda t: jl.from_numpy(ext_cols(t, start, width, p))
        flat = lambda t: jl.from_numpy(np.asfortranarray(ext_cols(t, start, width, p).reshape((-1, t.shape[-1]), order="F")))
        dk, dv = ops.attention_bwd_dkdv(kind, 0, ext(qs), band(ks), band(vs), ext(rs), flat(stats_full), flat(D_full),
                                        ws, band=(width + 2 * p, p))
        outs["dk"].append(jl.to_numpy(dk)); outs["dv"].append(jl.to_numpy(dv))
    cat = lambda name: np.concatenate(outs[name], axis=1).reshape(shape, order="F")
    assert rel_err(cat("y"), yo) < TOL
    assert rel_err(cat("dq"), dqo) < TOL
    assert rel_err(cat("dk"), dko) < TOL
    assert rel_err(cat("dv"), dvo) < TOL


def test_band_driver_single_rank(ca):
    """`band_attention_fwd/bwd` with no process group: the band is the whole image."""
    rng = np.random.default_rng(1)
    shape, ws, nheads = (32, 20, 32, 1), 7, 2
    qn, kn, vn, rn = (randn(rng, shape) for _ in range(4))
    q, k, v, dy = (ca.splitheads(ca.jl.from_numpy(t), nheads) for t in (qn, kn, vn, rn))
    y, stats, k_ext, v_ext = ca.parallel.band_attention_fwd(0, q, k, v, ws)
    dq, dk, dv = ca.parallel.band_attention_bwd(0, q, k, v, y, dy, stats, k_ext, v_ext, ws)
    yo, _ = orc.mh_attention(orc.DOT, up(qn), up(kn), up(vn), ws, nheads)
    dqo, dko, dvo = orc.mh_attention_pullback(orc.DOT, up(qn), up(kn), up(vn), ws, nheads, up(rn))
    for got, want in ((y, yo), (dq, dqo), (dk, dko), (dv, dvo)):
        assert rel_err(ca.jl.to_numpy(got), want) < TOL


@pytest.mark.parametrize("dtype,H", [(torch.float32, 64), (torch.float32, 37), (torch.bfloat16, 33), (torch.uint8, 13)])
def test_copy_chunks_gathers_strided_columns(ca, dtype, H):
    """ca_copy_chunks: several strided copies in one launch (16-byte, 4-byte and byte paths), checked against
    torch slicing: the halo columns of two tensors gathered into one message, and a band copied into its slab."""
    torch.manual_seed(0)
    W, p, outer = 24, 3, 5
    mk = lambda *shape: (torch.randn(*shape, device="cuda") * 50).to(dtype)
    a, b = mk(outer, W, H), mk(2 * outer, W, H)                   # C-order views of (H, W, outer) tensors
    es = a.element_size()
    col = H * es
    msg = torch.zeros((outer + 2 * outer) * p * H, dtype=dtype, device="cuda")
    ext = torch.zeros(outer, W + 2 * p, H, dtype=dtype, device="cuda")
    jobs = [
        (a.data_ptr() + (W - p) * col, msg.data_ptr(), p * col, outer, W * col, p * col),
        (b.data_ptr() + (W - p) * col, msg.data_ptr() + outer * p * col, p * col, 2 * outer, W * col, p * col),
        (a.data_ptr(), ext.data_ptr() + p * col, W * col, outer, W * col, (W + 2 * p) * col),
    ]
    ca.ops.copy_chunks(jobs)
    torch.cuda.synchronize()
    want = torch.cat([a[:, W - p:, :].reshape(-1), b[:, W - p:, :].reshape(-1)])
    assert torch.equal(msg.view(torch.uint8), want.contiguous().view(torch.uint8))
    assert torch.equal(ext[:, p:p + W, :].contiguous().view(torch.uint8), a.view(torch.uint8))
    assert float(ext[:, :p, :].float().abs().max()) == 0.0 and float(ext[:, p + W:, :].float().abs().max()) == 0.0
    with pytest.raises(RuntimeError, match="njobs"):
        ca.ops.lib.ca_copy_chunks(None, 33, None) and None or ca.ops.check(ca.ops.lib.ca_copy_chunks(None, 33, None))
