"""The BASELINE configurations at (or near) their full sizes.

Config 2 runs at full size against the full oracle.  Config 5 (1024 x 1024, ws 21, 16 channels
per head) runs at full spatial size with fewer units and is checked at sampled pixels: every
corner, border and tile seam plus random interior pixels, for y, dq, dk and dv (each value
depends only on windows around the sampled pixel).  Config 3 (1-D, entmax-1.5, Distance) and
config 4 (ComplexF32 + Circulant algebra) run at reduced extents against the full oracle, and
at larger extents through size-independent properties."""
import numpy as np
import pytest
import torch

from oracle import circatt_oracle as orc
from tests.helpers import KIND, TOL, randn, rel_err, up

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("simname", ["dot", "distance"])
def test_config2_full_size(ca, simname):
    """H,W,C,B = 128,96,64,2, ws 15, 4 heads: y, A, gradients of sum(r*y)."""
    rng = np.random.default_rng(0)
    shape, ws, nheads = (128, 96, 64, 2), 15, 4
    qn, kn, vn, rn = (randn(rng, shape) for _ in range(4))
    q, k, v = (ca.jl.from_numpy(t).requires_grad_(True) for t in (qn, kn, vn))
    sim = ca.DotSimilarity() if simname == "dot" else ca.DistanceSimilarity()
    y, A = ca.circulant_mh_attention(sim, q, k, v, ws, nheads)
    assert A.shape == (12288, 12288, 4, 2) and A.data.nnz == 12288 * 225 * 8
    (y * ca.jl.from_numpy(rn)).sum().backward()
    yo, nzo = orc.mh_attention(KIND[simname], up(qn), up(kn), up(vn), ws, nheads)
    dqo, dko, dvo = orc.mh_attention_pullback(KIND[simname], up(qn), up(kn), up(vn), ws, nheads, up(rn))
    assert rel_err(ca.jl.to_numpy(y), yo) < TOL
    assert rel_err(ca.jl.to_numpy(A.nzVal), nzo) < TOL
    assert rel_err(ca.jl.to_numpy(q.grad), dqo) < TOL
    assert rel_err(ca.jl.to_numpy(k.grad), dko) < TOL
    assert rel_err(ca.jl.to_numpy(v.grad), dvo) < TOL
    rows = ca.jl.to_numpy(ca.sum(A, dims=2))
    assert np.abs(rows - 1.0).max() < 1e-5                       # rows of a softmax sum to one


def test_config5_spatial_size_sampled(ca):
    """1024 x 1024, ws 21, 16 channels per head, flash mode; 2 heads x 1 batch of the 128 units."""
    H = W = 1024
    ws, nheads, C = 21, 2, 32
    g = torch.Generator(device="cuda").manual_seed(5)
    q, k, v, r = (ca.jl.randn(H, W, C, 1, generator=g) for _ in range(4))
    q.requires_grad_(True); k.requires_grad_(True); v.requires_grad_(True)
    y, A = ca.circulant_mh_attention(ca.DotSimilarity(), q, k, v, ws, nheads, return_A=False)
    assert A is None
    (y * r).sum().backward()
    torch.cuda.synchronize()
    rng = np.random.default_rng(5)
    edge = [0, 1, 9, 10, 11, 127, 128, 129, 511, 512, 1012, 1013, 1014, 1023]      # corners, halo width, tile seams
    pixels = [h + H * w for h in edge[::2] for w in edge[1::2]] + list(rng.integers(0, H * W, 40))
    qs, ks, vs, rs = (orc.splitheads(up(ca.jl.to_numpy(t)), nheads) for t in (q, k, v, r))
    flat = lambda t: orc._flat(orc.splitheads(ca.jl.to_numpy(t), nheads))[0]
    Y, DQ, DK, DV = flat(y), flat(q.grad), flat(k.grad), flat(v.grad)
    for unit in (0, 1):
        ys = orc.sampled_attention(orc.DOT, qs, ks, vs, ws, pixels, unit)
        dq, dk, dv = orc.sampled_attention_pullback(orc.DOT, qs, ks, vs, rs, ws, pixels, unit)
        for got, want in ((Y, ys), (DQ, dq), (DK, dk), (DV, dv)):
            assert np.abs(got[pixels, :, unit] - want).max() < TOL * max(1.0, np.abs(want).max())


def test_config3_1d_entmax_distance(ca):
    """1-D, ws 127, 8 heads of 8 channels, Distance + entmax-1.5, forward + backward (N reduced to 1024)."""
    rng = np.random.default_rng(3)
    shape, ws, nheads = (1024, 64, 2), 127, 8
    qn, kn, vn, rn = (randn(rng, shape) for _ in range(4))
    q, k, v = (ca.jl.from_numpy(t).requires_grad_(True) for t in (qn, kn, vn))
    y, A = ca.circulant_mh_attention(ca.DistanceSimilarity(), q, k, v, ws, nheads, normalizer=ca.ENTMAX15)
    (y * ca.jl.from_numpy(rn)).sum().backward()
    yo, nzo = orc.mh_attention(orc.DISTANCE, up(qn), up(kn), up(vn), ws, nheads, orc.ENTMAX15)
    dqo, dko, dvo = orc.mh_attention_pullback(orc.DISTANCE, up(qn), up(kn), up(vn), ws, nheads, up(rn), norm=orc.ENTMAX15)
    assert rel_err(ca.jl.to_numpy(y), yo) < TOL
    assert rel_err(ca.jl.to_numpy(A.nzVal), nzo) < TOL
    assert (ca.jl.to_numpy(A.nzVal) == 0).mean() > 0.2          # entmax is sparse
    assert rel_err(ca.jl.to_numpy(q.grad), dqo) < 2 * TOL
    assert rel_err(ca.jl.to_numpy(k.grad), dko) < 2 * TOL
    assert rel_err(ca.jl.to_numpy(v.grad), dvo) < TOL


def test_config3_full_length_properties(ca):
    """N = 16384, B reduced to 2: every row of the entmax A sums to one; A (x) v == y."""
    g = torch.Generator(device="cuda").manual_seed(3)
    q, k, v = (ca.jl.randn(16384, 64, 2, generator=g) for _ in range(3))
    y, A = ca.circulant_mh_attention(ca.DistanceSimilarity(), q, k, v, 127, 8, normalizer=ca.ENTMAX15)
    assert A.shape == (16384, 16384, 8, 2)
    rows = ca.sum(A, dims=2)
    assert float((rows - 1).abs().max()) < 2e-5
    u = ca.Otimes(A, v)
    assert float((u - y).abs().max()) < 1e-5 * float(y.abs().max()) + 1e-6


def test_config4_complex_with_algebra(ca):
    """ComplexF32, ws 7, single head, Dot: C = A + m*A2, C (x) u, sum(C; dims=2), with gradients
    (extents reduced to 40 x 36 x 32 channels x 2)."""
    rng = np.random.default_rng(4)
    shape, ws = (40, 36, 32, 2), 7
    qn, kn, vn, q2n, k2n, un, rn = (randn(rng, shape, True) for _ in range(7))
    mn = np.asfortranarray(rng.standard_normal((1, 1, 1, 2)).astype(np.float32))
    q, k, v, q2, k2, u = (ca.jl.from_numpy(t).requires_grad_(True) for t in (qn, kn, vn, q2n, k2n, un))
    m = ca.jl.from_numpy(mn).requires_grad_(True)
    y, A = ca.circulant_attention(ca.DotSimilarity(), q, k, v, ws)
    _, A2 = ca.circulant_attention(ca.DotSimilarity(), q2, k2, v, ws)
    Cm = A + m * A2
    w = ca.Otimes(Cm, u)
    rows = ca.sum(Cm, dims=2)
    loss = (w * ca.jl.from_numpy(rn).conj()).real.sum() + (y.conj() * y).real.sum()
    loss.backward()
    # oracle
    yo, P1 = orc.attention(orc.DOT, up(qn), up(kn), up(vn), ws)
    _, P2 = orc.attention(orc.DOT, up(q2n), up(k2n), up(vn), ws)
    Co = P1 + mn.astype(np.float64).reshape(1, 1, 2) * P2
    wo = orc.apply(Co, up(un), ws)
    assert rel_err(ca.jl.to_numpy(y), yo) < TOL
    assert rel_err(ca.jl.to_numpy(Cm.nzVal), Co) < TOL
    assert rel_err(ca.jl.to_numpy(w), wo) < TOL
    assert rel_err(ca.jl.to_numpy(rows), Co.sum(0)) < TOL
    # gradients of the algebra + apply chain: dC = similarity(dw, u), dm = sum(dC * A2), du = C^T dw
    dCo, duo = orc.apply_pullback(Co, up(un), ws, up(rn))
    dmo = (dCo * P2).sum(axis=(0, 1))
    assert rel_err(ca.jl.to_numpy(u.grad), duo) < TOL
    assert rel_err(ca.jl.to_numpy(m.grad).reshape(-1), dmo) < 5 * TOL
    dq2o, dk2o, _ = orc.attention_pullback(orc.DOT, up(q2n), up(k2n), up(vn), ws, np.zeros_like(up(vn)),
                                           dA=mn.astype(np.float64).reshape(1, 1, 2) * dCo)
    assert rel_err(ca.jl.to_numpy(q2.grad), dq2o) < 5 * TOL
    assert rel_err(ca.jl.to_numpy(k2.grad), dk2o) < 5 * TOL
    for t in (q, k, v):
        assert t.grad is not None and torch.isfinite(torch.view_as_real(t.grad)).all()
