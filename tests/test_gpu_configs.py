"""The BASELINE configurations at (or near) their full sizes.

Config 2 runs at full size against the full oracle.  Configs 3 (1-D, entmax-1.5, Distance), 4
(ComplexF32, A materialised) and 5 (1024 x 1024, ws 21, Float32 and BFloat16 storage) run at
their full extents and are checked at sampled pixels: every end / corner / border / tile seam
plus random interior pixels, for y, dq, dk and dv and (config 4) the rows of A; each of those
values depends only on windows around the sampled pixel, which the oracle evaluates exactly.
Configs 3 and 4 also run at reduced extents against the full oracle (with the Circulant
algebra of config 4), and config 3 through size-independent properties."""
import numpy as np
import pytest
import torch

from oracle import circatt_oracle as orc
from tests.helpers import KIND, TOL, randn, rel_err, up


def _sampled_check(ca, kind, norm, q, k, v, r, outs, ws, nheads, pixels, units, tol, A=None):
    """outs = (y, dq, dk, dv) (and the rows of A) at `pixels` of `units` against the sampled-pixel oracle."""
    qs, ks, vs, rs = (orc.splitheads(up(ca.jl.to_numpy(t)), nheads) for t in (q, k, v, r))
    flat = lambda t: orc._flat(orc.splitheads(ca.jl.to_numpy(t).astype(np.complex128 if t.is_complex() else np.float64), nheads))[0]
    Y, DQ, DK, DV = (flat(t) for t in outs)
    nz = None
    if A is not None:
        nz = ca.jl.to_numpy(A.nzVal)
        nz = nz.reshape((-1, Y.shape[0], nz.size // nz.shape[0]), order="F")       # (K, Np, units)
    for unit in units:
        ys = orc.sampled_attention(kind, qs, ks, vs, ws, pixels, unit, norm)
        dq, dk, dv = orc.sampled_attention_pullback(kind, qs, ks, vs, rs, ws, pixels, unit, norm)
        for name, got, want in (("y", Y, ys), ("dq", DQ, dq), ("dk", DK, dk), ("dv", DV, dv)):
            err = np.abs(got[pixels, :, unit] - want).max() / max(1e-30, np.abs(want).max())
            assert err < tol, f"{name} unit {unit}: {err:.3g}"
        if nz is not None:
            wins, rows = orc.sampled_rows(kind, qs, ks, ws, pixels, unit, norm)
            for n, j in enumerate(pixels):
                order = np.argsort(wins[n], kind="stable")                           # CSR rows are sorted by column
                assert np.abs(nz[:, j, unit] - rows[n][order]).max() < tol * max(1e-30, rows[n].max())

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


def test_config5_eight_units_and_bfloat16(ca):
    """Config 5 with 8 units (one batch element, 128 channels, 8 heads) in Float32, and the same in
    BFloat16 storage (bar 1e-2 of the largest value, against the oracle on the rounded inputs)."""
    H = W = 1024
    ws, nheads, C = 21, 8, 128
    g = torch.Generator(device="cuda").manual_seed(55)
    base = [ca.jl.randn(H, W, C, 1, generator=g) for _ in range(4)]
    rng = np.random.default_rng(55)
    edge = [0, 9, 10, 127, 128, 1013, 1023]
    pixels = [h + H * w for h in edge[::2] for w in edge[1::2]] + [int(x) for x in rng.integers(0, H * W, 12)]
    for dtype, tol in ((torch.float32, TOL), (torch.bfloat16, 1e-2)):
        q, k, v, r = (t.detach().to(dtype) for t in base)
        q.requires_grad_(True); k.requires_grad_(True); v.requires_grad_(True)
        y, A = ca.circulant_mh_attention(ca.DotSimilarity(), q, k, v, ws, nheads, return_A=False)
        (y.float() * r.float()).sum().backward()
        torch.cuda.synchronize()
        f32 = lambda t: t.detach().float()
        _sampled_check(ca, orc.DOT, orc.SOFTMAX, f32(q), f32(k), f32(v), f32(r),
                       (f32(y), f32(q.grad), f32(k.grad), f32(v.grad)), ws, nheads, pixels, (0, 5, 7), tol)
        del q, k, v, r, y
        ca.ops.release_scratch()
        torch.cuda.empty_cache()


def test_config3_full_size_sampled(ca):
    """Config 3 at its full size: N = 16384, C = 64, B = 16, ws 127, 8 heads, Distance + entmax-1.5,
    forward + backward, checked at sampled pixels (both ends of the signal, fold seams, random)."""
    g = torch.Generator(device="cuda").manual_seed(33)
    q, k, v, r = (ca.jl.randn(16384, 64, 16, generator=g) for _ in range(4))
    q.requires_grad_(True); k.requires_grad_(True); v.requires_grad_(True)
    y, A = ca.circulant_mh_attention(ca.DistanceSimilarity(), q, k, v, 127, 8, normalizer=ca.ENTMAX15, return_A=False)
    (y * r).sum().backward()
    torch.cuda.synchronize()
    rng = np.random.default_rng(33)
    pixels = [0, 1, 62, 63, 64, 127, 128, 129, 8191, 8192, 16320, 16321, 16383] + [int(x) for x in rng.integers(0, 16384, 12)]
    _sampled_check(ca, orc.DISTANCE, orc.ENTMAX15, q.detach(), k.detach(), v.detach(), r, (y, q.grad, k.grad, v.grad),
                   127, 8, pixels, (0, 77, 127), 2 * TOL)


def test_config4_full_size_sampled(ca):
    """Config 4 at its full size: ComplexF32, H = W = 320, C = 32, B = 8, ws 7, one head, Dot, A
    materialised; y, the rows of A and the gradients at sampled pixels."""
    g = torch.Generator(device="cuda").manual_seed(44)
    q, k, v, r = (ca.jl.randn(320, 320, 32, 8, generator=g, dtype=torch.complex64) for _ in range(4))
    q.requires_grad_(True); k.requires_grad_(True); v.requires_grad_(True)
    y, A = ca.circulant_attention(ca.DotSimilarity(), q, k, v, 7)
    assert A.shape == (102400, 102400, 1, 8)
    (y * r.conj()).real.sum().backward()
    torch.cuda.synchronize()
    rng = np.random.default_rng(44)
    H = 320
    edge = [0, 2, 3, 31, 32, 316, 317, 319]
    pixels = [h + H * w for h in edge[::2] for w in edge[1::2]] + [int(x) for x in rng.integers(0, H * H, 16)]
    _sampled_check(ca, orc.DOT, orc.SOFTMAX, q.detach(), k.detach(), v.detach(), r, (y, q.grad, k.grad, v.grad),
                   7, 1, pixels, (0, 7), TOL, A=A)


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
