"""Circulant algebra, sums, cat and the scale rrule against the oracle
(src/array.jl:66-189, src/rrules.jl:97-114, README.md:121-148)."""
import numpy as np
import pytest
import torch

from oracle import circatt_oracle as orc
from tests.helpers import TOL, randn, rel_err

pytestmark = pytest.mark.gpu

SPATIAL, WS = (9, 8), 5
K, NP = 25, 72


def make(ca, rng, batch):
    A = ca.Circulant(WS, SPATIAL + batch)
    nzn = np.asfortranarray(rng.standard_normal(tuple(A.nzVal.shape)).astype(np.float32))
    A.data.nzVal = ca.jl.from_numpy(nzn)
    return A, nzn.astype(np.float64).reshape((K, NP) + batch, order="F")


def test_add_sub_scalar_neg_dot_eq(ca):
    rng = np.random.default_rng(0)
    A, a = make(ca, rng, (2, 3))
    B, b = make(ca, rng, (2, 3))
    assert np.array_equal(ca.jl.to_numpy((A + B).nzVal).reshape(a.shape, order="F"), (a + b).astype(np.float32))
    assert np.array_equal(ca.jl.to_numpy((A - B).nzVal).reshape(a.shape, order="F"), (a - b).astype(np.float32))
    assert np.array_equal(ca.jl.to_numpy((2.5 * A).nzVal).reshape(a.shape, order="F"), (2.5 * a).astype(np.float32))
    assert np.array_equal(ca.jl.to_numpy((-A).nzVal).reshape(a.shape, order="F"), (-a).astype(np.float32))
    assert abs(float(ca.dot(A, B)) - (a * b).sum()) < 1e-4 * np.abs(a * b).sum()
    assert A == A.copy() and not (A == B)
    assert A.data.colVal.data_ptr() == B.data.colVal.data_ptr()      # structure is shared, not copied


@pytest.mark.parametrize("abatch,cshape", [((2, 3), (1, 1, 2, 3)), ((1, 3), (1, 1, 2, 3)), ((2, 3), (1, 1, 1, 3)),
                                           ((2, 1), (1, 1, 2, 4)), ((1, 2), (1, 1, 2, 2)), ((2, 2), (1, 1, 1, 1))])
def test_scale_and_pullback(ca, abatch, cshape):
    """test/rrule.jl:22 and README.md:130-134 (`m*B`)."""
    rng = np.random.default_rng(1)
    A, a = make(ca, rng, abatch)
    A.data.nzVal.requires_grad_(True)
    cn = np.asfortranarray(rng.standard_normal(cshape).astype(np.float32))
    c = ca.jl.from_numpy(cn).requires_grad_(True)
    Bm = c * A
    want = orc.scale(cn.astype(np.float64), a)
    assert Bm.shape == (NP, NP) + want.shape[2:]
    assert rel_err(ca.jl.to_numpy(Bm.nzVal), want) < 1e-6
    dBn = np.asfortranarray(rng.standard_normal(tuple(Bm.nzVal.shape)).astype(np.float32))
    (Bm.nzVal * ca.jl.from_numpy(dBn)).sum().backward()
    dco, dAo = orc.scale_pullback(cn.astype(np.float64), a, dBn.astype(np.float64).reshape(want.shape, order="F"))
    assert rel_err(ca.jl.to_numpy(c.grad), dco) < TOL
    assert rel_err(ca.jl.to_numpy(A.nzVal.grad), dAo) < TOL


def test_scale_rejects_non_batch_dims(ca):
    rng = np.random.default_rng(2)
    A, _ = make(ca, rng, (1, 2))
    with pytest.raises(AssertionError, match="Scaling of non-batchdims"):
        ca.scale(ca.jl.ones((1, 2, 1, 2)), A)


def test_sums(ca):
    """README.md:137-143."""
    rng = np.random.default_rng(3)
    A, a = make(ca, rng, (2, 3))
    assert rel_err(ca.jl.to_numpy(ca.sum(A, dims=2)), orc.sum_dims2(a).reshape((NP, 1, 2, 3))) < TOL
    assert rel_err(ca.jl.to_numpy(ca.sum(A, dims=1)), orc.sum_dims1(a, SPATIAL, WS).reshape((1, NP, 2, 3))) < TOL
    s3 = ca.sum(A, dims=3)
    assert isinstance(s3, ca.Circulant) and s3.shape == (NP, NP, 1, 3)
    assert rel_err(ca.jl.to_numpy(s3.nzVal), orc.sum_batch(a, (3,))) < TOL
    s4 = ca.sum(A, dims=4)
    assert s4.shape == (NP, NP, 2, 1)
    assert rel_err(ca.jl.to_numpy(s4.nzVal), orc.sum_batch(a, (4,))) < TOL
    s34 = ca.sum(A, dims=(3, 4))
    assert s34.shape == (NP, NP, 1, 1)
    assert rel_err(ca.jl.to_numpy(s34.nzVal), orc.sum_batch(a, (3, 4))) < TOL
    s12 = ca.sum(A, dims=(1, 2))
    assert tuple(s12.shape) == (1, 1, 2, 3)
    assert rel_err(ca.jl.to_numpy(s12), a.sum(axis=(0, 1)).reshape((1, 1, 2, 3))) < TOL
    assert abs(float(ca.sum(A)) - a.sum()) < 1e-3
    with pytest.raises(RuntimeError, match="not implemented"):
        ca.sum(A, dims=(1, 3))


def test_cat_repeat_reshape(ca):
    """README.md:145-148."""
    rng = np.random.default_rng(4)
    A, a = make(ca, rng, (2, 3))
    B, b = make(ca, rng, (1, 3))
    D = ca.cat(A, B, dims=3)
    assert D.shape == (NP, NP, 3, 3)
    assert np.array_equal(ca.jl.to_numpy(D.nzVal).reshape((K, NP, 3, 3), order="F"),
                          np.concatenate([a, b], axis=2).astype(np.float32))
    R = B.repeat(1, 1, 2, 1)
    assert R.shape == (NP, NP, 2, 3)
    assert np.array_equal(ca.jl.to_numpy(R.nzVal).reshape((K, NP, 2, 3), order="F"),
                          np.repeat(b, 2, axis=2).astype(np.float32))
    F = A.reshape(NP, NP, -1)
    assert F.shape == (NP, NP, 6)
    assert np.array_equal(ca.jl.to_numpy(F.nzVal).reshape((K, NP, 6), order="F"),
                          a.reshape((K, NP, 6), order="F").astype(np.float32))


def test_grad_smoke_network(ca):
    """test/grad.jl:17-21,34-38: C = α*A + (1-α)*B, z = C ⨷ v, gradients for every input."""
    rng = np.random.default_rng(5)
    shape, ws, nheads = (10, 10, 8, 2), 3, 2
    for sim in (ca.DotSimilarity(), ca.DistanceSimilarity()):
        xx, k, q, v = (ca.jl.from_numpy(randn(rng, shape)).requires_grad_(True) for _ in range(4))
        alpha = (0.8 * ca.jl.ones((1, 1, nheads, 1))).requires_grad_(True)
        A = ca.circulant_mh_adjacency(sim, k, q, ws, nheads)
        B = ca.circulant_mh_adjacency(sim, xx, xx, ws, nheads)
        Cm = alpha * A + (1.0 - alpha) * B
        z = ca.Otimes(Cm, v)
        assert tuple(z.shape) == shape
        (z * z).sum().backward()
        for t in (xx, k, q, v, alpha):
            assert t.grad is not None and torch.isfinite(t.grad).all() and t.grad.abs().sum() > 0


def test_mix_otimes_equals_materialised_sum(ca):
    """test/grad.jl:17-21 pattern: (α*A + (1-α)*B) ⨷ x and its gradients, computed without the sum."""
    import torch
    rng = np.random.default_rng(31)
    shape, ws, nheads = (24, 20, 32, 2), 5, 2
    q1, k1, q2, k2, xn, rn = (randn(rng, shape) for _ in range(6))
    def build():
        ts = [ca.jl.from_numpy(t).requires_grad_(True) for t in (q1, k1, q2, k2, xn)]
        A = ca.circulant_mh_adjacency(ca.DotSimilarity(), ts[0], ts[1], ws, nheads)
        B = ca.circulant_mh_adjacency(ca.DistanceSimilarity(), ts[2], ts[3], ws, nheads)
        alpha = ca.jl.from_numpy(rng_alpha.copy()).requires_grad_(True)
        return ts, A, B, alpha
    rng_alpha = np.asfortranarray(np.random.default_rng(32).uniform(0.2, 0.8, (1, 1, nheads, 2)).astype(np.float32))
    r = ca.jl.from_numpy(rn)
    # materialised: C = α*A + (1-α)*B ; y = C ⨷ x
    ts, A, B, alpha = build()
    y_ref = ca.Otimes(ca.scale(alpha, A) + ca.scale(1 - alpha, B), ts[4])
    (y_ref * r).sum().backward()
    g_ref = [ca.jl.to_numpy(t.grad) for t in ts] + [ca.jl.to_numpy(alpha.grad)]
    # fused by linearity
    ts, A, B, alpha = build()
    y = ca.mix_otimes([(alpha, A), (1 - alpha, B)], ts[4])
    (y * r).sum().backward()
    g = [ca.jl.to_numpy(t.grad) for t in ts] + [ca.jl.to_numpy(alpha.grad)]
    assert rel_err(ca.jl.to_numpy(y), ca.jl.to_numpy(y_ref).astype(np.float64)) < TOL
    for a, b in zip(g, g_ref):
        assert rel_err(a, b.astype(np.float64)) < TOL


@pytest.mark.parametrize("mh", [False, True])
@pytest.mark.parametrize("simname", ["dot", "distance"])
def test_lazy_adjacency_mix_equals_materialised(ca, mh, simname):
    """The pattern of the reference's gradient test (test/grad.jl:17-21, 34-38): C = α*A + (1-α)*B, z = C ⨷ v.
    With lazy adjacencies nothing A-sized is ever written; z and every gradient equal the materialised path."""
    rng = np.random.default_rng(17)
    shape, W, nheads = (20, 18, 32, 2), 5, (2 if mh else 1)
    sim = ca.DotSimilarity() if simname == "dot" else ca.DistanceSimilarity()
    data = [randn(rng, shape, scale=0.5) for _ in range(4)]
    rn = randn(rng, shape)
    an = np.asfortranarray(np.array([0.8, 0.3], dtype=np.float32).reshape(1, 1, 1, 2))
    outs = []
    for lazy in (False, True):
        k, q, xx, v = (ca.jl.from_numpy(t).requires_grad_(True) for t in data)
        alpha = ca.jl.from_numpy(an).requires_grad_(True)
        before = ca.lib.ca_probe_launch_count()
        if mh:
            A = ca.circulant_mh_adjacency(sim, k, q, W, nheads, lazy=lazy)
            B = ca.circulant_mh_adjacency(sim, xx, xx, W, nheads, lazy=lazy)
            z = ca.Otimes(alpha * A + (1.0 - alpha) * B, v)
        else:
            A = ca.circulant_adjacency(sim, k, q, W, lazy=lazy)
            B = ca.circulant_adjacency(sim, xx, xx, W, lazy=lazy)
            z = ca.otimes(alpha * A + (1.0 - alpha) * B, v)
        (z * ca.jl.from_numpy(rn)).sum().backward()
        outs.append([ca.jl.to_numpy(t) for t in (z, k.grad, q.grad, xx.grad, v.grad, alpha.grad)])
        if lazy:
            assert isinstance(A, ca.LazyAdjacency) and A._cache is None and B._cache is None     # never materialised
    for name, a, b in zip(("z", "dk", "dq", "dxx", "dv", "dalpha"), *outs):
        assert rel_err(b, a.astype(np.float64)) < 5 * TOL, name


def test_lazy_adjacency_materialises_on_demand(ca):
    rng = np.random.default_rng(18)
    x, y = (ca.jl.from_numpy(randn(rng, (12, 10, 8, 2))) for _ in range(2))
    L = ca.circulant_mh_adjacency(ca.DotSimilarity(), x, y, 5, 2, lazy=True)
    A = ca.circulant_mh_adjacency(ca.DotSimilarity(), x, y, 5, 2)
    assert L.shape == tuple(A.shape)
    assert rel_err(ca.jl.to_numpy((2.0 * L).nzVal), 2.0 * ca.jl.to_numpy(A.nzVal).astype(np.float64)) < TOL
    assert np.abs(ca.jl.to_numpy(ca.sum(L, dims=2)) - 1.0).max() < 1e-5
    with pytest.raises(TypeError, match="materialize"):
        L + A
