"""The 1-D (sliding register tile) kernels against the float64 oracle: forward and backward, softmax and
1.5-entmax, Dot and Distance, real and complex, lengths that are no multiple of the block's pixel count,
windows as long as the signal, channel counts that are zero-extended, and that they are the path that ran."""
import numpy as np
import pytest
import torch

from oracle import circatt_oracle as orc
from tests.helpers import KIND, TOL, assert_close, randn, up

pytestmark = pytest.mark.gpu


def sim_of(ca, name):
    return ca.DotSimilarity() if name == "dot" else ca.DistanceSimilarity()


CASES = [
    # (Julia shape (N, C, B), ws, heads, complex)
    ((700, 16, 2), 31, 2, False),        # 8 channels per head, N no multiple of 512
    ((130, 8, 1), 127, 1, False),        # the window almost as long as the signal: every block wraps
    ((127, 8, 1), 127, 1, False),        # window == signal
    ((1500, 32, 1), 9, 2, False),        # 16 channels per head, three blocks, ragged tail
    ((600, 12, 2), 15, 2, False),        # 6 channels per head (zero-extended to 8)
    ((520, 8, 2), 21, 2, True),          # ComplexF32: 4 complex = 8 real channels per head
    ((300, 3, 1), 5, 1, False),          # 3 channels, the shortest window the kernels take
    ((900, 8, 1), 255, 1, False),        # a long window: more than 48 KB of shared memory per block
]


@pytest.mark.parametrize("norm", ["softmax", "entmax"])
@pytest.mark.parametrize("simname", ["dot", "distance"])
@pytest.mark.parametrize("shape,ws,nheads,cplx", CASES)
def test_line_kernels_match_oracle(ca, shape, ws, nheads, cplx, simname, norm):
    rng = np.random.default_rng(11)
    qn, kn, vn, rn = (randn(rng, shape, cplx, scale=1.3) for _ in range(4))
    q, k, v = (ca.jl.from_numpy(t).requires_grad_(True) for t in (qn, kn, vn))
    nrm, onorm = (ca.SOFTMAX, orc.SOFTMAX) if norm == "softmax" else (ca.ENTMAX15, orc.ENTMAX15)
    before = ca._lib.lib.ca_probe_tiled_launch_count()
    y, _ = ca.circulant_mh_attention(sim_of(ca, simname), q, k, v, ws, nheads, normalizer=nrm, return_A=False)
    loss = (y * ca.jl.from_numpy(rn).conj()).real.sum() if cplx else (y * ca.jl.from_numpy(rn)).sum()
    loss.backward()
    assert ca._lib.lib.ca_probe_tiled_launch_count() - before == 3          # forward, dq, dk/dv: nothing else ran
    yo, nzo = orc.mh_attention(KIND[simname], up(qn), up(kn), up(vn), ws, nheads, onorm)
    dqo, dko, dvo = orc.mh_attention_pullback(KIND[simname], up(qn), up(kn), up(vn), ws, nheads, up(rn), norm=onorm)
    if norm == "entmax" and ws >= 15:
        assert (nzo == 0).any()                           # the threshold is active
    assert_close(ca.jl.to_numpy(y), yo, "y")
    assert_close(ca.jl.to_numpy(q.grad), dqo, "dq", tol=2 * TOL, elem_tol=4e-5)
    assert_close(ca.jl.to_numpy(k.grad), dko, "dk", tol=2 * TOL, elem_tol=4e-5)
    assert_close(ca.jl.to_numpy(v.grad), dvo, "dv")


@pytest.mark.parametrize("spread", [0.0, 1e-3, 30.0])
def test_line_entmax_threshold_extremes(ca, spread):
    """Flat rows (every score equal: all 63 entries carry 1/63), nearly flat rows, and rows with one
    dominant entry: the support iteration must end in all of them."""
    rng = np.random.default_rng(12)
    shape, ws = (640, 8, 1), 63
    qn, kn, vn = (randn(rng, shape, scale=1.0) for _ in range(3))
    if spread == 0.0:
        kn[:] = 0.0                                     # Dot scores all zero
    else:
        kn *= spread
    q, k, v = (ca.jl.from_numpy(np.asfortranarray(t)) for t in (qn, kn, vn))
    y, _, tau = ca.ops.attention_fwd(orc.DOT, ca.ENTMAX15, q, k, v, ws, False)
    yo, nzo = orc.mh_attention(orc.DOT, up(qn), up(kn), up(vn), ws, 1, orc.ENTMAX15)
    assert np.allclose(nzo.sum(axis=0), 1.0)
    assert_close(ca.jl.to_numpy(y), yo, "y")
    assert torch.isfinite(tau).all()


def test_line_forward_needs_no_workspace(ca):
    """Flash mode on a 1-D signal: no scratch memory at all, entmax included (the operator chain needs an
    A-sized buffer)."""
    x = ca.jl.randn(4096, 8, 4)
    m = ca.ops.meta_of(x, 127)
    for nrm in (ca.SOFTMAX, ca.ENTMAX15):
        d = m.desc(similarity=orc.DISTANCE, normalizer=nrm, scale=0.3)
        assert ca.ops.lib.ca_attention_fwd_workspace(d, 0) == 0


def _random_cases(n, seed):
    rng = np.random.default_rng(seed)
    cases = []
    for _ in range(n):
        ws = int(rng.choice([5, 7, 9, 13, 21, 33, 63, 127]))
        N = int(rng.integers(ws, 4 * ws + 1200))
        cplx = bool(rng.integers(0, 2))
        cper = int(rng.integers(1, 9 if cplx else 17))          # channels per head: up to 16 real
        heads = int(rng.integers(1, 4))
        cases.append(((N, cper * heads, int(rng.integers(1, 3))), ws, heads, cplx,
                      ["dot", "distance"][int(rng.integers(0, 2))], ["softmax", "entmax"][int(rng.integers(0, 2))]))
    return cases


@pytest.mark.parametrize("shape,ws,nheads,cplx,simname,norm", _random_cases(14, 2024))
def test_line_kernels_random_shapes(ca, shape, ws, nheads, cplx, simname, norm):
    """Seeded random lengths, windows, channel counts (zero-extended to 8 or 16), heads, similarity and normaliser:
    block tails, wraps shorter and longer than a block, every template instantiation."""
    rng = np.random.default_rng(hash((shape, ws, nheads)) % (2 ** 32))
    qn, kn, vn, rn = (randn(rng, shape, cplx, scale=1.2) for _ in range(4))
    q, k, v = (ca.jl.from_numpy(t).requires_grad_(True) for t in (qn, kn, vn))
    nrm, onorm = (ca.SOFTMAX, orc.SOFTMAX) if norm == "softmax" else (ca.ENTMAX15, orc.ENTMAX15)
    before = ca._lib.lib.ca_probe_tiled_launch_count()
    y, _ = ca.circulant_mh_attention(sim_of(ca, simname), q, k, v, ws, nheads, normalizer=nrm, return_A=False)
    loss = (y * ca.jl.from_numpy(rn).conj()).real.sum() if cplx else (y * ca.jl.from_numpy(rn)).sum()
    loss.backward()
    assert ca._lib.lib.ca_probe_tiled_launch_count() - before == 3
    yo, _ = orc.mh_attention(KIND[simname], up(qn), up(kn), up(vn), ws, nheads, onorm)
    dqo, dko, dvo = orc.mh_attention_pullback(KIND[simname], up(qn), up(kn), up(vn), ws, nheads, up(rn), norm=onorm)
    assert_close(ca.jl.to_numpy(y), yo, "y")
    assert_close(ca.jl.to_numpy(q.grad), dqo, "dq", tol=2 * TOL, elem_tol=4e-5)
    assert_close(ca.jl.to_numpy(k.grad), dko, "dk", tol=2 * TOL, elem_tol=4e-5)
    assert_close(ca.jl.to_numpy(v.grad), dvo, "dv")
