"""The 2-D 1.5-entmax forward in flash mode: repeated sweeps of the tiled kernels (row maximum, threshold search,
apply) instead of the operator chain, so no A-sized memory.  Checked against the float64 oracle, on ordinary
rows and on rows that stress the threshold search, together with the size of the workspace it asks for."""
import numpy as np
import pytest
import torch

from oracle import circatt_oracle as orc
from tests.helpers import KIND, assert_close, randn, up

pytestmark = pytest.mark.gpu


@pytest.fixture
def sweeps_forced(ca):
    """The test shapes are small, so the operator chain would be chosen: lower the scratch limit to zero."""
    old = ca.lib.ca_entmax_scratch_limit(0)
    yield
    ca.lib.ca_entmax_scratch_limit(old)


@pytest.mark.parametrize("simname", ["dot", "distance"])
@pytest.mark.parametrize("shape,ws,nheads,cplx", [((40, 36, 32, 1), 7, 2, False),      # 16 channels per head
                                                  ((33, 29, 16, 2), 9, 2, False),      # 8 channels per head, ragged tiles
                                                  ((20, 21, 8, 1), 15, 1, True),       # 8 complex = 16 real channels
                                                  ((64, 48, 16, 1), 21, 1, False)])    # config 5's window
def test_entmax_flash_forward_matches_oracle(ca, sweeps_forced, shape, ws, nheads, cplx, simname):
    rng = np.random.default_rng(21)
    qn, kn, vn = (randn(rng, shape, cplx, scale=1.4) for _ in range(3))
    q, k, v = (ca.splitheads(ca.jl.from_numpy(t), nheads) for t in (qn, kn, vn))
    m = ca.ops.meta_of(q, ws)
    d = m.desc(similarity=KIND[simname], normalizer=ca.ENTMAX15, scale=1.0 / np.sqrt(m.channels))
    nbytes = ca.lib.ca_attention_fwd_workspace(d, 0)
    H, W = m.spatial
    # the packed (k|v) -- 144 bytes per pixel of the row-padded image -- and two scalar planes; nothing grows with K
    assert 0 < nbytes <= 144 * (H + ws + 16) * W * m.units + 8 * m.Np * m.units + 4096, nbytes
    n0 = ca.lib.ca_probe_tiled_launch_count()
    y, _, tau = ca.ops.attention_fwd(KIND[simname], ca.ENTMAX15, q, k, v, ws, False)
    assert ca.lib.ca_probe_tiled_launch_count() - n0 >= 4          # pack, maximum, steps, apply: the tiled sweeps ran
    yo, nzo = orc.mh_attention(KIND[simname], up(qn), up(kn), up(vn), ws, nheads, orc.ENTMAX15)
    assert (nzo == 0).any()
    assert_close(ca.jl.to_numpy(y), yo, "y")                       # the head split is a pure column-major reshape
    # tau reproduces the rows: sum_k max(s/2 - tau, 0)^2 == 1
    s = orc.similarity(KIND[simname], up(orc.splitheads(qn, nheads)), up(orc.splitheads(kn, nheads)), ws) / np.sqrt(m.channels)
    t = ca.jl.to_numpy(tau).astype(np.float64).reshape(s.shape[1:], order="F")
    assert np.allclose((np.maximum(s / 2 - t[None], 0.0) ** 2).sum(axis=0), 1.0, atol=2e-5)


@pytest.mark.parametrize("spread", [0.0, 1e-3, 25.0])
def test_entmax_flash_forward_threshold_extremes(ca, sweeps_forced, spread):
    """Flat rows (all 81 entries equal), nearly flat rows and rows with one dominant entry."""
    rng = np.random.default_rng(22)
    shape, ws = (36, 40, 16, 1), 9
    qn, kn, vn = (randn(rng, shape) for _ in range(3))
    if spread == 0.0:
        kn[:] = 0.0
    else:
        kn *= spread
    q, k, v = (ca.jl.from_numpy(np.asfortranarray(t)) for t in (qn, kn, vn))
    y, _, tau = ca.ops.attention_fwd(orc.DOT, ca.ENTMAX15, q, k, v, ws, False)
    yo, nzo = orc.mh_attention(orc.DOT, up(qn), up(kn), up(vn), ws, 1, orc.ENTMAX15)
    assert_close(ca.jl.to_numpy(y), yo, "y")
    assert torch.isfinite(tau).all()


def test_entmax_route_follows_the_scratch_limit(ca):
    """Default limit: a small problem takes the chain (A-sized scratch), a large one the sweeps; the workspace
    query and the call agree."""
    x = ca.jl.randn(64, 64, 16, 2)
    m = ca.ops.meta_of(x, 9)
    d = m.desc(similarity=orc.DOT, normalizer=ca.ENTMAX15, scale=0.25)
    a_bytes = 4 * m.Np * m.K * m.units
    assert ca.lib.ca_entmax_scratch_limit(-1) == 256 << 20
    assert ca.lib.ca_attention_fwd_workspace(d, 0) >= a_bytes            # chain
    old = ca.lib.ca_entmax_scratch_limit(a_bytes - 1)
    try:
        assert ca.lib.ca_attention_fwd_workspace(d, 0) < a_bytes         # sweeps
        n0 = ca.lib.ca_probe_tiled_launch_count()
        y1, _, t1 = ca.ops.attention_fwd(orc.DOT, ca.ENTMAX15, x, x, x, 9, False)
        assert ca.lib.ca_probe_tiled_launch_count() - n0 >= 4
    finally:
        ca.lib.ca_entmax_scratch_limit(old)
    y0, _, t0 = ca.ops.attention_fwd(orc.DOT, ca.ENTMAX15, x, x, x, 9, False)
    assert float((y0 - y1).abs().max()) < 1e-5 and float((t0 - t1).abs().max()) < 1e-5
