"""The C + OpenMP restatement (timed CPU baseline) against the float64 numpy oracle."""
import numpy as np
import pytest

from oracle import circatt_oracle as orc
from oracle import cpu_baseline as cpu


@pytest.mark.parametrize("dist", [False, True])
@pytest.mark.parametrize("shape,ws,nheads", [((16, 4, 3), 7, 2), ((12, 9, 6, 2), 5, 3), ((7, 7, 4, 1), 7, 1)])
def test_c_oracle_matches_numpy_oracle(shape, ws, nheads, dist):
    rng = np.random.default_rng(11)
    q, k, v, dy = (np.asfortranarray(rng.standard_normal(shape)) for _ in range(4))
    kind = orc.DISTANCE if dist else orc.DOT
    yo, _ = orc.mh_attention(kind, q, k, v, ws, nheads)
    dqo, dko, dvo = orc.mh_attention_pullback(kind, q, k, v, ws, nheads, dy)
    qr, kr, vr, dyr = (orc.splitheads(t, nheads) for t in (q, k, v, dy))
    for dtype, tol in ((np.float64, 1e-12), (np.float32, 2e-5)):
        y, lse = cpu.attention_fwd(qr, kr, vr, ws, dist, dtype)
        dq, dk, dv = cpu.attention_bwd(qr, kr, vr, y, dyr, lse, ws, dist, dtype)
        for got, want in ((y, yo), (dq, dqo), (dk, dko), (dv, dvo)):
            got = got.reshape(shape, order="F")
            assert np.abs(got - want).max() <= tol * np.abs(want).max()


def test_c_oracle_reports_threads():
    assert cpu.threads() >= 1
