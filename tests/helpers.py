import numpy as np

from oracle import circatt_oracle as orc

TOL = 1e-5   # relative to the largest magnitude of the tensor (FP32 / ComplexF32 parity bar)


def rel_err(got, want):
    want = np.asarray(want)
    got = np.asarray(got).reshape(want.shape, order="F")
    scale = np.abs(want).max()
    return float(np.abs(got - want).max() / (scale if scale > 0 else 1.0))


def randn(rng, shape, cplx=False, scale=1.0):
    x = rng.standard_normal(shape)
    if cplx:
        x = (x + 1j * rng.standard_normal(shape)) / np.sqrt(2.0)
        return np.asfortranarray((scale * x).astype(np.complex64))
    return np.asfortranarray((scale * x).astype(np.float32))


def up(x):
    """float32/complex64 input -> the float64/complex128 the oracle computes in."""
    return x.astype(np.complex128 if np.iscomplexobj(x) else np.float64)


KIND = {"dot": orc.DOT, "distance": orc.DISTANCE}
