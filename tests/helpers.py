import numpy as np

from oracle import circatt_oracle as orc

TOL = 1e-5        # max-norm bar: largest |error| relative to the largest magnitude of the tensor
ELEM_TOL = 2e-5   # element-wise bar: |error_i| <= ELEM_TOL * (|want_i| + rms(want)) for every element i


def rel_err(got, want):
    """Max-norm relative error: max_i |got_i - want_i| / max_i |want_i|."""
    want = np.asarray(want)
    got = np.asarray(got).reshape(want.shape, order="F")
    scale = np.abs(want).max()
    return float(np.abs(got - want).max() / (scale if scale > 0 else 1.0))


def elem_err(got, want):
    """Element-wise relative error with an absolute floor: max_i |got_i - want_i| / (|want_i| + rms(want)).
    Every output here is a sum of K window terms of mixed sign, so a Float32 result cannot be
    relatively accurate where the exact value cancels to (almost) zero; the floor is the tensor's
    root-mean-square, i.e. the size of a typical element, not of the largest one."""
    want = np.asarray(want)
    got = np.asarray(got).reshape(want.shape, order="F")
    floor = float(np.sqrt(np.mean(np.abs(want) ** 2)))
    return float((np.abs(got - want) / (np.abs(want) + (floor if floor > 0 else 1.0))).max())


def assert_close(got, want, what="", tol=TOL, elem_tol=ELEM_TOL):
    """Both bars at once; the message carries both numbers."""
    r, e = rel_err(got, want), elem_err(got, want)
    assert r < tol and e < elem_tol, f"{what}: max-norm relative error {r:.3g} (bar {tol:g}), element-wise {e:.3g} (bar {elem_tol:g})"
    return r, e


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
