"""Pins the CPU oracle: structure against the literal restatement of the
reference's index function, values against a dense masked formulation, and
pullbacks against central finite differences at the shapes of the reference's
test/rrule.jl:1-23 (size 8 or 8x8, 4 channels, batch 2, ws 5)."""
import numpy as np
import pytest

from oracle import circatt_oracle as orc


def randn(rng, shape, cplx=False):
    x = rng.standard_normal(shape)
    if cplx:
        x = (x + 1j * rng.standard_normal(shape)) / np.sqrt(2.0)
    return np.asfortranarray(x)


# ---------------------------------------------------------------- structure
@pytest.mark.parametrize("spatial,ws", [
    ((8,), 5), ((5,), 5), ((6,), 5), ((12,), 3), ((31,), 9), ((16,), 7),
    ((8, 8), 5), ((5, 5), 5), ((7, 9), 5), ((9, 7), 7), ((10, 10), 3), ((12, 6), 5), ((16, 11), 9),
])
def test_structure_matches_literal_index_function(spatial, ws):
    _, colval = orc.structure(spatial, ws)
    lit = orc.structure_literal(spatial, ws)
    assert np.array_equal(colval, lit)


def test_structure_rowptr_and_sortedness():
    rowptr, colval = orc.structure((12, 9), 5)
    K, Np = 25, 108
    assert rowptr.dtype == np.int32 and colval.dtype == np.int32
    assert np.array_equal(rowptr, 1 + K * np.arange(Np + 1))
    rows = colval.reshape(Np, K)
    assert np.all(np.diff(rows, axis=1) > 0)            # strictly ascending: sorted, no duplicates
    assert rows.min() == 1 and rows.max() == Np


def test_structure_position_formula():
    """Closed-form position of offset (dh, dw) inside a row, used by the CUDA kernels."""
    for (H, W, ws) in [(8, 8, 5), (7, 11, 7), (5, 9, 5), (9, 1, 5)]:
        p = ws // 2
        spatial = (H,) if W == 1 else (H, W)
        cols, offs = orc.window_columns(spatial, ws)

        def pos(d, x, X):
            if x < p:
                return (d + x) % ws
            if x >= X - p:
                return (d + x - X) % ws
            return d + p
        for pix in range(H * W):
            h, w = pix % H, pix // H
            for dw in (range(-p, p + 1) if W > 1 else [0]):
                for dh in range(-p, p + 1):
                    k = (pos(dw, w, W) * ws if W > 1 else 0) + pos(dh, h, H)
                    col = (h + dh) % H + H * ((w + dw) % W)
                    assert cols[k, pix] == col
                    off = ((dw + p) * ws if W > 1 else 0) + dh + p
                    assert offs[k, pix] == off


def test_even_window_rejected():
    with pytest.raises(ValueError, match="must be odd"):
        orc.window_columns((8, 8), 4)


# ---------------------------------------------------------------- forward values vs dense
def dense_attention(kind, q, k, v, ws):
    Q, spatial = orc._flat(q)
    Kk, _ = orc._flat(k)
    V, _ = orc._flat(v)
    Np, c, B = Q.shape
    r = float(c) ** 0.25
    p = ws // 2
    if len(spatial) == 1:
        idx = np.arange(Np)
        d = np.abs(idx[:, None] - idx[None, :])
        mask = np.minimum(d, Np - d) <= p
    else:
        H, W = spatial
        h, w = np.arange(Np) % H, np.arange(Np) // H
        dh = np.abs(h[:, None] - h[None, :]); dh = np.minimum(dh, H - dh)
        dw = np.abs(w[:, None] - w[None, :]); dw = np.minimum(dw, W - dw)
        mask = (dh <= p) & (dw <= p)
    Y = np.zeros(Q.shape, dtype=V.dtype)
    A = np.zeros((Np, Np, B))
    for b in range(B):
        qb, kb = Q[:, :, b] / r, Kk[:, :, b] / r
        if kind == orc.DOT:
            S = np.real(qb @ np.conj(kb).T)
        else:
            S = -0.5 * (np.abs(qb[:, None, :] - kb[None, :, :]) ** 2).sum(-1)
        S = np.where(mask, S, -np.inf)
        P = np.exp(S - S.max(1, keepdims=True))
        P /= P.sum(1, keepdims=True)
        A[:, :, b] = P
        Y[:, :, b] = P @ V[:, :, b]
    return Y.reshape(np.asarray(q).shape, order="F"), A


@pytest.mark.parametrize("cplx", [False, True])
@pytest.mark.parametrize("kind", [orc.DOT, orc.DISTANCE])
@pytest.mark.parametrize("spatial,ws", [((11,), 5), ((7, 6), 5), ((5, 5), 5)])
def test_attention_matches_dense_masked(spatial, ws, kind, cplx):
    rng = np.random.default_rng(1)
    shape = spatial + (3, 2)
    q, k, v = (randn(rng, shape, cplx) for _ in range(3))
    y, nz = orc.attention(kind, q, k, v, ws)
    yd, Ad = dense_attention(kind, q, k, v, ws)
    np.testing.assert_allclose(y, yd, rtol=1e-12, atol=1e-12)
    cols, _ = orc.window_columns(spatial, ws)
    Np = cols.shape[1]
    A = np.zeros_like(Ad)
    for kk in range(cols.shape[0]):
        A[np.arange(Np), cols[kk], :] = nz[kk]
    np.testing.assert_allclose(A, Ad, rtol=1e-12, atol=1e-14)
    np.testing.assert_allclose(nz.sum(0), 1.0, rtol=1e-12)


def test_readme_identity_composed_equals_one_call():
    """README.md:115-119: softmax(similarity(q/sqrt(t), k/sqrt(t))) (x) v == y."""
    rng = np.random.default_rng(2)
    q, k, v = (randn(rng, (9, 8, 4, 2)) for _ in range(3))
    y, _ = orc.attention(orc.DISTANCE, q, k, v, 5)
    t = np.sqrt(4.0)
    S = orc.similarity(orc.DISTANCE, q / np.sqrt(t), k / np.sqrt(t), 5)
    u = orc.apply(orc.row_softmax(S), v, 5)
    np.testing.assert_allclose(u, y, rtol=1e-13)


def test_mh_attention_is_per_head_attention():
    rng = np.random.default_rng(3)
    q, k, v = (randn(rng, (8, 7, 6, 2)) for _ in range(3))
    y, nz = orc.mh_attention(orc.DOT, q, k, v, 3, 3)
    assert nz.shape == (9, 56, 6)
    for b in range(2):
        for hd in range(3):
            sl = slice(2 * hd, 2 * hd + 2)
            yh, nzh = orc.attention(orc.DOT, q[:, :, sl, b:b + 1], k[:, :, sl, b:b + 1], v[:, :, sl, b:b + 1], 3)
            np.testing.assert_allclose(y[:, :, sl, b:b + 1], yh, rtol=1e-13)
            np.testing.assert_allclose(nz[:, :, hd + 3 * b], nzh[:, :, 0], rtol=1e-13)


def test_entmax15_rows():
    rng = np.random.default_rng(4)
    nz = 3.0 * rng.standard_normal((25, 40, 3))
    P = orc.row_entmax15(nz)
    np.testing.assert_allclose(P.sum(0), 1.0, rtol=1e-12)
    assert (P == 0).any() and (P >= 0).all()
    # shift invariance and agreement with a bisection solve of the threshold
    np.testing.assert_allclose(orc.row_entmax15(nz + 7.0), P, atol=1e-12)
    z = nz[:, 5, 1] / 2
    lo, hi = z.max() - 1.0, z.max()
    for _ in range(200):
        mid = 0.5 * (lo + hi)
        if (np.clip(z - mid, 0, None) ** 2).sum() > 1.0:
            lo = mid
        else:
            hi = mid
    np.testing.assert_allclose(orc.entmax15_threshold(nz)[5, 1], lo, rtol=1e-10)


# ---------------------------------------------------------------- finite differences
def fd_grad(f, x, eps=1e-6):
    """central differences of scalar f wrt real array x (complex: re and im parts)."""
    g = np.zeros_like(x)
    it = np.nditer(x, flags=["multi_index"])
    for _ in it:
        idx = it.multi_index
        for unit in ([1.0, 1j] if np.iscomplexobj(x) else [1.0]):
            old = x[idx]
            x[idx] = old + eps * unit
            fp = f()
            x[idx] = old - eps * unit
            fm = f()
            x[idx] = old
            g[idx] += unit * (fp - fm) / (2 * eps)
    return g


RR_SHAPES = [((8,), 5), ((8, 8), 5)]


@pytest.mark.parametrize("cplx", [False, True])
@pytest.mark.parametrize("kind", [orc.DOT, orc.DISTANCE])
@pytest.mark.parametrize("spatial,ws", RR_SHAPES)
def test_similarity_pullback_fd(spatial, ws, kind, cplx):
    """test/rrule.jl:18-19."""
    rng = np.random.default_rng(5)
    c, B = (4, 2) if len(spatial) == 1 else (2, 1)
    x, y = randn(rng, spatial + (c, B), cplx), randn(rng, spatial + (c, B), cplx)
    dS = rng.standard_normal(orc.similarity(kind, x, y, ws).shape)
    dx, dy = orc.similarity_pullback(kind, x, y, ws, dS)
    f = lambda: float((dS * orc.similarity(kind, x, y, ws)).sum())
    np.testing.assert_allclose(dx, fd_grad(f, x), rtol=1e-6, atol=1e-7)
    np.testing.assert_allclose(dy, fd_grad(f, y), rtol=1e-6, atol=1e-7)


@pytest.mark.parametrize("cplx", [False, True])
@pytest.mark.parametrize("spatial,ws", RR_SHAPES)
def test_apply_pullback_fd(spatial, ws, cplx):
    """test/rrule.jl:20."""
    rng = np.random.default_rng(6)
    c, B = (4, 2) if len(spatial) == 1 else (2, 1)
    b = randn(rng, spatial + (c, B), cplx)
    K = ws ** len(spatial)
    Np = int(np.prod(spatial))
    nz = rng.standard_normal((K, Np, B))
    dc = randn(rng, spatial + (c, B), cplx)
    dA, db = orc.apply_pullback(nz, b, ws, dc)
    f = lambda: float(np.real(np.conj(dc) * orc.apply(nz, b, ws)).sum())
    np.testing.assert_allclose(dA, fd_grad(f, nz), rtol=1e-6, atol=1e-7)
    np.testing.assert_allclose(db, fd_grad(f, b), rtol=1e-6, atol=1e-7)


@pytest.mark.parametrize("norm", [orc.SOFTMAX, orc.ENTMAX15])
def test_row_normalize_pullback_fd(norm):
    """test/rrule.jl:21 (softmax); the entmax variant has no reference counterpart."""
    rng = np.random.default_rng(7)
    nz = rng.standard_normal((25, 6, 2)) * 2.0
    dP = rng.standard_normal(nz.shape)
    P = orc.row_normalize(norm, nz)
    dS = orc.row_normalize_pullback(norm, P, dP)
    f = lambda: float((dP * orc.row_normalize(norm, nz)).sum())
    np.testing.assert_allclose(dS, fd_grad(f, nz), rtol=1e-5, atol=1e-7)


def test_scale_pullback_fd():
    """test/rrule.jl:22: a of shape (1,1,2,2) against a Circulant with batch dims (1,2)."""
    rng = np.random.default_rng(8)
    nz = rng.standard_normal((5, 8, 1, 2))
    a = rng.standard_normal((1, 1, 2, 2))
    dB = rng.standard_normal((5, 8, 2, 2))
    dc, dA = orc.scale_pullback(a, nz, dB)
    f = lambda: float((dB * orc.scale(a, nz)).sum())
    np.testing.assert_allclose(dc, fd_grad(f, a), rtol=1e-6, atol=1e-8)
    np.testing.assert_allclose(dA, fd_grad(f, nz), rtol=1e-6, atol=1e-8)


@pytest.mark.parametrize("norm", [orc.SOFTMAX, orc.ENTMAX15])
@pytest.mark.parametrize("cplx", [False, True])
@pytest.mark.parametrize("kind", [orc.DOT, orc.DISTANCE])
@pytest.mark.parametrize("spatial,ws", [((8,), 5), ((6, 5), 3)])
def test_attention_pullback_fd(spatial, ws, kind, cplx, norm):
    """The composite gradient the fused backward must equal, including a
    cotangent arriving on the returned A."""
    rng = np.random.default_rng(9)
    shape = spatial + (3, 2)
    q, k, v = (randn(rng, shape, cplx) for _ in range(3))
    dy = randn(rng, shape, cplx)
    y0, nz0 = orc.attention(kind, q, k, v, ws, norm)
    dA = rng.standard_normal(nz0.shape)

    def f():
        y, nz = orc.attention(kind, q, k, v, ws, norm)
        return float(np.real(np.conj(dy) * y).sum() + (dA * nz).sum())
    dq, dk, dv = orc.attention_pullback(kind, q, k, v, ws, dy, dA, norm)
    np.testing.assert_allclose(dq, fd_grad(f, q), rtol=2e-5, atol=1e-7)
    np.testing.assert_allclose(dk, fd_grad(f, k), rtol=2e-5, atol=1e-7)
    np.testing.assert_allclose(dv, fd_grad(f, v), rtol=2e-5, atol=1e-7)


def test_sums():
    rng = np.random.default_rng(10)
    spatial, ws = (6, 5), 3
    nz = rng.standard_normal((9, 30, 2, 3))
    cols, _ = orc.window_columns(spatial, ws)
    dense = np.zeros((30, 30, 2, 3))
    for kk in range(9):
        dense[np.arange(30), cols[kk]] = nz[kk]
    np.testing.assert_allclose(orc.sum_dims2(nz), dense.sum(1), rtol=1e-12)
    np.testing.assert_allclose(orc.sum_dims1(nz, spatial, ws), dense.sum(0), rtol=1e-12, atol=1e-14)
    assert orc.sum_batch(nz, (3,)).shape == (9, 30, 1, 3)
    assert orc.sum_batch(nz, (3, 4)).shape == (9, 30, 1, 1)


def test_sampled_oracle_matches_full_oracle():
    rng = np.random.default_rng(12)
    shape, ws, nheads = (9, 8, 6, 2), 5, 2
    q, k, v, dy = (randn(rng, shape) for _ in range(4))
    qs, ks, vs, dys = (orc.splitheads(t, nheads) for t in (q, k, v, dy))
    pixels = [0, 7, 8, 35, 71, 40]
    for kind in (orc.DOT, orc.DISTANCE):
        y, _ = orc.attention(kind, qs, ks, vs, ws)
        dq, dk, dv = orc.attention_pullback(kind, qs, ks, vs, ws, dys)
        Y, _ = orc._flat(y); DQ, _ = orc._flat(dq); DK, _ = orc._flat(dk); DV, _ = orc._flat(dv)
        for unit in (0, 3):
            ys = orc.sampled_attention(kind, qs, ks, vs, ws, pixels, unit)
            sq, sk, sv = orc.sampled_attention_pullback(kind, qs, ks, vs, dys, ws, pixels, unit)
            np.testing.assert_allclose(ys, Y[pixels, :, unit], rtol=1e-11, atol=1e-13)
            np.testing.assert_allclose(sq, DQ[pixels, :, unit], rtol=1e-10, atol=1e-13)
            np.testing.assert_allclose(sk, DK[pixels, :, unit], rtol=1e-10, atol=1e-13)
            np.testing.assert_allclose(sv, DV[pixels, :, unit], rtol=1e-10, atol=1e-13)


@pytest.mark.parametrize("shape,ws,nheads,cplx,norm", [
    ((40, 6, 2), 9, 2, False, "entmax"),        # 1-D, entmax-1.5
    ((40, 6, 2), 9, 1, True, "softmax"),        # 1-D, complex
    ((9, 8, 4, 2), 5, 1, True, "softmax"),      # 2-D, complex
    ((9, 8, 6, 2), 5, 2, False, "entmax"),      # 2-D, entmax-1.5
])
def test_sampled_oracle_1d_entmax_complex(shape, ws, nheads, cplx, norm):
    """The sampled-pixel mode (used at the full BASELINE sizes) against the full oracle on small cases:
    1-D signals, the entmax normaliser, complex inputs, and the rows of A themselves."""
    rng = np.random.default_rng(21)
    nrm = orc.ENTMAX15 if norm == "entmax" else orc.SOFTMAX
    q, k, v, dy = (randn(rng, shape, cplx) for _ in range(4))
    qs, ks, vs, dys = (orc.splitheads(t.astype(np.complex128 if cplx else np.float64), nheads) for t in (q, k, v, dy))
    Np = int(np.prod(shape[:-2]))
    pixels = [0, 1, Np // 2, Np - 2, Np - 1, 7]
    for kind in (orc.DOT, orc.DISTANCE):
        y, P = orc.attention(kind, qs, ks, vs, ws, nrm)
        dq, dk, dv = orc.attention_pullback(kind, qs, ks, vs, ws, dys, norm=nrm)
        Y, _ = orc._flat(y); DQ, _ = orc._flat(dq); DK, _ = orc._flat(dk); DV, _ = orc._flat(dv)
        for unit in (0, qs.shape[-1] - 1):
            ys = orc.sampled_attention(kind, qs, ks, vs, ws, pixels, unit, nrm)
            sq, sk, sv = orc.sampled_attention_pullback(kind, qs, ks, vs, dys, ws, pixels, unit, nrm)
            np.testing.assert_allclose(ys, Y[pixels, :, unit], rtol=1e-10, atol=1e-12)
            np.testing.assert_allclose(sq, DQ[pixels, :, unit], rtol=1e-9, atol=1e-12)
            np.testing.assert_allclose(sk, DK[pixels, :, unit], rtol=1e-9, atol=1e-12)
            np.testing.assert_allclose(sv, DV[pixels, :, unit], rtol=1e-9, atol=1e-12)
            # rows of A: the sampled row holds the same values as the CSR row, which is sorted by column
            wins, rows = orc.sampled_rows(kind, qs, ks, ws, pixels, unit, nrm)
            for n, j in enumerate(pixels):
                order = np.argsort(wins[n], kind="stable")
                np.testing.assert_allclose(rows[n][order], P[:, j, unit], rtol=1e-10, atol=1e-13)
