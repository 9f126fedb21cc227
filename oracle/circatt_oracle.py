"""CPU oracle for circulant (sliding-window, circularly wrapped) attention.

TEST INFRASTRUCTURE ONLY.  This file is a float64 numpy restatement of the math
of nikopj/CirculantAttention.jl (v1.0.1).  It exists to check the CUDA library;
nothing in the shipped package may import it.

PARITY UNPINNED: the reference ships no golden vectors or known-answer tests for
forward values and it cannot run without Julia + CUDA.jl + a GPU.  What pins
this oracle instead:
  * the CSR structure is checked against a literal restatement of the
    reference's index function (`cartesian_circulant_*` below follows
    src/circulant.jl:4-44 line by line),
  * the similarity follows the reference kernels entry by entry
    (src/similarity.jl:55-103), and is cross-checked against a dense masked
    formulation,
  * every pullback is checked against central finite differences at the shapes
    and tolerances of the reference's own test/rrule.jl:1-23,
  * the README identity `softmax(S) (x) v == y` (README.md:115-119).

Array convention: arrays have the *Julia* logical shape, e.g. ``(H, W, C, B)``
or ``(N, C, B)``, and are indexed like Julia arrays (first index fastest in the
linearised pixel index ``h + H*w``).  Sparse values are kept as ``nz`` of shape
``(K, Np, *batch)`` -- the reference's ``reshape(nzVal, :, rows, batch)`` view
(src/similarity.jl:106) -- where ``K = ws**S`` entries of a row are in ascending
column order, exactly the CSR order of the reference.
"""
from __future__ import annotations

import numpy as np

DOT = 0
DISTANCE = 1
SOFTMAX = 0
ENTMAX15 = 1


# --------------------------------------------------------------------------
# R1: structure (src/circulant.jl)
# --------------------------------------------------------------------------
def _circshift_index(m, s, M):
    """src/circulant.jl:4 (1-based)."""
    return (m - 1 - s) % M + 1


def cartesian_circulant_1d(n, N, M):
    """Literal 1-based restatement of src/circulant.jl:6-18.

    ``n`` is the 1-based position of a stored entry.  Returns ``(i, j)``:
    ``j`` the CSR row (query pixel), ``i`` the CSR column (key pixel).
    """
    p = (M - 1) // 2
    j = -(-n // M)
    m = (n - 1) % M + 1
    if j <= p:
        m = _circshift_index(m, j - p - 1, M)
    elif j > N - p:
        m = _circshift_index(m, p - N + j, M)
    i = ((m - 1) + (j - 1) - p) % N + 1
    return i, j


def cartesian_circulant_2d(n, N1, N2, M):
    """Literal 1-based restatement of src/circulant.jl:21-43."""
    p = (M - 1) // 2
    j = -(-n // (M * M))
    jj = -(-j // N1)
    j0 = (j - 1) % N1 + 1
    nn = (-(-n // M) - 1) % M + 1 + M * (jj - 1)
    mm = (nn - 1) % M + 1
    m0 = n - M * (mm - 1) - (j - 1) * M * M
    if jj <= p:
        mm = _circshift_index(mm, jj - p - 1, M)
    elif jj > N2 - p:
        mm = _circshift_index(mm, p - N2 + jj, M)
    if j0 <= p:
        m0 = _circshift_index(m0, j0 - p - 1, M)
    elif j0 > N1 - p:
        m0 = _circshift_index(m0, p - N1 + j0, M)
    ii = ((mm - 1) + (jj - 1) - p) % N2 + 1
    i = N1 * (ii - 1) + ((m0 - 1) + (j0 - 1) - p) % N1 + 1
    return i, j


def structure_literal(spatial, ws):
    """colVal (1-based, length Np*K) by evaluating the literal index function
    for every stored entry, as the reference's structure kernels do
    (src/circulant.jl:46-62).  Slow; small sizes only."""
    spatial = tuple(int(s) for s in spatial)
    if len(spatial) == 1:
        N, = spatial
        return np.array([cartesian_circulant_1d(n, N, ws)[0]
                         for n in range(1, N * ws + 1)], dtype=np.int32)
    N1, N2 = spatial
    return np.array([cartesian_circulant_2d(n, N1, N2, ws)[0]
                     for n in range(1, N1 * N2 * ws * ws + 1)], dtype=np.int32)


def window_columns(spatial, ws):
    """Closed form of the structure.

    Returns ``cols`` of shape ``(K, Np)`` (0-based key pixel of every stored
    entry, ascending inside a row) and ``offs`` of the same shape: the index
    ``(dw+p)*ws + (dh+p)`` (``dh+p`` in 1-D) of the window offset stored there.
    """
    spatial = tuple(int(s) for s in spatial)
    if ws % 2 != 1:
        raise ValueError(f"filter size M={ws} must be odd.")  # src/circulant.jl:65,87
    if any(s < ws for s in spatial):
        raise ValueError("every spatial extent must be >= the window size")
    p = (ws - 1) // 2
    d = np.arange(-p, p + 1)
    if len(spatial) == 1:
        N, = spatial
        x = np.arange(N)
        col = (x[None, :] + d[:, None]) % N                       # (ws, N)
        off = np.broadcast_to(np.arange(ws)[:, None], col.shape)
    else:
        H, W = spatial
        pix = np.arange(H * W)
        h, w = pix % H, pix // H
        hh = (h[None, None, :] + d[None, :, None]) % H            # (1, ws, Np)
        ww = (w[None, None, :] + d[:, None, None]) % W            # (ws, 1, Np)
        col = (hh + H * ww).reshape(ws * ws, H * W)
        off = np.broadcast_to(np.arange(ws * ws)[:, None], col.shape)
    order = np.argsort(col, axis=0, kind="stable")
    cols = np.take_along_axis(col, order, axis=0)
    offs = np.take_along_axis(off, order, axis=0)
    return cols.astype(np.int64), offs.astype(np.int64)


def structure(spatial, ws):
    """rowPtr and colVal (both 1-based Int32) of one batch slice:
    ``rowPtr[r] = 1 + K*r`` (src/circulant.jl:71-73, 93-95)."""
    cols, _ = window_columns(spatial, ws)
    K, Np = cols.shape
    rowptr = (1 + K * np.arange(Np + 1)).astype(np.int32)
    colval = (cols.T.reshape(-1) + 1).astype(np.int32)
    return rowptr, colval


# --------------------------------------------------------------------------
# helpers
# --------------------------------------------------------------------------
def _flat(x):
    """(spatial..., c, batch) -> (Np, c, batch), Julia linearisation."""
    x = np.asarray(x)
    S = x.ndim - 2
    Np = int(np.prod(x.shape[:S]))
    return x.reshape((Np,) + x.shape[S:], order="F"), x.shape[:S]


def _unflat(X, shape):
    return X.reshape(shape, order="F")


def splitheads(x, nheads):
    """src/attention.jl:44 -- pure reshape, head index fastest in the merged
    batch dimension."""
    x = np.asarray(x)
    S = x.ndim - 2
    C = x.shape[S]
    assert C % nheads == 0
    return x.reshape(x.shape[:S] + (C // nheads, nheads * x.shape[-1]), order="F")


# --------------------------------------------------------------------------
# R3/R4: similarity (src/similarity.jl:55-103)
# --------------------------------------------------------------------------
def similarity(kind, x, y, ws):
    """nz[k, j, b] for row pixel j of x and the k-th stored key pixel i of y.

    Dot:      sum_m Re(x[j,m,b] * conj(y[i,m,b]))        (src/similarity.jl:98)
    Distance: -1/2 sum_m |x[j,m,b] - y[i,m,b]|^2          (src/similarity.jl:73-75)
    """
    X, spatial = _flat(x)
    Y, spatial_y = _flat(y)
    assert spatial == spatial_y and X.shape == Y.shape
    cols, _ = window_columns(spatial, ws)
    K, Np = cols.shape
    B = X.shape[2]
    out = np.empty((K, Np, B), dtype=np.float64)
    for k in range(K):
        Yk = Y[cols[k]]                                  # (Np, c, B)
        if kind == DOT:
            out[k] = np.real(X * np.conj(Yk)).sum(axis=1)
        elif kind == DISTANCE:
            out[k] = -0.5 * (np.abs(X - Yk) ** 2).sum(axis=1)
        else:
            raise ValueError("unknown similarity")
    return out


# --------------------------------------------------------------------------
# R5: row normalisers
# --------------------------------------------------------------------------
def row_softmax(nz):
    """softmax over the K stored entries of each row (src/similarity.jl:105-110)."""
    m = nz.max(axis=0, keepdims=True)
    e = np.exp(nz - m)
    return e / e.sum(axis=0, keepdims=True)


def row_logsumexp(nz):
    m = nz.max(axis=0)
    return m + np.log(np.exp(nz - m[None]).sum(axis=0))


def entmax15_threshold(nz):
    """tau of 1.5-entmax per row: sum_k max(nz/2 - tau, 0)^2 == 1 (exact, by
    sorting).  Not part of the reference."""
    z = np.sort(nz / 2.0, axis=0)[::-1]                   # descending
    K = z.shape[0]
    rho = np.arange(1, K + 1).reshape((K,) + (1,) * (z.ndim - 1))
    mean = np.cumsum(z, axis=0) / rho
    mean_sq = np.cumsum(z * z, axis=0) / rho
    ss = rho * (mean_sq - mean ** 2)
    delta = np.clip((1.0 - ss) / rho, 0.0, None)
    tau = mean - np.sqrt(delta)
    support = (tau <= z).sum(axis=0)                      # number of active entries
    return np.take_along_axis(tau, (support - 1)[None], axis=0)[0]


def row_entmax15(nz):
    tau = entmax15_threshold(nz)
    return np.clip(nz / 2.0 - tau[None], 0.0, None) ** 2


def row_normalize(norm, nz):
    return row_softmax(nz) if norm == SOFTMAX else row_entmax15(nz)


def row_normalize_pullback(norm, P, dP):
    """softmax: dS = P*(dP - sum_row P*dP)   (src/rrules.jl:42-56, NNlib's
    softmax gradient);  entmax-1.5: dS = g*(dP - sum g*dP / sum g), g = sqrt(P)."""
    if norm == SOFTMAX:
        return P * (dP - (P * dP).sum(axis=0, keepdims=True))
    g = np.sqrt(P)
    return g * (dP - (g * dP).sum(axis=0, keepdims=True) / g.sum(axis=0, keepdims=True))


# --------------------------------------------------------------------------
# R6: apply  (src/batchedmul.jl:82-110, src/attention.jl:53-80)
# --------------------------------------------------------------------------
def apply(nz, v, ws, transpose=False):
    """Y[j] = sum_i A[j,i] V[i]  ('N')  or  Y[i] = sum_j A[j,i] V[j]  ('T').
    ``nz`` is (K, Np, Bh) real; v is (spatial..., c, Bh), real or complex."""
    V, spatial = _flat(v)
    cols, _ = window_columns(spatial, ws)
    K, Np = cols.shape
    nzb = np.broadcast_to(nz, (K, Np, max(nz.shape[2], V.shape[2])))
    Bn = nzb.shape[2]
    V = np.broadcast_to(V, (Np, V.shape[1], Bn))
    Y = np.zeros((Np, V.shape[1], Bn), dtype=np.result_type(V.dtype, np.float64))
    for k in range(K):
        a = nzb[k][:, None, :]                            # (Np, 1, Bn)
        if not transpose:
            Y += a * V[cols[k]]
        else:
            np.add.at(Y, cols[k], a * V)
    return _unflat(Y, tuple(spatial) + Y.shape[1:])


# --------------------------------------------------------------------------
# R7/R8: attention (src/attention.jl:19-51)
# --------------------------------------------------------------------------
def attention(kind, q, k, v, ws, norm=SOFTMAX):
    """(y, nz).  tau = sqrt(c); both q and k are divided by sqrt(tau)
    (src/attention.jl:20-21); nz has shape (K, Np, B)."""
    q = np.asarray(q); k = np.asarray(k); v = np.asarray(v)
    c = k.shape[-2]
    r = np.sqrt(np.sqrt(float(c)))
    S = similarity(kind, q / r, k / r, ws)
    P = row_normalize(norm, S)
    y = apply(P, v, ws)
    return y, P


def mh_attention(kind, q, k, v, ws, nheads, norm=SOFTMAX):
    """src/attention.jl:38-42 with the similarity honoured (the reference drops
    it at :40 and always uses Dot).  nz has shape (K, Np, nheads*B), head
    fastest."""
    qr, kr, vr = (splitheads(t, nheads) for t in (q, k, v))
    y, P = attention(kind, qr, kr, vr, ws, norm)
    return y.reshape(np.asarray(q).shape, order="F"), P


# --------------------------------------------------------------------------
# R11: pullbacks of the pieces (src/rrules.jl)
# --------------------------------------------------------------------------
def similarity_pullback(kind, x, y, ws, dS):
    """src/rrules.jl:1-32.  Dot: dx = dS Y, dy = dS^T X.
    Distance: dx = dS Y - rowsum(dS) X, dy = dS^T X - colsum(dS) Y."""
    X, spatial = _flat(x)
    Y, _ = _flat(y)
    dx = apply(dS, y, ws)
    dy = apply(dS, x, ws, transpose=True)
    if kind == DISTANCE:
        rs = dS.sum(axis=0)                               # (Np, B)
        cs = sum_dims1(dS, spatial, ws)                   # (Np, B)
        dx = dx - _unflat(rs[:, None, :] * X, np.asarray(x).shape)
        dy = dy - _unflat(cs[:, None, :] * Y, np.asarray(y).shape)
    return dx, dy


def apply_pullback(nz, b, ws, dc):
    """src/rrules.jl:58-72: dA = Dot-similarity of (dc, b) on the window;
    db = A^T dc."""
    dA = similarity(DOT, dc, b, ws)
    db = apply(nz, dc, ws, transpose=True)
    return dA, db


def attention_pullback(kind, q, k, v, ws, dy, dA=None, norm=SOFTMAX):
    """Composite gradient of `attention` = composition of the reference's
    rrules for similarity, softmax and apply (src/rrules.jl:1-72).
    Returns (dq, dk, dv)."""
    q = np.asarray(q); k = np.asarray(k); v = np.asarray(v)
    c = k.shape[-2]
    r = np.sqrt(np.sqrt(float(c)))
    S = similarity(kind, q / r, k / r, ws)
    P = row_normalize(norm, S)
    dP, dv = apply_pullback(P, v, ws, dy)
    if dA is not None:
        dP = dP + dA
    dS = row_normalize_pullback(norm, P, dP)
    dqs, dks = similarity_pullback(kind, q / r, k / r, ws, dS)
    return dqs / r, dks / r, dv


def mh_attention_pullback(kind, q, k, v, ws, nheads, dy, dA=None, norm=SOFTMAX):
    qr, kr, vr, dyr = (splitheads(t, nheads) for t in (q, k, v, dy))
    dq, dk, dv = attention_pullback(kind, qr, kr, vr, ws, dyr, dA, norm)
    shp = np.asarray(q).shape
    return tuple(t.reshape(shp, order="F") for t in (dq, dk, dv))


# --------------------------------------------------------------------------
# R9: sums (src/array.jl:119-177)   nz: (K, Np, *batch)
# --------------------------------------------------------------------------
def sum_dims2(nz):
    """row sums (src/array.jl:126-130) -> (Np, *batch)."""
    return nz.sum(axis=0)


def sum_dims1(nz, spatial, ws):
    """column sums (src/array.jl:119-124) -> (Np, *batch)."""
    cols, _ = window_columns(spatial, ws)
    out = np.zeros(nz.shape[1:], dtype=nz.dtype)
    for k in range(cols.shape[0]):
        np.add.at(out, cols[k], nz[k])
    return out


def sum_batch(nz, dims):
    """sum over batch dims (Julia dims > 2, 1-based; src/array.jl:132-149).
    Julia dim d of the (Np, Np, batch...) array is axis d-1 of nz."""
    return nz.sum(axis=tuple(d - 1 for d in dims), keepdims=True)


# --------------------------------------------------------------------------
# R10: algebra (src/array.jl:66-85, 179-189)
# --------------------------------------------------------------------------
def scale(c, nz):
    """c has Julia shape (1, 1, batch...); values multiplied by c broadcast
    over the batch dims (src/array.jl:179-186)."""
    c = np.asarray(c)
    assert c.shape[0] == 1 and c.shape[1] == 1, \
        "Scaling of non-batchdims of CuSparseArrayCSR not implemented"
    return c.reshape((1,) + c.shape[1:]) * nz


def scale_pullback(c, nz, dB):
    """src/rrules.jl:97-114.  dc = sum of dB*A over the value dims and over the
    batch dims where c has extent 1; dA = scale(c, dB) summed over the batch
    dims where A has extent 1."""
    c = np.asarray(c)
    axes = (0, 1) + tuple(d for d in range(2, c.ndim) if c.shape[d] == 1)
    dc = (dB * nz).sum(axis=axes).reshape(c.shape)
    dA = scale(c, dB)
    axes = tuple(a for a in range(2, nz.ndim) if nz.shape[a] == 1)
    if axes:
        dA = dA.sum(axis=axes, keepdims=True)
    return dc, dA


# --------------------------------------------------------------------------
# Sampled-pixel mode for sizes where the full oracle is too slow (1-D or 2-D,
# real or complex, softmax or entmax-1.5).  y[j], the row A[j, :] and dq[j]
# depend only on the window of j; dk[i] and dv[i] only on the queries whose
# window contains i, each with its own window.  Same arithmetic as `attention`
# / `attention_pullback`, restricted to the requested pixels.  q, k, v, dy:
# head-split (spatial..., c, units) arrays.
# --------------------------------------------------------------------------
def _window_pixels(j, spatial, p):
    """key pixels of query pixel j (linear index) in ascending window-offset order: dw-major, dh-minor
    in 2-D (the CSR order of an interior row; border rows of the CSR are rotations of it)."""
    d = np.arange(-p, p + 1)
    if len(spatial) == 1:
        return (j + d) % spatial[0]
    H, W = spatial
    hh = (j % H + d) % H
    ww = (j // H + d) % W
    return (hh[None, :] + H * ww[:, None]).reshape(-1)


def _row(kind, qj, Kwin, scale):
    """scores of one query against its window keys: qj (c,), Kwin (K, c)."""
    if kind == DOT:
        return scale * np.real(Kwin.conj() @ qj)
    return -0.5 * scale * (np.abs(qj[None, :] - Kwin) ** 2).sum(axis=1)


def _normalize_row(norm, s):
    if norm == SOFTMAX:
        pr = np.exp(s - s.max())
        return pr / pr.sum()
    return row_entmax15(s[:, None])[:, 0]


def sampled_rows(kind, q, k, ws, pixels, unit, norm=SOFTMAX):
    """(window key pixels, normalised weights) of the rows A[j, :] at the given pixels of one unit,
    each (len(pixels), K), in window-offset order (not the sorted CSR order)."""
    Q, spatial = _flat(q); Kk, _ = _flat(k)
    scale = 1.0 / np.sqrt(float(Q.shape[1]))
    p = (ws - 1) // 2
    wins, rows = [], []
    for j in pixels:
        win = _window_pixels(int(j), spatial, p)
        wins.append(win)
        rows.append(_normalize_row(norm, _row(kind, Q[j, :, unit], Kk[win, :, unit], scale)))
    return np.array(wins), np.array(rows)


def sampled_attention(kind, q, k, v, ws, pixels, unit, norm=SOFTMAX):
    """y at the given linear pixels of one unit -> (len(pixels), c)."""
    V, _ = _flat(v)
    wins, rows = sampled_rows(kind, q, k, ws, pixels, unit, norm)
    out = np.zeros((len(pixels), V.shape[1]), dtype=np.result_type(V.dtype, np.float64))
    for n in range(len(pixels)):
        out[n] = rows[n] @ V[wins[n], :, unit]
    return out


def sampled_attention_pullback(kind, q, k, v, dy, ws, pixels, unit, norm=SOFTMAX):
    """(dq, dk, dv) rows at the given pixels of one unit, each (len(pixels), c)."""
    Q, spatial = _flat(q); Kk, _ = _flat(k); V, _ = _flat(v); DY, _ = _flat(dy)
    c = Q.shape[1]
    scale = 1.0 / np.sqrt(float(c))
    p = (ws - 1) // 2
    cache = {}

    def row_terms(j):
        """window, P and dS of query row j."""
        if j not in cache:
            win = _window_pixels(j, spatial, p)
            P = _normalize_row(norm, _row(kind, Q[j, :, unit], Kk[win, :, unit], scale))
            dP = np.real(V[win, :, unit].conj() @ DY[j, :, unit])
            dS = row_normalize_pullback(norm, P[:, None], dP[:, None])[:, 0]
            cache[j] = (win, P, dS)
        return cache[j]

    dq = np.zeros((len(pixels), c), dtype=Q.dtype); dk = np.zeros_like(dq); dv = np.zeros_like(dq)
    for n, j in enumerate(pixels):
        j = int(j)
        win, P, dS = row_terms(j)
        dq[n] = scale * (dS @ Kk[win, :, unit])
        if kind == DISTANCE:
            dq[n] -= scale * dS.sum() * Q[j, :, unit]
        # as a key: every query whose window contains j (window symmetry: the same pixel set)
        sum_ds = 0.0
        for jq in win:
            wq, Pq, dSq = row_terms(int(jq))
            pos = int(np.nonzero(wq == j)[0][0])
            dk[n] += scale * dSq[pos] * Q[jq, :, unit]
            dv[n] += Pq[pos] * DY[jq, :, unit]
            sum_ds += dSq[pos]
        if kind == DISTANCE:
            dk[n] -= scale * sum_ds * Kk[j, :, unit]
    return dq, dk, dv
