"""Host-side mirror of CirculantAttention.jl's public API.

Names, argument meaning and error behaviour follow the reference; Julia's `!`
suffix becomes a trailing underscore, `⊗` is `otimes` and `⨷` is `Otimes`.
Dense arrays are Julia-shaped column-major tensors (see `jl`).  Gradients are
attached with `torch.autograd.Function`s that play the role of the reference's
ChainRules rrules (src/rrules.jl); every forward and pullback is one or more
calls into the C ABI.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from . import jl, ops
from ._lib import CA_DISTANCE, CA_DOT, CA_ENTMAX15, CA_SOFTMAX


# ----------------------------------------------------------------- similarity types
class AbstractSimilarity:
    kind = None

    def __repr__(self):
        return type(self).__name__ + "()"


class DotSimilarity(AbstractSimilarity):
    """S_ij = Re(q_i^H k_j)  (src/similarity.jl:3-15)."""
    kind = CA_DOT


class DistanceSimilarity(AbstractSimilarity):
    """S_ij = -1/2 sum |q_i - k_j|^2.  The reference's code is negative
    (src/similarity.jl:73-75) although its docstring (:24) omits the sign."""
    kind = CA_DISTANCE


SOFTMAX, ENTMAX15 = CA_SOFTMAX, CA_ENTMAX15


# ----------------------------------------------------------------- CSR container
_STRUCT_CACHE = {}


class CuSparseArrayCSR:
    """Stand-in for CUDA.jl's CuSparseArrayCSR{Float32,Int32,N}: fields rowPtr,
    colVal, nzVal, dims, nnz.  rowPtr/colVal are replicated per batch slice as
    in the reference (src/array.jl:9) but are only generated when somebody
    reads them; the kernels never do."""

    def __init__(self, nzVal, dims, spatial, ws, rowPtr=None, colVal=None):
        self.nzVal = nzVal
        self.dims = tuple(int(d) for d in dims)
        self._spatial = tuple(spatial)
        self._ws = int(ws)
        self._rowPtr, self._colVal = rowPtr, colVal

    @property
    def nnz(self):
        return self.nzVal.numel()

    def _structure(self):
        if self._rowPtr is None:
            key = (self._spatial, self._ws, self.dims[2:], self.nzVal.device)
            if key not in _STRUCT_CACHE:
                _STRUCT_CACHE[key] = ops.structure(self._spatial, self._ws, self.dims[2:], self.nzVal.device)
            self._rowPtr, self._colVal = _STRUCT_CACHE[key]
        return self._rowPtr, self._colVal

    @property
    def rowPtr(self):
        return self._structure()[0]

    @property
    def colVal(self):
        return self._structure()[1]


class Circulant:
    """Circulant{T,N,M,S} (src/array.jl:1-18): `data` is the CSR array,
    `kernel_length` the window M, `spatial_size` the S spatial extents."""

    def __init__(self, *args, dtype=torch.float32, device="cuda"):
        if len(args) == 3 and isinstance(args[0], CuSparseArrayCSR):      # Circulant(D, M, spatsize)
            self.data, self.kernel_length, self.spatial_size = args[0], int(args[1]), tuple(args[2])
            return
        if len(args) == 2:                                                # Circulant(M, dims): ones
            M, dims = int(args[0]), tuple(int(d) for d in args[1])
            _check_odd(M)
            spatial, batch = dims[:-2], dims[-2:]
            Np, K = math.prod(spatial), M ** len(spatial)
            nz = jl.ones((Np * K,) + batch, torch.float32, device)
            self.data = CuSparseArrayCSR(nz, (Np, Np) + batch, spatial, M)
            self.kernel_length, self.spatial_size = M, spatial
            return
        raise TypeError("Circulant(M, dims) or Circulant(data, M, spatial_size)")

    # -- construction helper used by every op
    @staticmethod
    def _from_nz(nz, M, spatial):
        Np = math.prod(spatial)
        return Circulant(CuSparseArrayCSR(nz, (Np, Np) + tuple(nz.shape[1:]), spatial, M), M, spatial)

    # -- accessors (src/array.jl:31-42)
    @property
    def nzVal(self):
        return self.data.nzVal

    @property
    def shape(self):
        return self.data.dims

    def size(self, i: Optional[int] = None):
        return self.data.dims if i is None else self.data.dims[i - 1]     # 1-based like Julia

    @property
    def ndim(self):
        return len(self.data.dims)

    @property
    def batch(self):
        return self.data.dims[2:]

    def __repr__(self):
        return (f"Circulant{{Float32, {self.ndim}, {self.kernel_length}, {len(self.spatial_size)}}} with "
                f"kernel-length {self.kernel_length}, spatial-size {self.spatial_size}, and data,\n"
                f"{'×'.join(str(d) for d in self.shape)} CuSparseArrayCSR with {self.data.nnz} stored entries")

    def similar(self):
        return Circulant._from_nz(jl.empty(self.nzVal.shape, torch.float32, self.nzVal.device),
                                  self.kernel_length, self.spatial_size)

    def copy(self):
        return Circulant._from_nz(ops.axpby(1.0, self.nzVal.detach()), self.kernel_length, self.spatial_size)

    def reshape(self, *dims):
        """Base.reshape on the batch dims (src/array.jl:54-56); dims[0:2] stay (Np, Np)."""
        dims = list(dims[0]) if len(dims) == 1 and isinstance(dims[0], (tuple, list)) else list(dims)
        Np = self.shape[0]
        batch = dims[2:]
        total = math.prod(self.batch)
        if batch.count(-1) == 1:
            known = math.prod(b for b in batch if b != -1)
            batch[batch.index(-1)] = total // max(known, 1)
        if math.prod(batch) != total:
            raise AssertionError(f"cannot reshape batch dims {self.batch} to {tuple(batch)}")
        nz = jl.reshape(self.nzVal, (self.nzVal.shape[0],) + tuple(batch))
        return Circulant._from_nz(nz, self.kernel_length, self.spatial_size)

    def repeat(self, *reps):
        """Base.repeat (src/array.jl:49-52); reps[0:2] must be 1."""
        if len(reps) < 2 or reps[0] != 1 or reps[1] != 1:
            raise AssertionError("only batch dims of a Circulant can be repeated")
        breps = tuple(reps[2:]) + (1,) * (len(self.batch) - len(reps[2:]))
        c = jl.ones(breps, torch.float32, self.nzVal.device)
        return Circulant._from_nz(_ScaleFn.apply(c, self.nzVal), self.kernel_length, self.spatial_size)

    # -- algebra (src/array.jl:66-85, 179-189)
    def _same(self, other):
        if not isinstance(other, Circulant) or other.kernel_length != self.kernel_length \
                or other.spatial_size != self.spatial_size or other.shape != self.shape:
            raise TypeError("Circulant algebra needs equal window, spatial size and dims")

    def __add__(self, other):
        self._same(other)
        return Circulant._from_nz(_AxpbyFn.apply(self.nzVal, other.nzVal, 1.0, 1.0), self.kernel_length, self.spatial_size)

    def __sub__(self, other):
        self._same(other)
        return Circulant._from_nz(_AxpbyFn.apply(self.nzVal, other.nzVal, 1.0, -1.0), self.kernel_length, self.spatial_size)

    def __neg__(self):
        return -1 * self

    def __mul__(self, c):
        return self.__rmul__(c)

    def __rmul__(self, c):
        if isinstance(c, torch.Tensor) and c.ndim > 0:
            return scale(c, self)                                        # src/array.jl:189
        return Circulant._from_nz(_AxpbyFn.apply(self.nzVal, None, float(c), 0.0), self.kernel_length, self.spatial_size)

    def __eq__(self, other):                                             # src/array.jl:103-117
        if not isinstance(other, Circulant):
            return NotImplemented
        if self.shape != other.shape or self.spatial_size != other.spatial_size \
                or self.kernel_length != other.kernel_length:
            return False
        return bool(torch.equal(self.nzVal, other.nzVal))

    __hash__ = None

    def __matmul__(self, x):
        return otimes(self, x)


def _check_odd(M):
    assert M % 2 == 1, f"filter size M={M} must be odd."                 # src/circulant.jl:65,87


def circulant(M: int, x: torch.Tensor) -> Circulant:
    """src/array.jl:29: a ones-valued Circulant shaped for x."""
    return Circulant(M, tuple(x.shape[:-2]) + (1, x.shape[-1]), device=x.device)


def kernel_length(A):
    return A.kernel_length


def spatial_size(A):
    return A.spatial_size


def spatial_dims(A):
    return len(A.spatial_size)


# ----------------------------------------------------------------- autograd glue
class _AxpbyFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, y, alpha, beta):
        ctx.ab = (alpha, beta, y is not None)
        return ops.axpby(alpha, x, beta, y)

    @staticmethod
    def backward(ctx, g):
        alpha, beta, has_y = ctx.ab
        gx = ops.axpby(alpha, g) if ctx.needs_input_grad[0] else None
        gy = ops.axpby(beta, g) if has_y and ctx.needs_input_grad[1] else None
        return gx, gy, None, None


class _ScaleFn(torch.autograd.Function):
    """scale(c, A) and its pullback (src/array.jl:179-186, src/rrules.jl:97-114)."""

    @staticmethod
    def forward(ctx, c, nz):
        ctx.save_for_backward(c, nz)
        return ops.scale_batch(c, nz)

    @staticmethod
    def backward(ctx, dB):
        c, nz = ctx.saved_tensors
        dc = dA = None
        nb = max(c.ndim, nz.ndim - 1)
        cs = tuple(c.shape) + (1,) * (nb - c.ndim)
        as_ = tuple(nz.shape[1:]) + (1,) * (nb - (nz.ndim - 1))
        if ctx.needs_input_grad[0]:
            full = ops.dot_batch(dB, nz)                                  # (o1, o2): per-slice sum dB*A
            full = jl.reshape(full, (1,) + tuple(full.shape))
            s1 = cs[0] == 1 and full.shape[1] > 1
            s2 = len(cs) > 1 and cs[1] == 1 and full.ndim > 2 and full.shape[2] > 1
            red = ops.sum_batch(full, s1, s2) if (s1 or s2) else full
            dc = jl.reshape(red, tuple(c.shape))
        if ctx.needs_input_grad[1]:
            full = ops.scale_batch(c, dB)
            s1 = as_[0] == 1 and full.shape[1] > 1
            s2 = len(as_) > 1 and as_[1] == 1 and full.ndim > 2 and full.shape[2] > 1
            red = ops.sum_batch(full, s1, s2) if (s1 or s2) else full
            dA = jl.reshape(red, tuple(nz.shape))
        return dc, dA


class _SimilarityFn(torch.autograd.Function):
    """circulant_similarity and its rrules (src/similarity.jl:138-142, src/rrules.jl:1-32)."""

    @staticmethod
    def forward(ctx, x, y, kind, ws):
        ctx.save_for_backward(x, y)
        ctx.cfg = (kind, ws)
        return ops.similarity(kind, x, y, ws)

    @staticmethod
    def backward(ctx, dS):
        x, y = ctx.saved_tensors
        kind, ws = ctx.cfg
        dx, dy = ops.similarity_bwd(kind, x, y, ws, dS)
        return dx, dy, None, None


class _NormalizeFn(torch.autograd.Function):
    """NNlib.softmax(::Circulant) and its rrule (src/similarity.jl:113-126, src/rrules.jl:42-56)."""

    @staticmethod
    def forward(ctx, nz, spatial, ws, normalizer):
        p = ops.row_normalize(nz, spatial, ws, normalizer)
        ctx.save_for_backward(p)
        ctx.cfg = (spatial, ws, normalizer)
        return p

    @staticmethod
    def backward(ctx, dp):
        (p,) = ctx.saved_tensors
        spatial, ws, normalizer = ctx.cfg
        return ops.row_normalize_bwd(p, dp, spatial, ws, normalizer), None, None, None


class _ApplyFn(torch.autograd.Function):
    """A ⊗ x / Aᵀ ⊗ x and their rrules (src/attention.jl:53-80, src/rrules.jl:58-88)."""

    @staticmethod
    def forward(ctx, nz, x, ws, transpose):
        ctx.save_for_backward(nz, x)
        ctx.cfg = (ws, transpose)
        return ops.apply(jl.reshape(nz, (nz.shape[0], -1)), x, ws, transpose)

    @staticmethod
    def backward(ctx, dc):
        nz, x = ctx.saved_tensors
        ws, transpose = ctx.cfg
        ua = nz.numel() // nz.shape[0]
        if ua != x.shape[-1]:
            raise NotImplementedError("pullback of a batch-broadcast apply is not defined by the reference")
        dA = db = None
        if ctx.needs_input_grad[0]:
            d = ops.similarity(CA_DOT, dc, x, ws) if not transpose else ops.similarity(CA_DOT, x, dc, ws)
            dA = jl.reshape(d, tuple(nz.shape))
        if ctx.needs_input_grad[1]:
            db = ops.apply(jl.reshape(nz, (nz.shape[0], -1)), dc, ws, not transpose)
        return dA, db, None, None


class _AttentionFn(torch.autograd.Function):
    """Fused circulant_(mh_)attention with a direct pullback equal to the composition of the reference's
    rrules (src/rrules.jl:1-72).  The head split (src/attention.jl:44, a reshape) happens inside, so the
    autograd graph holds one node for the whole call instead of one per reshape."""

    @staticmethod
    def forward(ctx, q, k, v, kind, ws, normalizer, want_A, scale=None, nheads=1):
        qr, kr, vr = (splitheads(t, nheads) for t in (q, k, v)) if nheads != 1 else (q, k, v)
        # the forward's workspace (the packed copy of k and v) is kept for the pullback, like the
        # intermediates the reference's pullback closures capture (src/rrules.jl:44-55)
        y, nz, stats, fws = ops.attention_fwd(kind, normalizer, qr, kr, vr, ws, want_A, scale=scale, keep_workspace=True)
        ctx.set_materialize_grads(False)      # an unused A must arrive as None, not as zeros, in backward
        ctx.save_for_backward(qr, kr, vr, y, stats, nz if want_A else None)
        ctx.fws = fws if normalizer == 0 else None
        ctx.cfg = (kind, ws, normalizer, want_A, scale, nheads, tuple(q.shape))
        yo = jl.reshape(y, tuple(q.shape)) if nheads != 1 else y
        return (yo, nz) if want_A else (yo, None)

    @staticmethod
    def backward(ctx, dy, dnz):
        q, k, v, y, stats, nz = ctx.saved_tensors
        kind, ws, normalizer, want_A, scale, nheads, shape = ctx.cfg
        if dy is None:
            dy = jl.zeros(y.shape, y.dtype, y.device)
        elif nheads != 1:
            dy = splitheads(dy, nheads)
        # the saved A (when the forward materialised it) spares the operator-chain backward a recomputation
        dq, dk, dv = ops.attention_bwd(kind, normalizer, q, k, v, y, dy, stats, ws, nz=nz, dA=dnz, scale=scale,
                                       fwd_workspace=ctx.fws)
        ctx.fws = None
        if nheads != 1:
            dq, dk, dv = (jl.reshape(t, shape) for t in (dq, dk, dv))
        return dq, dk, dv, None, None, None, None, None, None


# ----------------------------------------------------------------- L2: similarity / adjacency
def _kind(simfun):
    if not isinstance(simfun, AbstractSimilarity):
        raise TypeError(f"simfun must be DotSimilarity() or DistanceSimilarity(), got {simfun!r}")
    return simfun.kind


def _check_xy(x, y):
    if x.shape != y.shape or x.dtype != y.dtype:
        raise TypeError("x and y must have the same element type and size")


def circulant_similarity(simfun, x, y, W: int) -> Circulant:
    """src/similarity.jl:138-142.  Returns a Circulant of size (Np, Np, 1, B)."""
    _check_odd(W)
    _check_xy(x, y)
    nz = _SimilarityFn.apply(x, y, _kind(simfun), int(W))
    nz = jl.reshape(nz, (nz.shape[0], 1, x.shape[-1]))
    return Circulant._from_nz(nz, int(W), tuple(x.shape[:-2]))


def circulant_similarity_(A: Circulant, simfun, x, y) -> Circulant:
    """circulant_similarity! (src/similarity.jl:31-53): overwrites A's values."""
    S, N = spatial_dims(A), x.ndim
    assert S == N - 2, f"spatial_dims ({S}) of circulant matrix must match those of data signal ({N - 2})."
    nb = math.prod(A.batch)
    assert nb == x.shape[-1], f"batchdim of circulant matrix ({nb}) must match that of x, y ({x.shape[-1]})."
    nz = ops.similarity(_kind(simfun), x, y, A.kernel_length)
    A.data.nzVal = jl.reshape(nz, tuple(A.nzVal.shape))
    return A


def softmax(A: Circulant, normalizer=SOFTMAX) -> Circulant:
    """NNlib.softmax(A::Circulant): row-wise (src/similarity.jl:113-126)."""
    p = _NormalizeFn.apply(A.nzVal, A.spatial_size, A.kernel_length, normalizer)
    return Circulant._from_nz(p, A.kernel_length, A.spatial_size)


def softmax_(A: Circulant, B: Optional[Circulant] = None, normalizer=SOFTMAX) -> Circulant:
    """NNlib.softmax!(A, B=A)."""
    src = A if B is None else B
    ops.row_normalize(src.nzVal.detach(), A.spatial_size, A.kernel_length, normalizer, out=A.nzVal)
    return A


def entmax15(A: Circulant) -> Circulant:
    """Row-wise 1.5-entmax (no counterpart in the reference)."""
    return softmax(A, normalizer=ENTMAX15)


def circulant_adjacency(simfun, x, y, W: int, normalizer=SOFTMAX, lazy=False):
    """(softmax ∘ circulant_similarity)(simfun, x, y, W)  (src/similarity.jl:157-161).
    `lazy=True` returns a LazyAdjacency: nothing is computed until the result is applied or inspected."""
    if lazy:
        _check_odd(W)
        _check_xy(x, y)
        return LazyAdjacency([(1, simfun, x, y, normalizer)], W, 1, tuple(x.shape[:-2]), x.shape[-1], False)
    return softmax(circulant_similarity(simfun, x, y, W), normalizer)


def circulant_adjacency_(A: Circulant, simfun, x, y) -> Circulant:
    circulant_similarity_(A, simfun, x, y)
    return softmax_(A)


# ----------------------------------------------------------------- L3: attention
def splitheads(x, nheads):
    """src/attention.jl:44: (spatial..., C, B) -> (spatial..., C/nheads, nheads*B), a reshape."""
    C = x.shape[-2]
    assert C % nheads == 0, f"channels ({C}) must be divisible by nheads ({nheads})"
    return jl.reshape(x, tuple(x.shape[:-2]) + (C // nheads, nheads * x.shape[-1]))


def _fused(simfun, q, k, v, W, nheads, normalizer, return_A):
    _check_odd(W)
    if not (q.shape == k.shape == v.shape and q.dtype == k.dtype == v.dtype):
        raise TypeError("q, k, v must have the same element type and size")
    B = q.shape[-1]
    assert q.shape[-2] % nheads == 0, f"channels ({q.shape[-2]}) must be divisible by nheads ({nheads})"
    y, nz = _AttentionFn.apply(q, k, v, _kind(simfun), int(W), normalizer, bool(return_A), None, int(nheads))
    if not return_A:
        return y, None
    nz = jl.reshape(nz, (nz.shape[0], nheads, B))
    return y, Circulant._from_nz(nz, int(W), tuple(q.shape[:-2]))


def circulant_attention(*args, normalizer=SOFTMAX, return_A=True):
    """circulant_attention(simfun, q, k, v, W) -> (y, A)     src/attention.jl:19-25
       circulant_attention(q, k, v, W)         -> (y, A)     src/attention.jl:26 (Dot)
       circulant_attention(A, x)               -> y = A ⊗ x  src/attention.jl:68
    One fused kernel instead of similarity + softmax + SpMM; tau = sqrt(channels) as
    in the reference.  `return_A=False` is the flash mode: A is never written."""
    if len(args) == 2 and isinstance(args[0], Circulant):
        return otimes(*args)
    if len(args) == 4:
        args = (DotSimilarity(),) + tuple(args)
    if len(args) != 5:
        raise TypeError("circulant_attention(simfun, q, k, v, W), (q, k, v, W) or (A, x)")
    simfun, q, k, v, W = args
    return _fused(simfun, q, k, v, W, 1, normalizer, return_A)


def circulant_mh_attention(*args, normalizer=SOFTMAX, return_A=True):
    """circulant_mh_attention(simfun, q, k, v, W, nheads) -> (y, A)   src/attention.jl:38-42
       circulant_mh_attention(q, k, v, W, nheads)         -> (y, A)   (Dot)
       circulant_mh_attention(A, x)                       -> y = A ⨷ x  src/attention.jl:89-94
    Unlike src/attention.jl:40 the similarity argument is honoured, and the 5-argument
    form works (src/attention.jl:43 calls a method that does not exist)."""
    if len(args) == 2 and isinstance(args[0], Circulant):
        return Otimes(*args)
    if len(args) == 5:
        args = (DotSimilarity(),) + tuple(args)
    if len(args) != 6:
        raise TypeError("circulant_mh_attention(simfun, q, k, v, W, nheads), (q, k, v, W, nheads) or (A, x)")
    simfun, q, k, v, W, nheads = args
    return _fused(simfun, q, k, v, W, int(nheads), normalizer, return_A)


def circulant_mh_adjacency(simfun, x, y, W: int, nheads: int, normalizer=SOFTMAX, lazy=False):
    """src/attention.jl:46-51.  `lazy=True` returns a LazyAdjacency (see there)."""
    if lazy:
        _check_odd(W)
        _check_xy(x, y)
        assert x.shape[-2] % nheads == 0, f"channels ({x.shape[-2]}) must be divisible by nheads ({nheads})"
        return LazyAdjacency([(1, simfun, x, y, normalizer)], W, nheads, tuple(x.shape[:-2]), x.shape[-1], True)
    xr, yr = splitheads(x, nheads), splitheads(y, nheads)
    A = circulant_adjacency(simfun, xr, yr, W, normalizer)
    return _circulant_reshape(A, nheads, x.shape[-1])


def _circulant_reshape(A: Circulant, *batch) -> Circulant:
    """src/array.jl:58-60 (its rrule, src/rrules.jl:34-40, is autograd's reshape)."""
    return A.reshape(A.shape[0], A.shape[1], *batch)


def _apply(A: Circulant, x, transpose):
    N = x.ndim
    assert spatial_dims(A) == N - 2, \
        f"spatial-dims ({spatial_dims(A)} of A must match spatial dims of x ({N - 2})"
    assert tuple(x.shape[:-2]) == A.spatial_size, \
        f"spatial size {A.spatial_size} of A must match that of x {tuple(x.shape[:-2])}"
    return _ApplyFn.apply(A.nzVal, x, A.kernel_length, transpose)


def otimes(A: Circulant, x):
    """y = A ⊗ x (src/attention.jl:53-70)."""
    if isinstance(A, LazyAdjacency):
        if A.mh:
            raise TypeError("A ⊗ x needs a single-head adjacency; use ⨷ (Otimes) for a multi-head one")
        return A.apply(x)
    return _apply(A, x, False)


def circulant_attention_(y, A: Circulant, x):
    """circulant_attention!(y, A, x) (src/attention.jl:53-59)."""
    ops.apply(jl.reshape(A.nzVal.detach(), (A.nzVal.shape[0], -1)), x, A.kernel_length, False, out=y)
    return y


def circulant_transposed_attention(A: Circulant, x):
    """src/attention.jl:72-80."""
    return _apply(A, x, True)


def circulant_transposed_attention_(y, A: Circulant, x):
    ops.apply(jl.reshape(A.nzVal.detach(), (A.nzVal.shape[0], -1)), x, A.kernel_length, True, out=y)
    return y


def Otimes(A: Circulant, x):
    """y = A ⨷ x: multi-head apply, nheads = size(A, 3) (src/attention.jl:89-94)."""
    if isinstance(A, LazyAdjacency):
        if not A.mh:
            raise TypeError("A ⨷ x needs a 4-dimensional Circulant (Np, Np, nheads, B)")
        return A.apply(x)
    if A.ndim != 4:
        raise TypeError("A ⨷ x needs a 4-dimensional Circulant (Np, Np, nheads, B)")
    xr = splitheads(x, A.size(3))
    return jl.reshape(otimes(A, xr), tuple(x.shape))


def circulant_mh_transposed_attention(A: Circulant, x):
    """src/attention.jl:98-103."""
    if A.ndim != 4:
        raise TypeError("needs a 4-dimensional Circulant (Np, Np, nheads, B)")
    xr = splitheads(x, A.size(3))
    return jl.reshape(circulant_transposed_attention(A, xr), tuple(x.shape))


def mix_otimes(terms, x):
    """y = (sum_i c_i * A_i) ⨷ x without ever materialising the sum.

    The pattern of the reference's gradient test and of GroupCDL-style models (test/grad.jl:17-21,
    README.md:126-136): `C = α*A + (1-α)*B; y = C ⨷ x`.  There `C` is a third A-sized array that is
    written and read again; by linearity y = sum_i c_i * (A_i ⨷ x), so each A_i is read exactly once and
    only pixel-sized arrays are combined.  `terms` is a sequence of (c_i, A_i): c_i a number or an array
    of size (1, 1, h', b') as accepted by `scale` (src/array.jl:179-186); the A_i are Circulants of equal
    window and spatial size, 4-dimensional (multi-head, ⨷) or 3-dimensional (⊗).  Differentiable in the
    c_i, the A_i and x through the rrules of ⊗ / ⨷ (src/rrules.jl:58-72)."""
    terms = list(terms)
    if not terms:
        raise TypeError("mix_otimes needs at least one (c, A) term")
    out = None
    for c, A in terms:
        if not isinstance(A, Circulant):
            raise TypeError("terms are (c, A) with A a Circulant")
        terms[0][1]._same(A)
        mh = A.ndim == 4
        xr = splitheads(x, A.size(3)) if mh else x
        y = otimes(A, xr)                                   # (spatial..., c, heads*B): head fastest in the last dim
        if isinstance(c, torch.Tensor) and c.ndim > 0:
            if c.ndim != A.ndim or c.shape[0] != 1 or c.shape[1] != 1:
                raise TypeError(f"coefficient of size {tuple(c.shape)} does not scale the batch dims of A {tuple(A.shape)}")
            cb = c[0, 0].expand(*A.shape[2:])               # (heads, B) or (B,)
            cu = (cb.t() if cb.ndim == 2 else cb).reshape(-1)    # one value per unit, head fastest
            y = y * cu.reshape((1,) * (y.ndim - 1) + (-1,))
        else:
            y = y * float(c)
        y = jl.reshape(y, tuple(x.shape)) if mh else y
        out = y if out is None else out + y
    return out


class LazyAdjacency:
    """A linear combination sum_i c_i * adjacency(simfun_i, x_i, y_i) that is only written to memory when
    somebody looks at its values.

    `circulant_mh_adjacency(..., lazy=True)` / `circulant_adjacency(..., lazy=True)` return one term.  `c * A`,
    `A * c`, `A + B`, `A - B`, `-A` and `scale(c, A)` (c a number or an array of size (1, 1, h', b') as in
    src/array.jl:179-186) stay lazy.  Applying the result with `⨷` / `⊗` (Otimes / otimes /
    circulant_(mh_)attention(A, x)) evaluates sum_i c_i * (A_i applied to x) with the fused flash kernels,
    i.e. as attention with an unscaled similarity: neither the A_i nor their combination ever exist in memory.
    This is the pattern of the reference's gradient test and of GroupCDL-style models
    (test/grad.jl:17-21, 34-38, README.md:126-136), where the reference writes and re-reads three A-sized
    arrays.  Gradients flow to every x_i, y_i, c_i and to x through the fused pullback.
    `materialize()` (also taken by `.nzVal`, `.data` and `sum`) builds the ordinary Circulant."""

    def __init__(self, terms, W, nheads, spatial, batch, mh):
        self.terms = terms                # [(coefficient, simfun, x, y, normalizer)]
        self.kernel_length, self.nheads, self.spatial_size, self.batch, self.mh = int(W), int(nheads), spatial, batch, mh
        self._cache = None

    # -- algebra that stays lazy
    def _with(self, terms):
        return LazyAdjacency(terms, self.kernel_length, self.nheads, self.spatial_size, self.batch, self.mh)

    def _check(self, other):
        if not isinstance(other, LazyAdjacency):
            raise TypeError("a lazy adjacency combines with lazy adjacencies only: materialize() it first")
        if (other.kernel_length, other.nheads, other.spatial_size, other.batch, other.mh) != \
                (self.kernel_length, self.nheads, self.spatial_size, self.batch, self.mh):
            raise TypeError("Circulants must have equal window, spatial size and batch dims")

    @staticmethod
    def _times(c, d):
        return d if isinstance(c, (int, float)) and c == 1 else (c if isinstance(d, (int, float)) and d == 1 else c * d)

    def __mul__(self, c):
        if isinstance(c, torch.Tensor) and c.ndim > 0:
            if c.ndim != 4 or c.shape[0] != 1 or c.shape[1] != 1:
                raise TypeError(f"coefficient of size {tuple(c.shape)} does not scale the batch dims of A")
        return self._with([(self._times(c, term[0]),) + tuple(term[1:]) for term in self.terms])

    __rmul__ = __mul__

    def __neg__(self):
        return self * -1.0

    def __add__(self, other):
        self._check(other)
        return self._with(self.terms + other.terms)

    def __sub__(self, other):
        return self + (-other)

    # -- evaluation
    def _units_coeff(self, c, like):
        """coefficient as one value per unit (head fastest), broadcastable against (spatial..., c, units)"""
        if not (isinstance(c, torch.Tensor) and c.ndim > 0):
            return c
        cb = c[0, 0].expand(self.nheads, self.batch)            # (heads, B); a single-head adjacency has heads == 1
        cu = cb.t().reshape(-1)                                  # one value per unit, head fastest
        return cu.reshape((1,) * (like.ndim - 1) + (-1,))

    def apply(self, x):
        """sum_i c_i * (A_i ⨷ x) on the fused flash kernels (unscaled similarity: the adjacency has no 1/sqrt(c))."""
        xr = splitheads(x, self.nheads) if self.mh else x
        out = None
        for c, simfun, a, b, normalizer in self.terms:
            ar, br = (splitheads(t, self.nheads) for t in (a, b)) if self.mh else (a, b)
            y, _ = _AttentionFn.apply(ar, br, xr, _kind(simfun), self.kernel_length, normalizer, False, 1.0)
            cu = self._units_coeff(c, y)
            y = y * cu if not (isinstance(cu, (int, float)) and cu == 1) else y
            out = y if out is None else out + y
        return jl.reshape(out, tuple(x.shape)) if self.mh else out

    def materialize(self) -> "Circulant":
        if self._cache is None:
            out = None
            for c, simfun, a, b, normalizer in self.terms:
                A = (circulant_mh_adjacency(simfun, a, b, self.kernel_length, self.nheads, normalizer) if self.mh
                     else circulant_adjacency(simfun, a, b, self.kernel_length, normalizer))
                A = scale(c, A) if isinstance(c, torch.Tensor) and c.ndim > 0 else (A if c == 1 else c * A)
                out = A if out is None else out + A
            self._cache = out
        return self._cache

    @property
    def nzVal(self):
        return self.materialize().nzVal

    @property
    def data(self):
        return self.materialize().data

    @property
    def shape(self):
        Np = 1
        for n in self.spatial_size:
            Np *= n
        return (Np, Np, self.nheads, self.batch) if self.mh else (Np, Np, 1, self.batch)


class BatchedTranspose:
    """NNlib.batched_transpose(A::Circulant) marker (src/batchedmul.jl:13-19)."""

    def __init__(self, parent):
        self.parent = parent


def batched_transpose(A: Circulant):
    return BatchedTranspose(A)


batched_adjoint = batched_transpose      # values are real (src/array.jl:12-14)


def batched_mul(A, B):
    """NNlib.batched_mul(A, B) for a (transposed) Circulant and a dense (Np, c, batch)
    array (src/batchedmul.jl:13-41)."""
    transpose = isinstance(A, BatchedTranspose)
    Ac = A.parent if transpose else A
    Ar = Ac.reshape(Ac.shape[0], Ac.shape[1], -1)
    x = jl.reshape(B, Ac.spatial_size + tuple(B.shape[1:]))
    y = _ApplyFn.apply(Ar.nzVal, x, Ac.kernel_length, transpose)
    return jl.reshape(y, (B.shape[0],) + tuple(y.shape[len(Ac.spatial_size):]))


# ----------------------------------------------------------------- algebra, sums, cat
def scale(c, A: Circulant) -> Circulant:
    """scale(c, A): c of size (1, 1, h', b') (src/array.jl:179-186)."""
    if isinstance(A, LazyAdjacency):
        return A * c
    if not isinstance(c, torch.Tensor):
        return c * A                                                     # src/array.jl:187
    if c.ndim == 0:
        return float(c) * A
    if c.ndim < 3:
        raise TypeError(f"scale needs c of size (1, 1, batch...), got {tuple(c.shape)}")
    assert c.shape[0] == 1 and c.shape[1] == 1, "Scaling of non-batchdims of CuSparseArrayCSR not implemented"
    if c.ndim != A.ndim:
        raise TypeError(f"scale needs c and A with the same number of dims ({c.ndim} vs {A.ndim})")
    cb = jl.reshape(c, tuple(c.shape[2:]))
    return Circulant._from_nz(_ScaleFn.apply(cb, A.nzVal), A.kernel_length, A.spatial_size)


def dot(X: Circulant, Y: Circulant):
    """LinearAlgebra.dot (src/array.jl:83-85)."""
    X._same(Y)
    return ops.dot_batch(jl.reshape(X.nzVal, (-1,)), jl.reshape(Y.nzVal, (-1,)))[0]


def sum(A: Circulant, dims=None):
    """Base.sum(A::Circulant; dims) (src/array.jl:156-177); dims are 1-based."""
    if isinstance(A, LazyAdjacency):
        A = A.materialize()
    nz = A.nzVal
    if dims is None:
        return ops.dot_batch(jl.reshape(nz, (-1,)))[0]
    dims_t = (dims,) if isinstance(dims, int) else tuple(dims)
    if dims_t == (1,):
        return ops.sum_cols(nz, A.spatial_size, A.kernel_length)
    if dims_t == (2,):
        return ops.sum_rows(nz, A.spatial_size, A.kernel_length)
    if all(d > 2 for d in dims_t):
        out = ops.sum_batch(nz, 3 in dims_t, 4 in dims_t)
        return Circulant._from_nz(out, A.kernel_length, A.spatial_size)
    if dims_t == (1, 2):
        s = ops.dot_batch(nz)
        return jl.reshape(s, (1, 1) + tuple(nz.shape[1:]))
    raise RuntimeError(f"dims={dims} not implemented.")


def cat(*As: Circulant, dims=3) -> Circulant:
    """Base.cat(As...; dims) along a batch dim (README.md:145-148; the reference's
    method body, src/array.jl:62-64, names an undefined variable and throws)."""
    A0 = As[0]
    assert dims > 2, "only batch dims of a Circulant can be concatenated"
    for A in As[1:]:
        if A.kernel_length != A0.kernel_length or A.spatial_size != A0.spatial_size or A.ndim != A0.ndim:
            raise TypeError("cat needs Circulants with equal window, spatial size and ndims")
    axis = dims - 2                                                      # axis of nzVal
    nd = A0.nzVal.ndim
    rev = tuple(range(nd - 1, -1, -1))
    # CUDA.jl's `cat` on the value arrays: a library copy, not arithmetic
    out = torch.cat([jl.colmajor(A.nzVal).permute(rev) for A in As], dim=nd - 1 - axis).permute(rev)
    return Circulant._from_nz(out, A0.kernel_length, A0.spatial_size)
