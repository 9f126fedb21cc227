"""Parity of the CUDA library (through the C ABI) with the CPU oracle on the
same seeded inputs.  Bar: bit-exact CSR structure; y, A and gradients within
1e-5 relative (to the tensor's largest magnitude) for Float32 / ComplexF32."""
import numpy as np
import pytest
import torch

from oracle import circatt_oracle as orc
from tests.helpers import KIND, TOL, assert_close, randn, rel_err, up

pytestmark = pytest.mark.gpu


def sim_of(ca, name):
    return ca.DotSimilarity() if name == "dot" else ca.DistanceSimilarity()


# ------------------------------------------------------------------ structure (bit exact)
@pytest.mark.parametrize("spatial,ws,batch", [
    ((8,), 5, (1, 2)), ((8, 8), 5, (1, 2)), ((5, 5), 5, (2, 1)), ((7, 9), 7, (1, 1)), ((12, 6), 5, (3, 2)),
    ((32, 32), 7, (1, 1)), ((31,), 9, (1, 3)), ((10, 10), 3, (2, 2)), ((128, 96), 15, (1, 1)),
])
def test_structure_bit_exact(ca, spatial, ws, batch):
    rowptr, colval = ca.ops.structure(spatial, ws, batch, "cuda")
    rp, cv = orc.structure(spatial, ws)
    got_rp, got_cv = ca.jl.to_numpy(rowptr), ca.jl.to_numpy(colval)
    assert got_rp.dtype == np.int32 and got_cv.dtype == np.int32
    assert got_rp.shape == (len(rp),) + batch and got_cv.shape == (len(cv),) + batch
    for idx in np.ndindex(*batch):
        assert np.array_equal(got_rp[(slice(None),) + idx], rp)
        assert np.array_equal(got_cv[(slice(None),) + idx], cv)


def test_structure_matches_literal_reference_index_function(ca):
    _, colval = ca.ops.structure((9, 7), 5, (1, 1), "cuda")
    assert np.array_equal(ca.jl.to_numpy(colval)[:, 0, 0], orc.structure_literal((9, 7), 5))


# ------------------------------------------------------------------ fused attention
CASES = [
    # (shape (spatial..., C, B), ws, nheads, cplx)
    ((32, 32, 16, 1), 7, 1, False),      # BASELINE config 1
    ((8, 8, 4, 2), 5, 1, False),         # reference test/rrule.jl shapes
    ((8, 4, 2), 5, 1, False),
    ((8, 8, 4, 2), 5, 1, True),
    ((8, 4, 2), 5, 1, True),
    ((10, 10, 8, 2), 3, 2, False),       # reference test/grad.jl shapes
    ((10, 8, 2), 3, 2, True),
    ((7, 7, 3, 1), 7, 1, False),         # extent == window: every row wraps on both sides
    ((8, 7, 5, 2), 7, 1, False),         # extent == window + 1
    ((13, 11, 6, 3), 5, 3, False),       # prime extents, odd channels per head
    ((37, 29, 32, 2), 9, 2, False),      # 16 channels per head, ragged tiles
    ((64, 48, 64, 1), 15, 4, False),     # quarter-size BASELINE config 2
    ((40, 6, 2), 13, 2, True),
    ((300, 16, 2), 31, 2, False),        # long 1-D window
    ((20, 20, 33, 1), 5, 1, False),      # 33 channels: 64-wide register path
    ((24, 20, 20, 2), 7, 1, True),       # 40 real channels
    ((40, 21, 16, 2), 7, 2, True),       # 8 complex = 16 real channels per head: tiled kernels, complex loads
    ((128, 24, 16, 1), 21, 1, False),    # window 21, full-height tile
    ((33, 9, 16, 1), 9, 1, False),       # ragged tile rows, extent == window along w
    ((50, 18, 32, 1), 11, 2, False),
    ((48, 16, 16, 2), 13, 1, False),
    ((16, 17, 16, 1), 3, 1, False),
    ((37, 29, 64, 2), 9, 2, False),      # 32 channels per head: chain of tiled operators with scratch scores
    ((24, 20, 32, 2), 5, 1, True),       # 32 complex = 64 real channels (BASELINE config 4's channel count)
    ((33, 16, 64, 1), 7, 1, False),      # 64 real channels
    ((256, 16, 2), 9, 1, False),         # 1-D, 16 channels: fused kernels on the folded signal (two columns)
    ((384, 32, 1), 33, 2, False),        # 1-D folded into three columns, window wider than a staging piece
    ((512, 16, 1), 127, 1, False),       # 1-D, the widest window the folded kernels take
    ((16, 16, 2), 15, 1, False),         # shortest 1-D signal, every row wraps
    ((16, 15, 16, 1), 15, 1, False),     # shortest 2-D image, extent == window along w
    ((37, 29, 16, 2), 9, 2, False),      # 8 channels per head: fused kernels on zero-extended units
    ((40, 21, 8, 2), 7, 2, True),        # 4 complex = 8 real channels per head
    ((256, 16, 2), 9, 2, False),         # 1-D, 8 channels per head
    ((40, 34, 64, 1), 15, 2, False),     # 32 channels per head, window 15: unchecked chunks of 5 keys
    ((44, 40, 64, 1), 21, 1, False),     # 64 channels per head, window 21: unchecked chunks of 7 keys
    ((32, 30, 32, 1), 29, 1, False),     # 32 channels per unit, window 29: wide units on the fused kernels
    ((34, 33, 64, 1), 31, 1, False),     # 64 channels per unit, window 31
    ((128, 32, 2), 33, 1, False),        # 1-D, 32 channels per unit
]


@pytest.mark.parametrize("simname", ["dot", "distance"])
@pytest.mark.parametrize("shape,ws,nheads,cplx", CASES)
def test_attention_forward_backward(ca, shape, ws, nheads, cplx, simname):
    rng = np.random.default_rng(0)
    qn, kn, vn, rn = (randn(rng, shape, cplx) for _ in range(4))
    q, k, v = (ca.jl.from_numpy(t).requires_grad_(True) for t in (qn, kn, vn))
    y, A = ca.circulant_mh_attention(sim_of(ca, simname), q, k, v, ws, nheads)
    B = shape[-1]
    Np = int(np.prod(shape[:-2]))
    assert tuple(y.shape) == shape and A.shape == (Np, Np, nheads, B)
    r = ca.jl.from_numpy(rn)
    loss = (y * r.conj()).real.sum() if cplx else (y * r).sum()
    loss.backward()

    yo, nzo = orc.mh_attention(KIND[simname], up(qn), up(kn), up(vn), ws, nheads)
    dqo, dko, dvo = orc.mh_attention_pullback(KIND[simname], up(qn), up(kn), up(vn), ws, nheads, up(rn))
    assert_close(ca.jl.to_numpy(y), yo, "y")
    assert_close(ca.jl.to_numpy(A.nzVal), nzo, "A")
    assert_close(ca.jl.to_numpy(q.grad), dqo, "dq")
    assert_close(ca.jl.to_numpy(k.grad), dko, "dk")
    assert_close(ca.jl.to_numpy(v.grad), dvo, "dv")


@pytest.mark.parametrize("simname", ["dot", "distance"])
def test_flash_mode_equals_materialised(ca, simname):
    """return_A=False never writes A; y and gradients agree with the materialising path
    (different kernels, so to rounding, not to the bit)."""
    rng = np.random.default_rng(1)
    shape = (24, 20, 32, 2)
    qn, kn, vn, rn = (randn(rng, shape) for _ in range(4))
    outs = []
    for want in (True, False):
        q, k, v = (ca.jl.from_numpy(t).requires_grad_(True) for t in (qn, kn, vn))
        y, A = ca.circulant_mh_attention(sim_of(ca, simname), q, k, v, 7, 2, return_A=want)
        assert (A is None) == (not want)
        (y * ca.jl.from_numpy(rn)).sum().backward()
        outs.append([ca.jl.to_numpy(t) for t in (y, q.grad, k.grad, v.grad)])
    for a, b in zip(*outs):
        assert rel_err(a, b.astype(np.float64)) < TOL


@pytest.mark.parametrize("shape,ws,nheads", [((12, 10, 8, 2), 5, 2), ((20, 12, 64, 2), 5, 2), ((40, 24, 16, 2), 7, 1),
                                             ((32, 30, 32, 1), 29, 1), ((34, 33, 64, 1), 31, 1)])
def test_cotangent_on_returned_A(ca, shape, ws, nheads):
    """Loss uses both y and A (e.g. sparsity penalties): dA flows into the fused backward."""
    rng = np.random.default_rng(2)
    qn, kn, vn, rn = (randn(rng, shape) for _ in range(4))
    q, k, v = (ca.jl.from_numpy(t).requires_grad_(True) for t in (qn, kn, vn))
    y, A = ca.circulant_mh_attention(ca.DistanceSimilarity(), q, k, v, ws, nheads)
    dAn = np.asfortranarray(rng.standard_normal(tuple(A.nzVal.shape)).astype(np.float32))
    ((y * ca.jl.from_numpy(rn)).sum() + (A.nzVal * ca.jl.from_numpy(dAn)).sum()).backward()
    K = ws * ws
    dA64 = dAn.astype(np.float64).reshape((K, shape[0] * shape[1], nheads * shape[-1]), order="F")
    dqo, dko, dvo = orc.mh_attention_pullback(orc.DISTANCE, up(qn), up(kn), up(vn), ws, nheads, up(rn), dA64)
    assert rel_err(ca.jl.to_numpy(q.grad), dqo) < TOL
    assert rel_err(ca.jl.to_numpy(k.grad), dko) < TOL
    assert rel_err(ca.jl.to_numpy(v.grad), dvo) < TOL


@pytest.mark.parametrize("simname", ["dot", "distance"])
@pytest.mark.parametrize("shape,ws,nheads", [((37, 29, 32, 2), 9, 2), ((64, 48, 64, 1), 15, 4), ((256, 16, 2), 9, 1),
                                             ((40, 24, 16, 2), 7, 2)])
def test_bfloat16_storage(ca, shape, ws, nheads, simname):
    """BFloat16 tensors in and out, Float32 arithmetic (no reference counterpart).  The oracle runs in
    float64 on the bfloat16-rounded inputs, so the differences are Float32 accumulation, the final rounding
    of the outputs to bfloat16 (half an ulp = 2^-9 of each value) and, in the backward, the bfloat16-rounded
    y that was saved by the forward: bar 1e-2 of the largest value."""
    import torch
    BF16_TOL = 1e-2
    rng = np.random.default_rng(11)
    qn, kn, vn, rn = (randn(rng, shape) for _ in range(4))
    to_bf = lambda a: ca.jl.from_numpy(a).to(torch.bfloat16)
    q, k, v, r = (to_bf(t) for t in (qn, kn, vn, rn))
    back = lambda t: ca.jl.to_numpy(t.float()).astype(np.float64)
    q64, k64, v64, r64 = (back(t) for t in (q, k, v, r))
    q, k, v = (t.requires_grad_(True) for t in (q, k, v))
    n0 = ca._lib.lib.ca_probe_tiled_launch_count()
    y, A = ca.circulant_mh_attention(sim_of(ca, simname), q, k, v, ws, nheads)
    (y.float() * r.float()).sum().backward()
    assert ca._lib.lib.ca_probe_tiled_launch_count() > n0
    assert y.dtype == torch.bfloat16 and q.grad.dtype == torch.bfloat16 and A.nzVal.dtype == torch.float32
    yo, nzo = orc.mh_attention(KIND[simname], q64, k64, v64, ws, nheads)
    dqo, dko, dvo = orc.mh_attention_pullback(KIND[simname], q64, k64, v64, ws, nheads, r64)
    assert rel_err(back(y), yo) < BF16_TOL
    assert rel_err(ca.jl.to_numpy(A.nzVal), nzo) < TOL                 # A stays Float32
    assert rel_err(back(q.grad), dqo) < BF16_TOL
    assert rel_err(back(k.grad), dko) < BF16_TOL
    assert rel_err(back(v.grad), dvo) < BF16_TOL


def test_bfloat16_is_refused_outside_the_fused_kernels(ca):
    import torch
    x = ca.jl.randn(16, 16, 4, 1).to(torch.bfloat16)
    with pytest.raises(ca._lib.CircAttError, match="bfloat16"):
        ca.ops.similarity(0, x, x, 5)
    with pytest.raises(ca._lib.CircAttError, match="bfloat16"):
        ca.ops.attention_fwd(0, 0, x, x, x, 5, False)                 # 4 channels per unit: no tiled kernel


@pytest.mark.parametrize("shape,nheads", [((256, 32, 2), 2), ((256, 32, 2), 4), ((40, 24, 32, 1), 4)])
def test_folded_1d_and_narrow_units_run_on_the_fused_tiled_kernels(ca, shape, nheads):
    """1-D signals and units of 16 or 8 channels per head take the TMA-tiled forward and backward (pack, fwd,
    pack, dq, dk/dv), not the generic kernels."""
    rng = np.random.default_rng(12)
    q, k, v = (ca.jl.from_numpy(randn(rng, shape)).requires_grad_(True) for _ in range(3))
    lib = ca._lib.lib
    n0 = lib.ca_probe_tiled_launch_count()
    y, _ = ca.circulant_mh_attention(ca.DotSimilarity(), q, k, v, 9, nheads, return_A=False)
    assert lib.ca_probe_tiled_launch_count() == n0 + 1
    y.sum().backward()
    assert lib.ca_probe_tiled_launch_count() == n0 + 3


def test_large_scores_running_max(ca):
    """Inputs scaled x30: scores in the hundreds; exercises the online-softmax rescale."""
    rng = np.random.default_rng(3)
    shape = (16, 16, 16, 1)
    qn, kn, vn = (randn(rng, shape, scale=30.0) for _ in range(3))
    q, k, v = (ca.jl.from_numpy(t) for t in (qn, kn, vn))
    y, A = ca.circulant_attention(q, k, v, 7)
    yo, nzo = orc.attention(orc.DOT, up(qn), up(kn), up(vn), 7)
    assert np.isfinite(ca.jl.to_numpy(y)).all()
    # scores ~ 1e3, so one float32 ulp of a score is ~1e-4 relative in exp(): looser bar, stated here
    assert rel_err(ca.jl.to_numpy(y), yo) < 2e-3
    assert rel_err(ca.jl.to_numpy(A.nzVal), nzo) < 2e-3


def test_deterministic_gradients(ca):
    rng = np.random.default_rng(4)
    shape = (40, 33, 32, 2)
    qn, kn, vn, rn = (randn(rng, shape) for _ in range(4))
    runs = []
    for _ in range(2):
        q, k, v = (ca.jl.from_numpy(t).requires_grad_(True) for t in (qn, kn, vn))
        y, _ = ca.circulant_mh_attention(ca.DotSimilarity(), q, k, v, 9, 2, return_A=False)
        (y * ca.jl.from_numpy(rn)).sum().backward()
        runs.append([ca.jl.to_numpy(t) for t in (y, q.grad, k.grad, v.grad)])
    for a, b in zip(*runs):
        assert np.array_equal(a, b)


# ------------------------------------------------------------------ entmax (no reference counterpart)
@pytest.mark.parametrize("want_A", [True, False])
@pytest.mark.parametrize("shape,ws,nheads,simname", [((64, 16, 2), 15, 2, "distance"), ((12, 11, 8, 1), 5, 2, "dot"),
                                                     ((40, 24, 32, 1), 7, 2, "distance"), ((40, 24, 32, 1), 7, 2, "dot"),
                                                     ((2048, 32, 2), 127, 4, "distance"),      # config 3's window and head size
                                                     ((37, 29, 16, 1), 9, 1, "dot")])
def test_entmax_attention(ca, shape, ws, nheads, simname, want_A):
    rng = np.random.default_rng(5)
    qn, kn, vn, rn = (randn(rng, shape, scale=1.5) for _ in range(4))
    q, k, v = (ca.jl.from_numpy(t).requires_grad_(True) for t in (qn, kn, vn))
    y, A = ca.circulant_mh_attention(sim_of(ca, simname), q, k, v, ws, nheads, normalizer=ca.ENTMAX15, return_A=want_A)
    (y * ca.jl.from_numpy(rn)).sum().backward()
    yo, nzo = orc.mh_attention(KIND[simname], up(qn), up(kn), up(vn), ws, nheads, orc.ENTMAX15)
    dqo, dko, dvo = orc.mh_attention_pullback(KIND[simname], up(qn), up(kn), up(vn), ws, nheads, up(rn),
                                              norm=orc.ENTMAX15)
    assert (nzo == 0).any()
    assert rel_err(ca.jl.to_numpy(y), yo) < TOL
    if want_A:
        assert rel_err(ca.jl.to_numpy(A.nzVal), nzo) < TOL
    assert rel_err(ca.jl.to_numpy(q.grad), dqo) < 2 * TOL
    assert rel_err(ca.jl.to_numpy(k.grad), dko) < 2 * TOL
    assert rel_err(ca.jl.to_numpy(v.grad), dvo) < TOL


# ------------------------------------------------------------------ the unfused pieces and their rrules
@pytest.mark.parametrize("cplx", [False, True])
@pytest.mark.parametrize("simname", ["dot", "distance"])
@pytest.mark.parametrize("spatial", [(8,), (8, 8), (11, 7)])
def test_similarity_and_pullback(ca, spatial, simname, cplx):
    """test/rrule.jl:18-19 shapes (8 / 8x8, 4 channels, batch 2, ws 5)."""
    rng = np.random.default_rng(6)
    shape, ws = spatial + (4, 2), 5
    xn, yn = randn(rng, shape, cplx), randn(rng, shape, cplx)
    x, y = (ca.jl.from_numpy(t).requires_grad_(True) for t in (xn, yn))
    S = ca.circulant_similarity(sim_of(ca, simname), x, y, ws)
    Np = int(np.prod(spatial))
    assert S.shape == (Np, Np, 1, 2)
    So = orc.similarity(KIND[simname], up(xn), up(yn), ws)
    assert rel_err(ca.jl.to_numpy(S.nzVal), So) < TOL
    dSn = rng.standard_normal(So.shape).astype(np.float32)
    (S.nzVal * ca.jl.from_numpy(np.asfortranarray(dSn.reshape(tuple(S.nzVal.shape), order="F")))).sum().backward()
    dxo, dyo = orc.similarity_pullback(KIND[simname], up(xn), up(yn), ws, dSn.astype(np.float64))
    assert rel_err(ca.jl.to_numpy(x.grad), dxo) < TOL
    assert rel_err(ca.jl.to_numpy(y.grad), dyo) < TOL


@pytest.mark.parametrize("norm", ["softmax", "entmax"])
def test_row_normalize_and_pullback(ca, norm):
    """test/rrule.jl:21."""
    rng = np.random.default_rng(7)
    spatial, ws = (9, 8), 5
    A = ca.Circulant(ws, spatial + (2, 3))
    nzn = np.asfortranarray((2.0 * rng.standard_normal(tuple(A.nzVal.shape))).astype(np.float32))
    A.data.nzVal = ca.jl.from_numpy(nzn).requires_grad_(True)
    nrm = ca.SOFTMAX if norm == "softmax" else ca.ENTMAX15
    P = ca.softmax(A, normalizer=nrm)
    onorm = orc.SOFTMAX if norm == "softmax" else orc.ENTMAX15
    nz64 = nzn.astype(np.float64).reshape((25, 72, 2, 3), order="F")
    Po = orc.row_normalize(onorm, nz64)
    assert rel_err(ca.jl.to_numpy(P.nzVal), Po) < TOL
    dPn = np.asfortranarray(rng.standard_normal(nzn.shape).astype(np.float32))
    (P.nzVal * ca.jl.from_numpy(dPn)).sum().backward()
    dSo = orc.row_normalize_pullback(onorm, Po, dPn.astype(np.float64).reshape(Po.shape, order="F"))
    assert rel_err(ca.jl.to_numpy(A.nzVal.grad), dSo) < TOL
    # in-place form
    B = ca.Circulant._from_nz(ca.jl.from_numpy(nzn), ws, spatial)
    ca.softmax_(B, normalizer=nrm)
    assert rel_err(ca.jl.to_numpy(B.nzVal), Po) < TOL


@pytest.mark.parametrize("cplx", [False, True])
@pytest.mark.parametrize("transpose", [False, True])
@pytest.mark.parametrize("spatial", [(8,), (8, 8), (9, 12)])
def test_apply_and_pullback(ca, spatial, transpose, cplx):
    """test/rrule.jl:20 (and the transposed apply, which the reference does not test)."""
    rng = np.random.default_rng(8)
    ws, c, B = 5, 4, 2
    A = ca.Circulant(ws, spatial + (1, B))
    nzn = np.asfortranarray(rng.standard_normal(tuple(A.nzVal.shape)).astype(np.float32))
    A.data.nzVal = ca.jl.from_numpy(nzn).requires_grad_(True)
    bn, dcn = randn(rng, spatial + (c, B), cplx), randn(rng, spatial + (c, B), cplx)
    b = ca.jl.from_numpy(bn).requires_grad_(True)
    out = ca.circulant_transposed_attention(A, b) if transpose else ca.otimes(A, b)
    K, Np = ws ** len(spatial), int(np.prod(spatial))
    nz64 = nzn.astype(np.float64).reshape((K, Np, B), order="F")
    oo = orc.apply(nz64, up(bn), ws, transpose)
    assert rel_err(ca.jl.to_numpy(out), oo) < TOL
    dc = ca.jl.from_numpy(dcn)
    ((out * dc.conj()).real.sum() if cplx else (out * dc).sum()).backward()
    if not transpose:
        dAo, dbo = orc.apply_pullback(nz64, up(bn), ws, up(dcn))
    else:
        dAo = orc.similarity(orc.DOT, up(bn), up(dcn), ws)
        dbo = orc.apply(nz64, up(dcn), ws, False)
    assert rel_err(ca.jl.to_numpy(A.nzVal.grad), dAo) < TOL
    assert rel_err(ca.jl.to_numpy(b.grad), dbo) < TOL


TILED_OPERATOR_CASES = [
    # (spatial, ws, channels, units, cplx): 16 real channels per unit -> the TMA-tiled operator kernels
    ((37, 29), 9, 16, 2, False),        # ragged tiles
    ((40, 21), 7, 8, 2, True),          # 8 complex channels
    ((16, 9), 9, 16, 1, False),         # smallest tile, extent == window along w
    ((128, 24), 21, 16, 1, False),      # full-height tile, window 21
    ((70, 10), 5, 16, 3, False),        # three warps of rows, W not a multiple of the four-column tile
    ((64, 48), 15, 16, 4, False),       # quarter-size BASELINE config 2
    ((37, 29), 9, 32, 2, False),        # 32 real channels: two lanes per pixel
    ((33, 12), 7, 16, 2, True),         # 16 complex channels
    ((24, 20), 5, 64, 2, False),        # 64 real channels: four lanes per pixel
    ((40, 21), 7, 32, 1, True),         # 32 complex channels (BASELINE config 4's channel count)
    ((16, 16), 3, 64, 3, False),        # smallest window, two warps of rows
    ((40, 24), 7, 8, 2, False),         # 8 channels per unit: zero-extended to one slab
    ((64, 40), 35, 16, 1, False),       # window wider than the 32-row staging chunk
    ((256,), 9, 16, 2, False),          # 1-D signal, folded into 128-row columns
    ((384,), 33, 8, 3, False),          # 1-D, 8 channels, three columns, chunked window
    ((4096,), 127, 8, 2, False),        # BASELINE config 3's window and channel count
    ((96,), 5, 16, 1, True),            # 1-D that folds into a single column (wraps onto itself)
    ((64,), 7, 64, 2, False),           # 1-D, four lanes per pixel
    ((16,), 15, 16, 2, False),          # shortest 1-D signal, window = extent - 1: every row wraps
    ((48,), 31, 16, 1, False),          # one 48-row column
    ((16, 15), 15, 16, 1, False),       # shortest 2-D image, extent == window along w
]


@pytest.mark.parametrize("simname", ["dot", "distance"])
@pytest.mark.parametrize("spatial,ws,c,units,cplx", TILED_OPERATOR_CASES)
def test_tiled_similarity_and_pullback(ca, spatial, ws, c, units, cplx, simname):
    """R3/R4 and their rrules (src/similarity.jl:55-103, src/rrules.jl:1-32) on the tiled kernels."""
    rng = np.random.default_rng(21)
    shape = spatial + (c, units)
    xn, yn = randn(rng, shape, cplx), randn(rng, shape, cplx)
    x, y = ca.jl.from_numpy(xn), ca.jl.from_numpy(yn)
    m = ca.ops.meta_of(x, ws)
    assert ca._lib.lib.ca_operator_workspace(m.desc()) > 0           # the shape is covered by the tiled kernels
    scale = 0.37
    lib = ca._lib.lib
    n0 = lib.ca_probe_tiled_launch_count()
    S = ca.ops.similarity(KIND[simname], x, y, ws, scale)
    assert lib.ca_probe_tiled_launch_count() == n0 + 1               # ... and ran on them
    So = scale * orc.similarity(KIND[simname], up(xn), up(yn), ws)
    assert rel_err(ca.jl.to_numpy(S), So.reshape(S.shape, order="F")) < TOL
    dSn = np.asfortranarray(rng.standard_normal(tuple(S.shape)).astype(np.float32))
    dx, dy = ca.ops.similarity_bwd(KIND[simname], x, y, ws, ca.jl.from_numpy(dSn), scale)
    assert lib.ca_probe_tiled_launch_count() == n0 + 3               # one plain and one transposed apply
    dxo, dyo = orc.similarity_pullback(KIND[simname], up(xn), up(yn), ws,
                                       scale * dSn.astype(np.float64).reshape(So.shape, order="F"))
    assert rel_err(ca.jl.to_numpy(dx), dxo) < TOL
    assert rel_err(ca.jl.to_numpy(dy), dyo) < TOL


@pytest.mark.parametrize("transpose", [False, True])
@pytest.mark.parametrize("spatial,ws,c,units,cplx", TILED_OPERATOR_CASES)
def test_tiled_apply(ca, spatial, ws, c, units, cplx, transpose):
    """R6 (src/batchedmul.jl:82-150 as used by src/attention.jl:53-80) on the tiled kernels."""
    rng = np.random.default_rng(22)
    K, Np = ws ** len(spatial), int(np.prod(spatial))
    nzn = np.asfortranarray(rng.standard_normal((Np * K, units)).astype(np.float32))
    vn = randn(rng, spatial + (c, units), cplx)
    n0 = ca._lib.lib.ca_probe_tiled_launch_count()
    out = ca.ops.apply(ca.jl.from_numpy(nzn), ca.jl.from_numpy(vn), ws, transpose)
    assert ca._lib.lib.ca_probe_tiled_launch_count() == n0 + 1       # the tiled kernel ran, not the generic one
    oo = orc.apply(nzn.astype(np.float64).reshape((K, Np, units), order="F"), up(vn), ws, transpose)
    assert rel_err(ca.jl.to_numpy(out), oo) < TOL


def test_readme_identity_and_mh_apply(ca):
    """README.md:115-119: softmax(S) ⊗ v ≈ y, and A ⨷ v ≈ y for the multi-head A."""
    rng = np.random.default_rng(9)
    shape, ws, nheads = (16, 12, 8, 2), 5, 2
    q, k, v = (ca.jl.from_numpy(randn(rng, shape)) for _ in range(3))
    y, A = ca.circulant_attention(ca.DistanceSimilarity(), q, k, v, ws)
    t = float(np.sqrt(shape[2]))
    S = ca.circulant_similarity(ca.DistanceSimilarity(), q / np.sqrt(t), k / np.sqrt(t), ws)
    u = ca.otimes(ca.softmax(S), v)
    assert rel_err(ca.jl.to_numpy(u), ca.jl.to_numpy(y).astype(np.float64)) < TOL
    ym, Am = ca.circulant_mh_attention(ca.DotSimilarity(), q, k, v, ws, nheads)
    um = ca.Otimes(Am, v)
    assert rel_err(ca.jl.to_numpy(um), ca.jl.to_numpy(ym).astype(np.float64)) < TOL
    ut = ca.circulant_mh_transposed_attention(Am, v)
    nz64 = ca.jl.to_numpy(Am.nzVal).astype(np.float64).reshape((25, 192, 4), order="F")
    uo = orc.apply(nz64, orc.splitheads(up(ca.jl.to_numpy(v)), nheads), ws, True)
    assert rel_err(ca.jl.to_numpy(ut), uo) < TOL


def test_no_stage_copy_timed_out(ca):
    """Every device-side wait is bounded; a healthy run never hits the bound."""
    import ctypes
    n = ctypes.c_int32(-1)
    assert ca.lib.ca_stage_timeouts(ctypes.byref(n)) == 0
    # only the self test of the bounded wait (tests/test_gpu_timeout.py) may have bumped the counter
    assert n.value == getattr(ca.ops, "probe_timeouts_provoked", 0)
