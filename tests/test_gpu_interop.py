"""The CSR wire format of `Circulant.data` handed to another sparse library, and memory guards.

The reference hands rowPtr / colVal / nzVal to cuSPARSE's batched CSR SpMM (CUSPARSE.bmm!,
src/batchedmul.jl:82-90).  The first test does the equivalent here: the arrays produced by this
library (1-based Int32, replicated per batch slice) become one `torch.sparse_csr_tensor` per batch
slice, whose product with V (cuSPARSE underneath) must equal ca_apply.  Test-only use of that
library.  The second test places outputs and workspaces inside larger sentinel-filled buffers
and checks that nothing outside the requested region is written (a stand-in for a memory
checker at the shapes where tiles are ragged)."""
import numpy as np
import pytest
import torch

from tests.helpers import TOL, randn, rel_err

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("shape,ws,nheads", [((12, 10, 8, 2), 5, 2), ((33, 16, 1), 7, 1)])
def test_csr_arrays_feed_a_cusparse_spmm(ca, shape, ws, nheads):
    rng = np.random.default_rng(8)
    q, k, v = (ca.jl.from_numpy(randn(rng, shape)) for _ in range(3))
    if len(shape) == 4:
        y, A = ca.circulant_mh_attention(ca.DotSimilarity(), q, k, v, ws, nheads)
    else:
        y, A = ca.circulant_attention(ca.DotSimilarity(), q, k, v, ws)
    Np = int(np.prod(shape[:-2]))
    c = shape[-2] // nheads
    rowptr, colval, nzval = A.data.rowPtr, A.data.colVal, A.data.nzVal
    assert rowptr.dtype == torch.int32 and colval.dtype == torch.int32
    vr = ca.splitheads(v, nheads)                                   # (spatial..., c, nheads*B)
    V = ca.jl.reshape(vr, (Np, c, -1))
    got = ca.jl.reshape(y, (Np, c, -1)) if nheads == 1 else ca.jl.reshape(ca.splitheads(y, nheads), (Np, c, -1))
    rp = ca.jl.reshape(rowptr, (Np + 1, -1))
    cv = ca.jl.reshape(colval, (colval.shape[0], -1))
    nz = ca.jl.reshape(nzval, (nzval.shape[0], -1))
    for u in range(V.shape[-1]):
        crow = (rp[:, u] - 1).to(torch.int64).contiguous()          # the reference's arrays are 1-based
        col = (cv[:, u] - 1).to(torch.int64).contiguous()
        S = torch.sparse_csr_tensor(crow, col, nz[:, u].contiguous(), size=(Np, Np))
        want = S @ V[:, :, u].contiguous()
        err = float((got[:, :, u] - want).abs().max() / want.abs().max())
        assert err < 2 * TOL, (u, err)
        # every row's columns are ascending, as cuSPARSE's CSR routines expect
        cols2d = col.reshape(Np, -1)
        assert bool((cols2d[:, 1:] > cols2d[:, :-1]).all())


SENTINEL = 12345.678


def _guarded(ca, shape, dtype=torch.float32, pad=4096, fill=SENTINEL):
    """A column-major tensor of `shape` inside a larger buffer filled with a sentinel."""
    n = int(np.prod(shape))
    buf = torch.full((n + 2 * pad,), fill, dtype=dtype, device="cuda")
    view = buf[pad:pad + n].view(tuple(reversed(shape))).permute(tuple(range(len(shape) - 1, -1, -1)))
    return buf, view, pad, n


def _intact(buf, pad, n):
    return bool((buf[:pad] == SENTINEL).all()) and bool((buf[pad + n:] == SENTINEL).all())


@pytest.mark.parametrize("shape,ws,nheads", [((33, 15, 16, 1), 15, 1),      # ragged tile rows, extent == window
                                             ((37, 29, 64, 2), 9, 2),       # 32 channels per unit, ragged tiles
                                             ((272, 16, 1), 9, 1)])         # 1-D signal: sliding-tile kernels, no workspace
def test_outputs_and_workspaces_stay_inside_their_buffers(ca, shape, ws, nheads):
    lib, ops, jl = ca.lib, ca.ops, ca.jl
    rng = np.random.default_rng(9)
    q, k, v, dy = (ca.splitheads(jl.from_numpy(randn(rng, shape)), nheads) for _ in range(4))
    m = ops.meta_of(q, ws)
    d = m.desc(scale=1.0 / np.sqrt(m.channels))
    st = torch.cuda.current_stream().cuda_stream
    P = ops.ptr
    gy, y, py, ny = _guarded(ca, tuple(q.shape))
    gs, stats, ps, nst = _guarded(ca, (m.Np, m.units))
    nfw = lib.ca_attention_fwd_workspace(d, 0)
    assert nfw > 0 or len(shape) == 3                                # the 2-D shapes run on the tiled kernels
    gw, wsf, pw, nw = _guarded(ca, (nfw,), torch.uint8, fill=77)
    ca._lib.check(lib.ca_attention_fwd(d, P(q), P(k), P(v), P(y), None, P(stats), P(wsf), st))
    grads = [_guarded(ca, tuple(q.shape)) for _ in range(3)]
    nbw = lib.ca_attention_bwd_workspace(d, 0)
    gb, wsb, pb, nb = _guarded(ca, (nbw,), torch.uint8, fill=77)
    ca._lib.check(lib.ca_attention_bwd(d, P(q), P(k), P(v), P(y), P(dy), P(stats), None, None,
                                       P(grads[0][1]), P(grads[1][1]), P(grads[2][1]), P(wsb), P(wsf), st))
    torch.cuda.synchronize()
    assert _intact(gy, py, ny) and _intact(gs, ps, nst)
    assert bool((gw[:pw] == 77).all()) and bool((gw[pw + nw:] == 77).all())
    assert bool((gb[:pb] == 77).all()) and bool((gb[pb + nb:] == 77).all())
    for buf, view, pad, n in grads:
        assert _intact(buf, pad, n)
        assert bool(torch.isfinite(view).all()) and not bool((view == SENTINEL).any())
    assert not bool((y == SENTINEL).any())
