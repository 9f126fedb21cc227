"""The library's calls are capture-safe: a forward + backward through the public API recorded into a CUDA graph
replays to the same results as the eager call, also after new values were written into its static inputs."""
import numpy as np
import pytest
import torch

from tests.helpers import randn

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("shape,ws,nheads,norm", [((64, 48, 32, 2), 9, 2, "softmax"),      # tiled kernels, two streams in the backward
                                                  ((1500, 16, 2), 31, 2, "entmax"),       # 1-D kernels
                                                  ((40, 36, 32, 1), 7, 2, "entmax")])     # operator chain
def test_captured_step_replays_like_the_eager_call(ca, shape, ws, nheads, norm):
    rng = np.random.default_rng(31)
    nrm = ca.SOFTMAX if norm == "softmax" else ca.ENTMAX15
    first = [randn(rng, shape) for _ in range(4)]
    second = [randn(rng, shape) for _ in range(4)]
    q, k, v = (ca.jl.from_numpy(t).requires_grad_(True) for t in first[:3])
    r = ca.jl.from_numpy(first[3])

    def step():
        q.grad = k.grad = v.grad = None
        y, _ = ca.circulant_mh_attention(ca.DotSimilarity(), q, k, v, ws, nheads, normalizer=nrm, return_A=False)
        (y * r).sum().backward()
        return y

    def eager(vals):
        qe, ke, ve = (ca.jl.from_numpy(t).requires_grad_(True) for t in vals[:3])
        y, _ = ca.circulant_mh_attention(ca.DotSimilarity(), qe, ke, ve, ws, nheads, normalizer=nrm, return_A=False)
        (y * ca.jl.from_numpy(vals[3])).sum().backward()
        return [t.detach().clone() for t in (y, qe.grad, ke.grad, ve.grad)]

    graph, y = ca.capture(step)
    for vals in (first, second, first):
        with torch.no_grad():
            for dst, src in zip((q, k, v, r), vals):
                dst.copy_(ca.jl.from_numpy(src))
        graph.replay()
        torch.cuda.synchronize()
        want = eager(vals)
        for got, w in zip((y, q.grad, k.grad, v.grad), want):
            assert torch.equal(got, w)                # the same kernels on the same values: bit-identical
    ca.ops.check_status(q.device)


def test_nvtx_ranges_are_optional_and_harmless(ca):
    """NVTX ranges around the fused calls: off by default, switchable, results unchanged."""
    x = ca.jl.randn(64, 32, 16, 2)
    y0, _, _ = ca.ops.attention_fwd(0, 0, x, x, x, 7, False)
    assert ca.ops.enable_nvtx(True) is False
    try:
        y1, _, _ = ca.ops.attention_fwd(0, 0, x, x, x, 7, False)
    finally:
        assert ca.ops.enable_nvtx(False) is True
    assert torch.equal(y0, y1)
