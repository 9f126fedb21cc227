"""The allocation-free forward, ca_attention_fwd_static.

Some callers of the library are not allowed to allocate device memory where
they need the forward pass (they live inside another component's memory pool,
or run with a fixed memory budget).  For them the library carries its own
fixed scratch array.  This test calls that entry point through the C ABI,
twice in a row (the array is shared and keeps the previous call's contents),
and checks y and the row statistics against the ordinary entry point, which
is given a caller-allocated workspace, and against the float64 oracle; it also
checks that the device's free memory is the same before and after the calls
(nothing was allocated).  The file name makes pytest collect it last, so a
failure here cannot hide the result of any other test."""
import ctypes

import numpy as np
import pytest
import torch

from oracle import circatt_oracle as orc
from tests.helpers import TOL, randn, rel_err, up

pytestmark = pytest.mark.gpu


def _run(ca, entry, d, q, k, v, with_workspace):
    lib, ops, jl = ca.lib, ca.ops, ca.jl
    y = jl.empty(q.shape, q.dtype, q.device)
    stats = jl.empty((q.shape[0] * q.shape[1], q.shape[-1]), torch.float32, q.device)
    stream = torch.cuda.current_stream().cuda_stream
    if with_workspace:
        nbytes = lib.ca_attention_fwd_workspace(d, 0)
        ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=q.device)
        rc = entry(d, ops.ptr(q), ops.ptr(k), ops.ptr(v), ops.ptr(y), None, ops.ptr(stats), ops.ptr(ws), stream)
    else:
        rc = entry(d, ops.ptr(q), ops.ptr(k), ops.ptr(v), ops.ptr(y), None, ops.ptr(stats), stream)
    assert rc == 0, ca.lib.ca_last_error().decode()
    torch.cuda.synchronize()
    return jl.to_numpy(y), jl.to_numpy(stats)


@pytest.mark.parametrize("simname", ["dot", "distance"])
def test_static_scratch_forward_matches_workspace_forward(ca, simname):
    rng = np.random.default_rng(0)
    lib, ops, jl = ca.lib, ca.ops, ca.jl
    ws = 7
    shapes = [(48, 20, 16, 3), (33, 12, 16, 2)]          # two different problems share the one array
    for shape in shapes:
        qn, kn, vn = (randn(rng, shape) for _ in range(3))
        q, k, v = (jl.from_numpy(t) for t in (qn, kn, vn))
        kind = orc.DISTANCE if simname == "distance" else orc.DOT
        y_orc, _ = orc.attention(kind, up(qn), up(kn), up(vn), ws)
        r4 = float(shape[-2]) ** 0.25
        lse_orc = orc.row_logsumexp(orc.similarity(kind, up(qn) / r4, up(kn) / r4, ws))
        m = ops.meta_of(q, ws)
        d = m.desc(similarity=1 if simname == "distance" else 0, normalizer=0, scale=1.0 / np.sqrt(m.channels))
        assert 0 < lib.ca_attention_fwd_workspace(d, 0) <= lib.ca_static_scratch_bytes()
        y_ref, s_ref = _run(ca, lib.ca_attention_fwd, d, q, k, v, True)
        _run(ca, lib.ca_attention_fwd_static, d, q, k, v, False)    # first call on the device: address set-up
        free_before, _ = torch.cuda.mem_get_info()
        for _ in range(2):                               # second call sees the first call's leftovers
            y, s = _run(ca, lib.ca_attention_fwd_static, d, q, k, v, False)
            assert rel_err(y, y_ref.astype(np.float64)) < TOL
            assert rel_err(s, s_ref.astype(np.float64)) < TOL
            assert rel_err(y, y_orc) < TOL               # and against the float64 oracle itself
            assert rel_err(s, lse_orc) < TOL
        # outputs of _run come from torch's caching allocator, whose pool already holds blocks of these
        # sizes after the warm-up call: the driver-level free memory must not have moved
        free_after, _ = torch.cuda.mem_get_info()
        assert free_after == free_before


def test_static_scratch_rejects_oversized_problems(ca):
    lib, ops = ca.lib, ca.ops
    m = ops.Meta((1024, 1024), 16, 128, 21, False)       # BASELINE config 5: far beyond 64 MiB
    d = m.desc(scale=0.25)
    assert lib.ca_attention_fwd_workspace(d, 0) > lib.ca_static_scratch_bytes()
    one = ctypes.c_void_p(256)                            # never dereferenced: the size check comes first
    rc = lib.ca_attention_fwd_static(d, one, one, one, one, None, None, None)
    assert rc == -5
    assert "built-in scratch array" in lib.ca_last_error().decode()
