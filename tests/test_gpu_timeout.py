"""The bounded device-side waits and their failure reporting.

Every wait in the library's kernels has an iteration limit.  This test makes one run out on
purpose through the self-test entry ca_probe_stage_timeout (a one-block kernel whose stage
barrier expects more bytes than its copy delivers): the block must give up after the requested
number of polls, report through the same counter and status word as the tiled kernels, and
return; the process must keep working afterwards.  Nothing here faults, traps or hangs."""
import ctypes

import numpy as np
import pytest
import torch

from oracle import circatt_oracle as orc
from tests.helpers import TOL, randn, rel_err, up

pytestmark = pytest.mark.gpu


def _timeouts(lib):
    n = ctypes.c_int32(-1)
    assert lib.ca_stage_timeouts(ctypes.byref(n)) == 0
    return n.value


def test_wait_that_runs_out_is_reported_and_the_process_keeps_working(ca):
    lib, ops, jl = ca.lib, ca.ops, ca.jl
    dev = torch.device("cuda", torch.cuda.current_device())
    before = _timeouts(lib)
    status = ops._status_word(dev)           # registers the word for this host thread
    status.zero_()
    out = torch.full((1,), -1, dtype=torch.int32, device=dev)
    rc = lib.ca_probe_stage_timeout(64, ops.ptr(out), torch.cuda.current_stream().cuda_stream)
    assert rc == 0, lib.ca_last_error().decode()
    torch.cuda.synchronize()
    ops.probe_timeouts_provoked = getattr(ops, "probe_timeouts_provoked", 0) + 1
    assert int(out.item()) == 1              # the wait ran out (0 would mean the barrier completed)
    assert _timeouts(lib) == before + 1
    assert int(status.item()) & 1
    with pytest.raises(ca._lib.CircAttError, match="bounded wait"):
        ops.check_status(dev)
    ops.check_status(dev)                    # the flag was cleared by the raising check

    # the context is intact: a tiled forward still matches the oracle and sets no flag
    rng = np.random.default_rng(0)
    qn, kn, vn = (randn(rng, (32, 24, 16, 2)) for _ in range(3))
    y, _, _ = ops.attention_fwd(0, 0, *(jl.from_numpy(t) for t in (qn, kn, vn)), 7, False)
    yo, _ = orc.mh_attention(orc.DOT, up(qn), up(kn), up(vn), 7, 1)
    assert rel_err(jl.to_numpy(y), yo) < TOL
    ops.check_status(dev)
    assert _timeouts(lib) == before + 1


def test_bad_try_counts_are_rejected_on_the_host(ca):
    assert ca.lib.ca_probe_stage_timeout(0, None, None) == -1
    assert ca.lib.ca_probe_stage_timeout(1 << 21, None, None) == -1
