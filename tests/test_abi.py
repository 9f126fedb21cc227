"""CPU-side checks of the drop-in boundary: the shared library loads, exports
every symbol the header declares, and rejects bad descriptors with the
reference's messages before any device work (no GPU needed)."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADERS = sorted(os.path.join(ROOT, "include", f) for f in os.listdir(os.path.join(ROOT, "include")) if f.endswith(".h"))


def declared_symbols():
    names = set()
    for header in HEADERS:
        text = re.sub(r"/\*.*?\*/", "", open(header).read(), flags=re.S)
        names.update(re.findall(r"\b(ca_[a-z0-9_]+)\s*\(", text))
    return sorted(names)


def test_header_declares_the_expected_surface():
    syms = declared_symbols()
    for name in ("ca_structure", "ca_similarity", "ca_similarity_bwd", "ca_row_normalize", "ca_row_normalize_bwd",
                 "ca_apply", "ca_attention_fwd", "ca_attention_bwd", "ca_axpby", "ca_scale_batch", "ca_dot_batch",
                 "ca_sum_batch", "ca_sum_rows", "ca_sum_cols", "ca_version", "ca_last_error"):
        assert name in syms


def test_library_exports_every_declared_symbol(ca):
    lib = C.CDLL(ca.LIB_PATH)
    for name in declared_symbols():
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"
    assert lib.ca_version() >= 100


def test_python_prototypes_cover_the_header(ca):
    from circatt_b200 import _lib
    assert sorted(_lib.PROTOTYPES) == declared_symbols()


def _desc(ca, **kw):
    from circatt_b200._lib import ca_desc
    base = dict(H=8, W=8, ndim=2, channels=4, units=2, ws=5, dtype=0, similarity=0, normalizer=0, Wk=0, wk_off=0,
                scale=1.0)
    base.update(kw)
    return ca_desc(**base)


@pytest.mark.parametrize("kw,code,msg", [
    (dict(ws=4), -1, "filter size M=4 must be odd."),
    (dict(H=3), -1, "smaller than the window"),
    (dict(W=3), -1, "smaller than the window"),
    (dict(ndim=3), -1, "only 1 or 2 spatial dims"),
    (dict(ndim=1, W=8), -1, "1-D signals must have W == 1"),
    (dict(dtype=7), -1, "unknown dtype"),
    (dict(similarity=5), -1, "unknown similarity"),
    (dict(channels=0), -1, "must be positive"),
    (dict(Wk=12, wk_off=2), -2, "band mode"),
])
def test_bad_descriptors_are_rejected_on_the_host(ca, kw, code, msg):
    from circatt_b200._lib import lib, last_error
    d = _desc(ca, **kw)
    one = C.c_void_p(16)        # never dereferenced: validation comes first
    rc = lib.ca_similarity(d, one, one, one, None, None)
    assert rc == code
    assert msg in last_error()


def test_null_pointers_are_rejected(ca):
    from circatt_b200._lib import lib, last_error
    assert lib.ca_similarity(_desc(ca), None, None, None, None, None) == -3
    assert "NULL" in last_error()
    assert lib.ca_attention_bwd_workspace(_desc(ca), 0) == 8 * 8 * 2 * 4
    assert lib.ca_attention_fwd_workspace(_desc(ca, normalizer=1), 0) == 64 * 25 * 2 * 4
    assert lib.ca_attention_fwd_workspace(_desc(ca), 0) == 0


def test_cpu_tensors_fail_loudly(ca):
    import torch
    x = ca.jl.randn(8, 8, 4, 2, device="cpu")
    with pytest.raises(RuntimeError, match="only CUDA compatible"):
        ca.circulant_similarity(ca.DotSimilarity(), x, x, 5)
    with pytest.raises(AssertionError, match="must be odd"):
        ca.circulant_similarity(ca.DotSimilarity(), x, x, 4)


def test_julia_shaped_tensors(ca):
    import numpy as np
    a = np.asfortranarray(np.arange(24, dtype=np.float32).reshape((2, 3, 4), order="F"))
    t = ca.jl.from_numpy(a, device="cpu")
    assert tuple(t.shape) == (2, 3, 4) and ca.jl.is_colmajor(t)
    assert np.array_equal(ca.jl.to_numpy(t), a)
    r = ca.jl.reshape(t, 6, 4)
    assert np.array_equal(ca.jl.to_numpy(r), a.reshape((6, 4), order="F"))
    s = ca.splitheads(ca.jl.from_numpy(np.asfortranarray(np.zeros((5, 6, 2), np.float32)), device="cpu"), 3)
    assert tuple(s.shape) == (5, 2, 6)


def test_entmax_scratch_limit_round_trip(ca):
    """Process-wide setting: a negative argument queries, a non-negative one sets and returns the previous value;
    the workspace query follows it (a 32 x 32 image of 16 channels, ws 5: 205 KB of scores)."""
    from circatt_b200._lib import lib
    assert lib.ca_entmax_scratch_limit(-1) == 256 << 20
    d = _desc(ca, H=32, W=32, channels=16, normalizer=1)
    chain = lib.ca_attention_fwd_workspace(d, 0)
    assert chain >= 1024 * 25 * 2 * 4
    assert lib.ca_entmax_scratch_limit(0) == 256 << 20
    try:
        sweeps = lib.ca_attention_fwd_workspace(d, 0)
        assert 0 < sweeps != chain                       # the packed (k|v) and two planes instead of the scores
    finally:
        assert lib.ca_entmax_scratch_limit(256 << 20) == 0
    assert lib.ca_attention_fwd_workspace(d, 0) == chain


def test_copy_chunks_validates_on_the_host(ca):
    from circatt_b200._lib import lib, last_error
    assert lib.ca_copy_chunks(None, 0, None) == 0
    assert lib.ca_copy_chunks(None, 33, None) == -1 and "njobs" in last_error()
    assert lib.ca_copy_chunks(None, 2, None) == -3


def test_line_kernels_need_no_workspace_query(ca):
    """1-D signals of up to 16 real channels per unit in flash mode: no scratch at all, entmax included."""
    from circatt_b200._lib import lib
    for nrm in (0, 1):
        d = _desc(ca, H=4096, W=1, ndim=1, channels=8, units=4, ws=127, normalizer=nrm)
        assert lib.ca_attention_fwd_workspace(d, 0) == 0
    wide = _desc(ca, H=4096, W=1, ndim=1, channels=32, units=4, ws=127, normalizer=0)
    assert lib.ca_attention_fwd_workspace(wide, 0) > 0
