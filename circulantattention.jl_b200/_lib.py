"""ctypes binding of libcircatt_b200.so (the C ABI declared in include/circatt_b200.h).

There is no CPU path, as in the reference ("only CUDA compatible",
README.md:20): if the shared library has not been built, importing this module
raises, and every op raises on non-CUDA tensors.
"""
from __future__ import annotations

import ctypes as C
import os

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("CIRCATT_B200_LIB") or os.path.join(PKG_DIR, "libcircatt_b200.so")

CA_F32, CA_C64, CA_BF16 = 0, 1, 2
CA_DOT, CA_DISTANCE = 0, 1
CA_SOFTMAX, CA_ENTMAX15 = 0, 1


class CircAttError(RuntimeError):
    """A non-zero status from the C ABI (the Julia wrapper would raise ErrorException)."""


class ca_desc(C.Structure):
    _fields_ = [
        ("H", C.c_int32), ("W", C.c_int32), ("ndim", C.c_int32), ("channels", C.c_int32),
        ("units", C.c_int32), ("ws", C.c_int32), ("dtype", C.c_int32), ("similarity", C.c_int32),
        ("normalizer", C.c_int32), ("Wk", C.c_int32), ("wk_off", C.c_int32), ("scale", C.c_float),
    ]


class ca_chunk_job(C.Structure):
    _fields_ = [
        ("src", C.c_void_p), ("dst", C.c_void_p), ("chunk_bytes", C.c_int64), ("nchunks", C.c_int64),
        ("src_stride_bytes", C.c_int64), ("dst_stride_bytes", C.c_int64),
    ]


CA_MAX_CHUNK_JOBS = 32


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -c 'import __graft_entry__ as g; g.build()'` "
            "(nvcc, sm_100a). There is no CPU or PyTorch fallback.")
    return C.CDLL(LIB_PATH)


lib = _load()

_p = C.c_void_p
_D = C.POINTER(ca_desc)
_i32, _i64, _f32 = C.c_int32, C.c_int64, C.c_float

PROTOTYPES = {
    "ca_version": (C.c_int, []),
    "ca_last_error": (C.c_char_p, []),
    "ca_structure": (C.c_int, [_i32, _i32, _i32, _i32, _i64, _p, _p, _p]),
    "ca_operator_workspace": (C.c_size_t, [_D]),
    "ca_similarity": (C.c_int, [_D, _p, _p, _p, _p, _p]),
    "ca_similarity_bwd": (C.c_int, [_D, _p, _p, _p, _p, _p, _p, _p]),
    "ca_row_normalize": (C.c_int, [_D, _p, _p, _p, _p]),
    "ca_row_normalize_bwd": (C.c_int, [_D, _p, _p, _p, _p]),
    "ca_apply": (C.c_int, [_D, _p, _p, _p, _i32, _i32, _i32, _p, _p]),
    "ca_attention_fwd_workspace": (C.c_size_t, [_D, _i32]),
    "ca_attention_fwd": (C.c_int, [_D, _p, _p, _p, _p, _p, _p, _p, _p]),
    "ca_static_scratch_bytes": (C.c_size_t, []),
    "ca_attention_fwd_static": (C.c_int, [_D, _p, _p, _p, _p, _p, _p, _p]),
    "ca_attention_bwd_workspace": (C.c_size_t, [_D, _i32]),
    "ca_attention_bwd": (C.c_int, [_D] + [_p] * 14),
    "ca_attention_bwd_pre": (C.c_int, [_D] + [_p] * 10),
    "ca_attention_bwd_stage_workspace": (C.c_size_t, [_D]),
    "ca_attention_bwd_dq": (C.c_int, [_D] + [_p] * 10),
    "ca_attention_bwd_dkdv": (C.c_int, [_D] + [_p] * 11),
    "ca_status_word": (C.c_int, [_p]),
    "ca_stage_timeouts": (C.c_int, [C.POINTER(C.c_int32)]),
    "ca_entmax_scratch_limit": (C.c_int64, [C.c_int64]),
    "ca_comm_unique_id": (C.c_int, [_p]),
    "ca_comm_init": (C.c_int, [_i32, _i32, _p, C.POINTER(C.c_void_p)]),
    "ca_comm_destroy": (C.c_int, [_p]),
    "ca_halo_exchange": (C.c_int, [_p, _p, _p, _p, _p, C.c_size_t, _p]),
    "ca_copy_chunks": (C.c_int, [C.POINTER(ca_chunk_job), _i32, _p]),
    "ca_axpby": (C.c_int, [_i64, _f32, _p, _f32, _p, _p, _p]),
    "ca_scale_batch": (C.c_int, [_i64, _i32, _i32, _p, _i32, _i32, _p, _i32, _i32, _p, _p]),
    "ca_dot_batch": (C.c_int, [_i64, _i32, _i32, _p, _i32, _i32, _p, _i32, _i32, _p, _p]),
    "ca_sum_batch": (C.c_int, [_i64, _i32, _i32, _i32, _i32, _p, _p, _p]),
    "ca_sum_rows": (C.c_int, [_D, _p, _p, _p]),
    "ca_sum_cols": (C.c_int, [_D, _p, _p, _p]),
    "ca_probe_launch_count": (C.c_int64, []),
    "ca_probe_tiled_launch_count": (C.c_int64, []),
    "ca_probe_ffma": (C.c_int, [_i32, _i32, _p, _p]),
    "ca_probe_stage_timeout": (C.c_int, [_i32, _p, _p]),
}

for _name, (_res, _args) in PROTOTYPES.items():
    _fn = getattr(lib, _name)
    _fn.restype = _res
    _fn.argtypes = _args


def last_error() -> str:
    return lib.ca_last_error().decode()


def check(rc: int) -> None:
    if rc != 0:
        raise CircAttError(f"circatt_b200 status {rc}: {last_error()}")


def ptr(t):
    """Device pointer of a tensor (None -> NULL)."""
    return None if t is None else C.c_void_p(t.data_ptr())
