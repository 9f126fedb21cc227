"""ctypes wrapper of oracle/libcircatt_cpu.so (plain C + OpenMP restatement).

TEST INFRASTRUCTURE ONLY: used by tests/, by `__graft_entry__.smoke()` and by the
CPU-baseline legs of bench.py.  Arrays are numpy, Julia-shaped, Fortran order.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
SO = os.path.join(HERE, "libcircatt_cpu.so")


def load():
    if not os.path.exists(SO):
        subprocess.run(["make", "-s", "-C", HERE], check=True)
    lib = C.CDLL(SO)
    lib.ca_cpu_threads.restype = C.c_int
    return lib


_lib = None


def lib():
    global _lib
    if _lib is None:
        _lib = load()
    return _lib


def threads() -> int:
    return int(lib().ca_cpu_threads())


def use_all_cores() -> int:
    """Run on every core this process may use, whatever OMP_NUM_THREADS says; returns the count."""
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    lib().ca_cpu_set_threads(n)
    return threads()


def _prep(x, dtype):
    x = np.asfortranarray(x, dtype=dtype)
    return x, x.ctypes.data_as(C.c_void_p)


def _dims(q):
    spatial = q.shape[:-2]
    H = spatial[0]
    W = spatial[1] if len(spatial) == 2 else 1
    return H, W, len(spatial), q.shape[-2], q.shape[-1]


def attention_fwd(q, k, v, ws, dist=False, dtype=np.float32):
    """(y, lse) for head-split real tensors (spatial..., c, units); scale = 1/sqrt(c)."""
    H, W, nd, c, units = _dims(q)
    suffix, real = ("f32", C.c_float) if dtype == np.float32 else ("f64", C.c_double)
    q, qp = _prep(q, dtype); k, kp = _prep(k, dtype); v, vp = _prep(v, dtype)
    y = np.empty(q.shape, dtype=dtype, order="F")
    lse = np.empty((H * W, units), dtype=dtype, order="F")
    fn = getattr(lib(), "ca_cpu_attention_fwd_" + suffix)
    rc = fn(H, W, nd, c, units, ws, int(dist), real(1.0 / np.sqrt(c)), qp, kp, vp,
            y.ctypes.data_as(C.c_void_p), lse.ctypes.data_as(C.c_void_p))
    if rc != 0:
        raise ValueError("bad window/extent")
    return y, lse


def attention_bwd(q, k, v, y, dy, lse, ws, dist=False, dtype=np.float32):
    H, W, nd, c, units = _dims(q)
    suffix, real = ("f32", C.c_float) if dtype == np.float32 else ("f64", C.c_double)
    arrs = [_prep(t, dtype) for t in (q, k, v, y, dy, lse)]
    outs = [np.empty(arrs[0][0].shape, dtype=dtype, order="F") for _ in range(3)]
    fn = getattr(lib(), "ca_cpu_attention_bwd_" + suffix)
    rc = fn(H, W, nd, c, units, ws, int(dist), real(1.0 / np.sqrt(c)), *[p for _, p in arrs],
            *[o.ctypes.data_as(C.c_void_p) for o in outs])
    if rc != 0:
        raise ValueError("bad window/extent")
    return tuple(outs)
