"""numpy front end of the C oracle in scan_oracle.c.

TEST INFRASTRUCTURE ONLY: the checker the CUDA path is compared against.  The
product package never imports this module; only the test suite, the smoke check
and the benchmark's CPU-baseline leg do.

Functions mirror the reference's oracle accelerated_scan/ref.py:49-57
(`scan(gates, tokens, reverse=False)` on `(B, C, T)` arrays) and the hand-written
backward of accelerated_scan/warp.py:50-65 / accelerated_scan/complex.py:190-219.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")
_lib = None


def build(force: bool = False) -> str:
    """Compile scan_oracle.c into liboracle.so next to it (gcc via the Makefile)."""
    src = os.path.join(_HERE, "scan_oracle.c")
    if (force or not os.path.exists(_LIB_PATH)
            or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src)):
        subprocess.run(["make", "-C", _HERE, "-B", "liboracle.so"], check=True,
                       stdout=subprocess.DEVNULL)
    return _LIB_PATH


def _load():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        lib = ctypes.CDLL(_LIB_PATH)
        p, i64, i32 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int
        for name in ("oracle_tree_scan_f32", "oracle_tree_scan_c64"):
            getattr(lib, name).argtypes = [p, p, p, i64, i64, i32]
            getattr(lib, name).restype = i32
        lib.oracle_seq_scan_f64.argtypes = [p, p, p, i64, i64, i32]
        lib.oracle_seq_scan_f64.restype = i32
        for name in ("oracle_backward_f32", "oracle_backward_c64"):
            getattr(lib, name).argtypes = [p, p, p, p, p, i64, i64]
            getattr(lib, name).restype = i32
        lib.oracle_num_threads.restype = i32
        lib.oracle_set_num_threads.argtypes = [i32]
        _lib = lib
    return _lib


def num_threads() -> int:
    return int(_load().oracle_num_threads())


def set_num_threads(n: int) -> None:
    _load().oracle_set_num_threads(int(n))


def _prep(x, dtype):
    x = np.ascontiguousarray(x, dtype=dtype)
    if x.ndim != 3:
        raise ValueError("expected a (B, C, T) array")
    return x


def _ptr(x):
    return x.ctypes.data_as(ctypes.c_void_p)


def scan(gates, tokens, reverse: bool = False):
    """Inclusive scan x[t] = gates[t]*x[t-1] + tokens[t] along the last axis with
    the tree of ref.py:49-121.  float32 or complex64 `(B, C, T)` arrays; real
    tokens with complex gates are promoted (complex.py:168-169)."""
    lib = _load()
    if np.iscomplexobj(gates):
        g = _prep(gates, np.complex64)
        x = _prep(np.asarray(tokens).astype(np.complex64), np.complex64)
        fn = lib.oracle_tree_scan_c64
    else:
        g, x = _prep(gates, np.float32), _prep(tokens, np.float32)
        fn = lib.oracle_tree_scan_f32
    if g.shape != x.shape:
        raise ValueError("gates and tokens differ in shape")
    out = np.empty_like(x)
    B, C, T = x.shape
    rc = fn(_ptr(g), _ptr(x), _ptr(out), B * C, T, int(bool(reverse)))
    if rc:
        raise RuntimeError(f"oracle scan failed ({rc})")
    return out


def scan_backward(gates, states, grad_out):
    """(d_gates, d_tokens) from the saved states and the output gradient
    (warp.py:53-65, complex.py:190-219)."""
    lib = _load()
    cplx = np.iscomplexobj(gates)
    dt = np.complex64 if cplx else np.float32
    g, s = _prep(gates, dt), _prep(states, dt)
    go = _prep(np.asarray(grad_out).astype(dt), dt)
    dg, dx = np.empty_like(g), np.empty_like(g)
    B, C, T = g.shape
    fn = lib.oracle_backward_c64 if cplx else lib.oracle_backward_f32
    rc = fn(_ptr(g), _ptr(s), _ptr(go), _ptr(dg), _ptr(dx), B * C, T)
    if rc:
        raise RuntimeError(f"oracle backward failed ({rc})")
    return dg, dx


def scan_exact(gates, tokens, reverse: bool = False):
    """The recurrence evaluated step by step in float64 (real inputs only)."""
    lib = _load()
    g, x = _prep(gates, np.float32), _prep(tokens, np.float32)
    out = np.empty(x.shape, dtype=np.float64)
    B, C, T = x.shape
    rc = lib.oracle_seq_scan_f64(_ptr(g), _ptr(x), _ptr(out), B * C, T, int(bool(reverse)))
    if rc:
        raise RuntimeError(f"oracle exact scan failed ({rc})")
    return out
