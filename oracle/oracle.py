"""numpy front end to the CPU oracle (linear_ref.c) and, when it was built, to
the shim around the reference's own sources (oracle/_ref/).

TEST INFRASTRUCTURE ONLY.  Importers are the test-suite, the smoke check and the
benchmark's CPU-baseline leg; the product package never imports this module.

Function -> reference location it restates:
    pack            utils/packer.cpp:3-18
    unpack          utils/packer.cpp:20-31
    linear_ref      test/test_correctness.cu:12-19
    is_same         test/test_correctness.cu:22-27
"""
from __future__ import annotations

import ctypes
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_I32P = ctypes.POINTER(ctypes.c_int)


def _ptr(a: np.ndarray):
    return a.ctypes.data_as(_I32P)


def _as_i32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.int32)


_lib = None


def lib() -> ctypes.CDLL:
    """Load liboracle.so, building it first if the file is missing."""
    global _lib
    if _lib is None:
        path = os.path.join(_HERE, "liboracle.so")
        if not os.path.exists(path):
            from . import build
            build.build_oracle()
        L = ctypes.CDLL(path)
        L.oracle_pack.argtypes = [_I32P, _I32P, ctypes.c_int, ctypes.c_int]
        L.oracle_unpack.argtypes = [_I32P, _I32P, ctypes.c_int, ctypes.c_int]
        L.oracle_linear_ref.argtypes = [_I32P, _I32P, _I32P] + [ctypes.c_int] * 3
        L.oracle_linear_ref_1t.argtypes = [_I32P, _I32P, _I32P] + [ctypes.c_int] * 3
        L.oracle_linear_ref_rows.argtypes = [_I32P, _I32P, _I32P, _I32P] + [ctypes.c_int] * 3
        L.oracle_linear_packed.argtypes = [_I32P, _I32P, _I32P] + [ctypes.c_int] * 3
        L.oracle_linear_packed.restype = ctypes.c_int
        L.oracle_is_same.argtypes = [_I32P, _I32P, ctypes.c_longlong]
        L.oracle_is_same.restype = ctypes.c_int
        _lib = L
    return _lib


def pack(src: np.ndarray) -> np.ndarray:
    """[m, n] ints in [-8, 7] -> [m, ceil(n/8)] int32 words (utils/packer.cpp:3-18)."""
    src = _as_i32(src)
    m, n = src.shape
    dst = np.empty((m, (n + 7) // 8), dtype=np.int32)
    lib().oracle_pack(_ptr(src), _ptr(dst), m, n)
    return dst


def unpack(src: np.ndarray, n: int) -> np.ndarray:
    """[m, ceil(n/8)] int32 words -> [m, n] sign-extended ints (utils/packer.cpp:20-31)."""
    src = _as_i32(src)
    m = src.shape[0]
    assert src.shape[1] == (n + 7) // 8
    dst = np.empty((m, n), dtype=np.int32)
    lib().oracle_unpack(_ptr(src), _ptr(dst), m, n)
    return dst


def linear_ref(x: np.ndarray, w: np.ndarray, single_thread: bool = False) -> np.ndarray:
    """y[m, n] = x[m, k] @ w[n, k].T in int32 (test/test_correctness.cu:12-19)."""
    x, w = _as_i32(x), _as_i32(w)
    m, k = x.shape
    n, k2 = w.shape
    assert k == k2
    y = np.empty((m, n), dtype=np.int32)
    fn = lib().oracle_linear_ref_1t if single_thread else lib().oracle_linear_ref
    fn(_ptr(x), _ptr(w), _ptr(y), m, n, k)
    return y


def linear_ref_rows(x: np.ndarray, w: np.ndarray, rows) -> np.ndarray:
    """Rows `rows` of linear_ref(x, w), computed without the other rows."""
    x, w = _as_i32(x), _as_i32(w)
    rows = _as_i32(rows)
    n, k = w.shape
    assert x.shape[1] == k and rows.min() >= 0 and rows.max() < x.shape[0]
    y = np.empty((len(rows), n), dtype=np.int32)
    lib().oracle_linear_ref_rows(_ptr(x), _ptr(w), _ptr(y), _ptr(rows), len(rows), n, k)
    return y


def linear_packed(x_packed: np.ndarray, w_packed: np.ndarray, k: int) -> np.ndarray:
    """The operator as the device sees it: packed int32 words in, int32 out."""
    x_packed, w_packed = _as_i32(x_packed), _as_i32(w_packed)
    m, n = x_packed.shape[0], w_packed.shape[0]
    y = np.empty((m, n), dtype=np.int32)
    rc = lib().oracle_linear_packed(_ptr(x_packed), _ptr(w_packed), _ptr(y), m, n, k)
    if rc != 0:
        raise MemoryError("oracle_linear_packed: scratch allocation failed")
    return y


def is_same(a: np.ndarray, b: np.ndarray) -> bool:
    """Exact equality of two int32 arrays (test/test_correctness.cu:22-27)."""
    a, b = _as_i32(a), _as_i32(b)
    if a.size != b.size:
        return False
    return bool(lib().oracle_is_same(_ptr(a), _ptr(b), a.size))


def linear_ref_sgemm(x: np.ndarray, w: np.ndarray) -> np.ndarray:
    """Fast exact checker for full-size shapes: the same product through a
    float32 BLAS GEMM.  Every operand is an integer in [-8, 7] and every partial
    sum is an integer of magnitude <= 64*k, so for k <= 2**18 all intermediate
    values are exactly representable in float32 (< 2**24) whatever the
    summation order, and the result equals linear_ref bit for bit.  The tests
    check that claim against linear_ref on small shapes before relying on it."""
    k = x.shape[1]
    assert 64 * k < (1 << 24), "float32 would no longer be exact"
    y = np.asarray(x, dtype=np.float32) @ np.asarray(w, dtype=np.float32).T
    return y.astype(np.int32)


# ---------------------------------------------------------------------------
# The reference's own code, when oracle/_ref/ was built from its sources.
# ---------------------------------------------------------------------------
_ref = None


def ref_lib():
    """ctypes handle on oracle/_ref/libint4linear_ref.so or None if absent."""
    global _ref
    if _ref is None:
        path = os.path.join(_HERE, "_ref", "libint4linear_ref.so")
        if not os.path.exists(path):
            return None
        L = ctypes.CDLL(path)
        L.ref_pack.argtypes = [_I32P, _I32P, ctypes.c_int, ctypes.c_int]
        L.ref_unpack.argtypes = [_I32P, _I32P, ctypes.c_int, ctypes.c_int]
        L.ref_linear_ref.argtypes = [_I32P, _I32P, _I32P] + [ctypes.c_int] * 3
        L.ref_is_same.argtypes = [_I32P, _I32P, ctypes.c_int]
        L.ref_is_same.restype = ctypes.c_int
        L.ref_linear_v21_launch.argtypes = [ctypes.c_void_p] * 3 + [ctypes.c_int] * 3
        _ref = L
    return _ref


def ref_pack(src: np.ndarray) -> np.ndarray:
    src = _as_i32(src)
    m, n = src.shape
    dst = np.empty((m, (n + 7) // 8), dtype=np.int32)
    ref_lib().ref_pack(_ptr(src), _ptr(dst), m, n)
    return dst


def ref_unpack(src: np.ndarray, n: int) -> np.ndarray:
    src = _as_i32(src)
    dst = np.empty((src.shape[0], n), dtype=np.int32)
    ref_lib().ref_unpack(_ptr(src), _ptr(dst), src.shape[0], n)
    return dst


def ref_linear_ref(x: np.ndarray, w: np.ndarray) -> np.ndarray:
    x, w = _as_i32(x), _as_i32(w)
    m, k = x.shape
    n = w.shape[0]
    y = np.empty((m, n), dtype=np.int32)
    ref_lib().ref_linear_ref(_ptr(x), _ptr(w), _ptr(y), m, n, k)
    return y
