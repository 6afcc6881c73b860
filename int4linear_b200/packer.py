"""Host-side nibble packer with the reference's interface and bit layout.

`pack` / `unpack` mirror `void pack(const int* src, int* dst, int m, int n)` and
`void unpack(...)` of the reference (utils/packer.h:5-6, utils/packer.cpp:3-31):
eight signed 4-bit values per little-endian 32-bit word, element j*8+t of a row
in bits [4t, 4t+4), rows padded with zero nibbles to a multiple of eight
elements; unpack sign-extends.  They are vectorised numpy, not a loop, and are
what callers use to prepare operands for the device entry points.

`pack_bytes` / `unpack_bytes` are the same format seen as bytes (low nibble =
even index), which is how the kernels address it.
"""
from __future__ import annotations

import numpy as np


def pack(src: np.ndarray) -> np.ndarray:
    """[m, n] integers in [-8, 7] -> [m, ceil(n/8)] int32 words."""
    src = np.asarray(src)
    if src.ndim != 2:
        raise ValueError("pack expects a 2-D array")
    m, n = src.shape
    n_dst = (n + 7) // 8
    nib = np.zeros((m, n_dst * 8), dtype=np.uint32)
    nib[:, :n] = src.astype(np.int64) & 0xF
    nib = nib.reshape(m, n_dst, 8)
    shifts = (4 * np.arange(8, dtype=np.uint32))[None, None, :]
    words = np.bitwise_or.reduce(nib << shifts, axis=2).astype(np.uint32)
    return words.view(np.int32)


def unpack(src: np.ndarray, n: int) -> np.ndarray:
    """[m, ceil(n/8)] int32 words -> [m, n] sign-extended int32 values."""
    src = np.ascontiguousarray(src, dtype=np.int32)
    m, n_src = src.shape
    if n_src != (n + 7) // 8:
        raise ValueError("word count does not match n")
    words = src.view(np.uint32)[:, :, None]
    shifts = (4 * np.arange(8, dtype=np.uint32))[None, None, :]
    nib = ((words >> shifts) & 0xF).astype(np.int32).reshape(m, n_src * 8)[:, :n]
    return np.where(nib >= 8, nib - 16, nib).astype(np.int32)


def pack_bytes(vals: np.ndarray) -> np.ndarray:
    """[m, k] int8 values in [-8, 7], k even -> [m, k/2] uint8 (low nibble = even index)."""
    vals = np.asarray(vals)
    if vals.shape[1] % 2:
        raise ValueError("k must be even")
    v = vals.astype(np.uint8) & 0xF
    return (v[:, 0::2] | (v[:, 1::2] << 4)).astype(np.uint8)


def unpack_bytes(packed: np.ndarray) -> np.ndarray:
    """[m, k/2] uint8 -> [m, k] int8 sign-extended values."""
    p = np.asarray(packed, dtype=np.uint8)
    out = np.empty((p.shape[0], p.shape[1] * 2), dtype=np.int8)
    lo = (p & 0xF).astype(np.int8)
    hi = (p >> 4).astype(np.int8)
    out[:, 0::2] = np.where(lo >= 8, lo - 16, lo)
    out[:, 1::2] = np.where(hi >= 8, hi - 16, hi)
    return out
