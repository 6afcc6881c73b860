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


def pack_device(src, stream=None):
    """Device-side pack: a CUDA tensor [m, n] of int32 or int8 values in [-8, 7] ->
    CUDA int32 tensor [m, ceil(n/8)] in the reference's word layout (asynchronous)."""
    import torch
    from . import _lib
    from .linear import Int4LinearError
    if not src.is_cuda or src.dim() != 2:
        raise ValueError("pack_device expects a 2-D CUDA tensor")
    src = src.contiguous()
    m, n = src.shape
    dst = torch.empty((m, (n + 7) // 8), dtype=torch.int32, device=src.device)
    handle = (stream or torch.cuda.current_stream()).cuda_stream
    lib = _lib.load()
    with torch.cuda.device(src.device):
        if src.dtype == torch.int32:
            st = lib.int4_linear_pack_i32(src.data_ptr(), dst.data_ptr(), m, n, handle)
        elif src.dtype == torch.int8:
            st = lib.int4_linear_pack_i8(src.data_ptr(), dst.data_ptr(), m, n, handle)
        else:
            raise TypeError("pack_device takes int32 or int8 tensors")
    if st != 0:
        raise Int4LinearError(st, "int4_linear_pack")
    return dst


def unpack_device(src, n: int, stream=None):
    """Device-side unpack: CUDA int32 words [m, ceil(n/8)] -> CUDA int32 tensor [m, n]."""
    import torch
    from . import _lib
    from .linear import Int4LinearError
    src = src.contiguous()
    m = src.shape[0]
    if src.dtype != torch.int32 or src.shape[1] != (n + 7) // 8:
        raise ValueError("unpack_device expects int32 words [m, ceil(n/8)]")
    dst = torch.empty((m, n), dtype=torch.int32, device=src.device)
    handle = (stream or torch.cuda.current_stream()).cuda_stream
    with torch.cuda.device(src.device):
        st = _lib.load().int4_linear_unpack_i32(src.data_ptr(), dst.data_ptr(), m, n, handle)
    if st != 0:
        raise Int4LinearError(st, "int4_linear_unpack_i32")
    return dst
