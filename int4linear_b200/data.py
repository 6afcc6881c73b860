"""Seeded synthetic operands: i.i.d. uniform signed 4-bit values in [-8, 7].

The reference's harnesses fill operands with `rand() % 15 - 7` under a time
seed (test/test_correctness.cu:33,43-44), which never produces -8 and cannot be
reproduced.  This generator is counter based -- element i of a stream is a pure
function of (seed, i) -- so any slice can be produced independently, in
parallel, on any machine, and a shard of W on one GPU is bit-identical to the
same rows of the full W.

    value(seed, i) = (splitmix64(seed + (i + 1) * 0x9E3779B97F4A7C15) >> 60) - 8
"""
from __future__ import annotations

import numpy as np

_GOLDEN = np.uint64(0x9E3779B97F4A7C15)
_M1 = np.uint64(0xBF58476D1CE4E5B9)
_M2 = np.uint64(0x94D049BB133111EB)


def _mix(z: np.ndarray) -> np.ndarray:
    z = (z ^ (z >> np.uint64(30))) * _M1
    z = (z ^ (z >> np.uint64(27))) * _M2
    return z ^ (z >> np.uint64(31))


def _nibbles(seed: int, start: int, count: int) -> np.ndarray:
    """uint8 values 0..15 for stream positions [start, start+count)."""
    with np.errstate(over="ignore"):
        idx = np.arange(start + 1, start + count + 1, dtype=np.uint64)
        z = _mix(np.uint64(seed & 0xFFFFFFFFFFFFFFFF) + idx * _GOLDEN)
    return (z >> np.uint64(60)).astype(np.uint8)


def uniform_s4(seed: int, rows: int, cols: int, row_start: int = 0) -> np.ndarray:
    """[rows, cols] int8 in [-8, 7]; row r here is row row_start + r of the stream's matrix."""
    nib = _nibbles(seed, row_start * cols, rows * cols)
    return (nib.astype(np.int8) - 8).reshape(rows, cols)


def uniform_s4_packed(seed: int, rows: int, cols: int, row_start: int = 0,
                      chunk_rows: int | None = None) -> np.ndarray:
    """Same values as uniform_s4, already packed: [rows, cols/2] uint8, low nibble = even index.

    Generated in row chunks so that the largest shapes never hold more than a few
    hundred MB of temporaries."""
    if cols % 2:
        raise ValueError("cols must be even")
    if chunk_rows is None:
        chunk_rows = max(1, (1 << 24) // cols)
    out = np.empty((rows, cols // 2), dtype=np.uint8)
    for r0 in range(0, rows, chunk_rows):
        r1 = min(rows, r0 + chunk_rows)
        nib = _nibbles(seed, (row_start + r0) * cols, (r1 - r0) * cols).reshape(r1 - r0, cols)
        # stored nibble = two's complement of (value) = (nib - 8) & 15 = nib ^ 8
        nib ^= np.uint8(8)
        out[r0:r1] = nib[:, 0::2] | (nib[:, 1::2] << 4)
    return out
