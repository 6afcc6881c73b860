"""GPU: the entry point that allocates nothing (int4_linear_launch_static_scratch_async).

Some users of this library cannot let it call cudaMalloc: their process has already given all
device memory to another allocator, or may not stall on the synchronisation an allocation
implies.  For them the two-pass operator exists in a form whose scratch is a fixed array inside
the library.  This file checks, through the C ABI, that it returns exactly what the regular entry
point returns, on two consecutive calls (the second finds the first call's bytes still in the
shared scratch), that it refuses shapes beyond its fixed capacity, and that it works both as the
very first thing a fresh process does with the library and after every other test (the file name
makes pytest collect it last).
"""
import ctypes

import numpy as np
import pytest

import int4linear_b200 as L
from int4linear_b200 import _lib
from conftest import make_case

pytestmark = pytest.mark.gpu


def _call_static(lib, xd, wd, yd, m, n, k, bias=None):
    import torch
    stream = torch.cuda.current_stream().cuda_stream
    return lib.int4_linear_launch_static_scratch_async(
        xd.data_ptr(), wd.data_ptr(), bias.data_ptr() if bias is not None else None, yd.data_ptr(), m, n, k, stream)


def test_static_scratch_matches_regular_entry_point_twice(cuda):
    import torch
    lib = _lib.load()
    # two different problems back to back: the second one reuses (and partly overlaps) the bytes
    # the first one left in the shared scratch
    cases = [(384, 520, 1024, 41), (200, 1000, 416, 42)]
    for rep, (m, n, k, seed) in enumerate(cases):
        x, w, xp, wp = make_case(m, n, k, seed=seed)
        xd, wd = torch.from_numpy(xp).to(cuda), torch.from_numpy(wp).to(cuda)
        bias = torch.from_numpy(((np.arange(n) * 31) % 1001 - 500).astype(np.int32)).to(cuda) if rep else None
        want = torch.full((m, n), -1, dtype=torch.int32, device=cuda)
        st = lib.int4_linear_bias_launch_async(xd.data_ptr(), wd.data_ptr(),
                                               bias.data_ptr() if bias is not None else None,
                                               want.data_ptr(), m, n, k, torch.cuda.current_stream().cuda_stream)
        assert st == 0
        got = torch.full((m, n), -2, dtype=torch.int32, device=cuda)
        assert _call_static(lib, xd, wd, got, m, n, k, bias) == 0
        torch.cuda.synchronize()
        assert lib.int4_linear_last_status() == 0
        assert bool((got == want).all()), f"call {rep}: static-scratch result differs from the regular entry point"
        # and the regular entry point is itself pinned to the CPU reference arithmetic
        ref = x.astype(np.int64) @ w.astype(np.int64).T
        if bias is not None:
            ref = ref + bias.cpu().numpy()[None, :]
        assert np.array_equal(want.cpu().numpy(), ref.astype(np.int32))


def test_static_scratch_rejects_what_does_not_fit(cuda):
    import torch
    lib = _lib.load()
    buf = torch.zeros(4096, dtype=torch.uint8, device=cuda)
    p = buf.data_ptr()
    # (m + n) * k = 16384 * 8192 = 128 Mi > 64 Mi: refused before anything is launched
    assert lib.int4_linear_launch_static_scratch_async(p, p, None, p, 8192, 8192, 8192, None) == 7
    assert lib.int4_linear_status_string(7).decode().startswith("size beyond")
    # exactly at the limit the size check passes (64 Mi) -- only checked, not run: pointers are dummies
    assert lib.int4_linear_launch_static_scratch_async(p, p, None, p, 8192, 8192, 4096 + 32, None) == 7
    assert lib.int4_linear_launch_static_scratch_async(None, p, None, p, 8, 8, 32, None) == 1
    assert lib.int4_linear_launch_static_scratch_async(p, p, None, p, 8, 8, 40, None) == 2
