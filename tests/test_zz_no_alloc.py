"""GPU: the entry point that allocates nothing (int4_linear_launch_static_scratch_async).

Some users of this library cannot let it call cudaMalloc: their process has already given all
device memory to another allocator, or may not stall on the synchronisation an allocation
implies.  For them the two-pass operator exists in a form whose scratch is a fixed array inside
the library.  This file checks, through the C ABI, that it returns exactly what the regular entry
point returns, on two consecutive calls (the second finds the first call's bytes still in the
shared scratch); that it accepts and computes a problem that fills the array to the last byte and
refuses anything larger; that its status word is read back by int4_linear_last_status; and that
it works when it is the very first call a fresh process makes into the library (a child process)
as well as after every other test (the file name makes pytest collect it last).
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
    # one K step beyond the capacity: (8192 + 8192) * 4128 > 64 Mi
    assert lib.int4_linear_launch_static_scratch_async(p, p, None, p, 8192, 8192, 4096 + 32, None) == 7
    assert lib.int4_linear_launch_static_scratch_async(None, p, None, p, 8, 8, 32, None) == 1
    assert lib.int4_linear_launch_static_scratch_async(p, p, None, p, 8, 8, 40, None) == 2


def test_static_scratch_exactly_at_capacity(cuda):
    """(m + n) * k = (8192 + 8192) * 4096 = 67 108 864 bytes: the whole array, to the last byte."""
    import torch
    lib = _lib.load()
    m = n = 8192
    k = 4096
    xd = torch.from_numpy(L.uniform_s4_packed(0xA0C1, m, k)).to(cuda)
    wd = torch.from_numpy(L.uniform_s4_packed(0xB0C1, n, k)).to(cuda)
    want = torch.empty((m, n), dtype=torch.int32, device=cuda)
    got = torch.full((m, n), -2, dtype=torch.int32, device=cuda)
    stream = torch.cuda.current_stream().cuda_stream
    assert lib.int4_linear_launch_async(xd.data_ptr(), wd.data_ptr(), want.data_ptr(), m, n, k, stream) == 0
    assert _call_static(lib, xd, wd, got, m, n, k) == 0
    torch.cuda.synchronize()
    assert lib.int4_linear_last_status() == 0   # polls the regular AND the static-scratch status word
    assert torch.equal(got, want)


_CHILD = r"""
import sys
import numpy as np
import torch
sys.path.insert(0, sys.argv[1])
from int4linear_b200 import _lib, uniform_s4, pack_bytes
torch.cuda.set_device(0)
dev = torch.device("cuda:0")
m, n, k = 300, 520, 512
x, w = uniform_s4(0xA0C2, m, k), uniform_s4(0xB0C2, n, k)
xd, wd = torch.from_numpy(pack_bytes(x)).to(dev), torch.from_numpy(pack_bytes(w)).to(dev)
got = torch.full((m, n), -2, dtype=torch.int32, device=dev)
want = torch.full((m, n), -1, dtype=torch.int32, device=dev)
lib = _lib.load()
assert lib.int4_linear_launch_count() == 0
# the first call this process makes into the library
st = lib.int4_linear_launch_static_scratch_async(xd.data_ptr(), wd.data_ptr(), None, got.data_ptr(), m, n, k, None)
assert st == 0, st
torch.cuda.synchronize()
assert lib.int4_linear_last_status() == 0
assert lib.int4_linear_launch_async(xd.data_ptr(), wd.data_ptr(), want.data_ptr(), m, n, k, None) == 0
torch.cuda.synchronize()
assert torch.equal(got, want)
assert np.array_equal(got.cpu().numpy(), (x.astype(np.int64) @ w.astype(np.int64).T).astype(np.int32))
print("STATIC_FIRST_OK")
"""


def test_static_scratch_as_first_call_of_a_fresh_process(cuda):
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = subprocess.run([sys.executable, "-c", _CHILD, root], capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-2000:]
    assert "STATIC_FIRST_OK" in out.stdout
