"""GPU: the device-side packer against the oracle's pack/unpack (bit-exact, ragged widths included)."""
import numpy as np
import pytest

import int4linear_b200 as L
from oracle import oracle as O

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("shape", [(1, 1), (5, 19), (33, 64), (128, 4096), (7, 8), (3, 1000), (257, 24)],
                         ids=lambda s: "x".join(map(str, s)))
def test_pack_unpack_device(cuda, shape):
    import torch
    m, n = shape
    vals = L.uniform_s4(90 + m, m, n)
    want = O.pack(vals.astype(np.int32))
    got32 = L.pack_device(torch.from_numpy(vals.astype(np.int32)).to(cuda))
    got8 = L.pack_device(torch.from_numpy(vals).to(cuda))
    torch.cuda.synchronize()
    assert O.is_same(got32.cpu().numpy(), want)
    assert O.is_same(got8.cpu().numpy(), want)
    back = L.unpack_device(got32, n)
    torch.cuda.synchronize()
    assert O.is_same(back.cpu().numpy(), O.unpack(want, n))
    assert O.is_same(back.cpu().numpy(), vals.astype(np.int32))


def test_device_packed_operands_feed_the_gemm(cuda):
    import torch
    m, n, k = 200, 328, 512
    x = L.uniform_s4(3, m, k)
    w = L.uniform_s4(4, n, k)
    xp = L.pack_device(torch.from_numpy(x).to(cuda))
    wp = L.pack_device(torch.from_numpy(w.astype(np.int32)).to(cuda))
    y = L.linear(xp, wp)
    torch.cuda.synchronize()
    assert O.is_same(y.cpu().numpy(), O.linear_ref(x.astype(np.int32), w.astype(np.int32)))
