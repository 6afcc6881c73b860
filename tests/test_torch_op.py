"""The PyTorch operator binding: registration and shape inference on CPU, execution on the GPU."""
import numpy as np
import pytest
import torch

import int4linear_b200 as L
import int4linear_b200.torch_op  # noqa: F401  (registers torch.ops.int4linear.*)
from oracle import oracle as O


def test_ops_are_registered_with_shape_inference():
    x = torch.empty((5, 64), dtype=torch.uint8, device="meta")
    w = torch.empty((9, 64), dtype=torch.uint8, device="meta")
    y = torch.ops.int4linear.linear(x, w)
    assert y.shape == (5, 9) and y.dtype == torch.int32
    p = torch.ops.int4linear.pack(torch.empty((3, 19), dtype=torch.int8, device="meta"))
    assert p.shape == (3, 3) and p.dtype == torch.int32
    with pytest.raises(Exception):
        torch.ops.int4linear.linear(x, torch.empty((9, 32), dtype=torch.uint8, device="meta"))


def test_no_cpu_kernel():
    x = torch.zeros((4, 16), dtype=torch.uint8)
    with pytest.raises(Exception):
        torch.ops.int4linear.linear(x, x)


@pytest.mark.gpu
def test_op_matches_oracle(cuda):
    m, n, k = 72, 136, 256
    x = L.uniform_s4(11, m, k)
    w = L.uniform_s4(12, n, k)
    xp = torch.ops.int4linear.pack(torch.from_numpy(x).to(cuda))
    wp = torch.ops.int4linear.pack(torch.from_numpy(w).to(cuda))
    y = torch.ops.int4linear.linear(xp, wp)
    torch.cuda.synchronize()
    assert O.is_same(y.cpu().numpy(), O.linear_ref(x.astype(np.int32), w.astype(np.int32)))
