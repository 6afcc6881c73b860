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
    z = torch.ops.int4linear.linear_scaled(x, w, None, torch.empty(9, device="meta"), None)
    assert z.shape == (5, 9) and z.dtype == torch.bfloat16


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


@pytest.mark.gpu
def test_scaled_op_matches_the_integer_op(cuda):
    """linear_scaled = the integer result of the same operands, scaled in float32 and rounded to bf16."""
    m, n, k = 48, 264, 512
    xp = torch.from_numpy(L.uniform_s4_packed(21, m, k)).to(cuda)
    wp = torch.from_numpy(L.uniform_s4_packed(22, n, k)).to(cuda)
    rs = torch.rand(m, device=cuda) * 0.1 + 0.01
    cs = torch.rand(n, device=cuda) * 0.1 + 0.01
    b = torch.randn(n, device=cuda)
    acc = torch.ops.int4linear.linear(xp, wp).float()
    z = torch.ops.int4linear.linear_scaled(xp, wp, rs, cs, b)
    ref = torch.addcmul(b[None, :].expand(m, n), acc * rs[:, None], cs[None, :].expand(m, n))
    torch.cuda.synchronize()
    err = (z.float() - ref).abs()
    assert bool((err <= ref.abs() * 2.0 ** -7 + 1e-6).all())  # one bf16 unit in the last place
