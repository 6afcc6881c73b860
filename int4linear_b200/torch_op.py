"""PyTorch operator binding over the C ABI.

    import int4linear_b200.torch_op            # registers the ops
    y = torch.ops.int4linear.linear(x_packed, w_packed)     # [m, k/2] u8, [n, k/2] u8 -> [m, n] i32
    p = torch.ops.int4linear.pack(values)                   # [m, n] i8/i32 -> [m, ceil(n/8)] i32

The ops run on the tensors' device and the current CUDA stream, have shape-inference ("fake")
implementations so they trace under FakeTensor / torch.compile graphs, and have no CPU kernels:
the operator exists only as the sm_100a library.  This is the natural caller of the launcher the
reference exposes as linear_v21_launch (kernels/linear_v21.h:760) on a PyTorch stack; the
reference itself has no Python binding.
"""
from __future__ import annotations

import torch

from .linear import linear as _linear_fn
from .packer import pack_device as _pack_device


@torch.library.custom_op("int4linear::linear", mutates_args=(), device_types="cuda")
def linear(x_packed: torch.Tensor, w_packed: torch.Tensor) -> torch.Tensor:
    return _linear_fn(x_packed, w_packed)


@linear.register_fake
def _(x_packed, w_packed):
    if x_packed.dim() != 2 or w_packed.dim() != 2:
        raise ValueError("int4linear::linear expects 2-D packed operands")
    bx = x_packed.shape[1] * x_packed.element_size()
    bw = w_packed.shape[1] * w_packed.element_size()
    if bx != bw:
        raise ValueError("packed operands disagree on K")
    return x_packed.new_empty((x_packed.shape[0], w_packed.shape[0]), dtype=torch.int32)


@torch.library.custom_op("int4linear::pack", mutates_args=(), device_types="cuda")
def pack(values: torch.Tensor) -> torch.Tensor:
    return _pack_device(values)


@pack.register_fake
def _(values):
    return values.new_empty((values.shape[0], (values.shape[1] + 7) // 8), dtype=torch.int32)
