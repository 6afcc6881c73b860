"""PyTorch operator binding over the C ABI.

    import int4linear_b200.torch_op            # registers the ops
    y = torch.ops.int4linear.linear(x_packed, w_packed)     # [m, k/2] u8, [n, k/2] u8 -> [m, n] i32
    z = torch.ops.int4linear.linear_scaled(x_packed, w_packed, row_scale, col_scale, bias)   # -> [m, n] bf16
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
from .linear import linear_scaled as _linear_scaled_fn
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


@torch.library.custom_op("int4linear::linear_scaled", mutates_args=(), device_types="cuda")
def linear_scaled(x_packed: torch.Tensor, w_packed: torch.Tensor, row_scale: torch.Tensor | None,
                  col_scale: torch.Tensor | None, bias: torch.Tensor | None) -> torch.Tensor:
    """bf16((X @ W^T) * row_scale[:, None] * col_scale[None, :] + bias): the dequantising epilogue of
    int4_linear_scaled_launch_async.  Scales and bias are float32 CUDA vectors or None."""
    return _linear_scaled_fn(x_packed, w_packed, row_scale, col_scale, bias)


@linear_scaled.register_fake
def _(x_packed, w_packed, row_scale, col_scale, bias):
    if x_packed.dim() != 2 or w_packed.dim() != 2:
        raise ValueError("int4linear::linear_scaled expects 2-D packed operands")
    if x_packed.shape[1] * x_packed.element_size() != w_packed.shape[1] * w_packed.element_size():
        raise ValueError("packed operands disagree on K")
    return x_packed.new_empty((x_packed.shape[0], w_packed.shape[0]), dtype=torch.bfloat16)


@torch.library.custom_op("int4linear::pack", mutates_args=(), device_types="cuda")
def pack(values: torch.Tensor) -> torch.Tensor:
    return _pack_device(values)


@pack.register_fake
def _(values):
    return values.new_empty((values.shape[0], (values.shape[1] + 7) // 8), dtype=torch.int32)
