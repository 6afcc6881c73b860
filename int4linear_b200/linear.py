"""Host-side mirror of the reference's launcher interface.

Reference                                   here
------------------------------------------  ---------------------------------
struct LinearArgs {X_ptr, W_ptr, Y_ptr,     LinearArgs (same field names/order)
  m, n, k}      kernels/linear_v21.h:62-69
void linear_v21_launch(x_packed_d,          linear_v21_launch(...) -- device
  w_packed_d, y_d, m, n, k)                   pointers or CUDA tensors, blocking,
                kernels/linear_v21.h:760      result complete on return
main() of test/test_correctness.cu:53-63    linear_host(...) -- host arrays in,
  (malloc/H2D/launch/D2H)                     host array out

`linear` is the convenience form for CUDA tensors.  All of them end in the
C ABI of libint4linear_b200.so; none computes anything on the CPU.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from . import _lib

PATH_AUTO, PATH_TCGEN05, PATH_LEGACY, PATH_SKINNY = 0, 1, 2, 3


class Int4LinearError(RuntimeError):
    """A C-ABI call returned a non-zero status."""

    def __init__(self, status: int, where: str):
        self.status = status
        msg = _lib.load().int4_linear_status_string(status).decode()
        super().__init__(f"{where}: {msg} (status {status})")


@dataclass
class LinearArgs:
    """Field-for-field the reference's kernel argument block (kernels/linear_v21.h:62-69)."""
    X_ptr: int
    W_ptr: int
    Y_ptr: int
    m: int
    n: int
    k: int


def _ptr(t) -> int:
    if isinstance(t, int):
        return t
    if hasattr(t, "data_ptr"):
        if not t.is_cuda:
            raise ValueError("expected a CUDA tensor (device pointer)")
        if not t.is_contiguous():
            raise ValueError("tensor must be contiguous")
        return t.data_ptr()
    raise TypeError(f"cannot take a device pointer from {type(t)!r}")


def linear_v21_launch(x_packed_d, w_packed_d, y_d, m: int, n: int, k: int) -> None:
    """Blocking launch on the current device's default stream, as the reference's
    launcher.  Arguments are device pointers (ints) or CUDA tensors.  Unlike the
    reference, which returns nothing and prints only in debug builds, a failure
    raises Int4LinearError."""
    lib = _lib.load()
    lib.int4_linear_launch(_ptr(x_packed_d), _ptr(w_packed_d), _ptr(y_d), m, n, k)
    st = lib.int4_linear_last_status()
    if st != 0:
        raise Int4LinearError(st, "linear_v21_launch")


def launch(args: LinearArgs, stream=None) -> None:
    """Asynchronous launch from a LinearArgs block on `stream` (a torch.cuda.Stream,
    a raw cudaStream_t handle, or None for the current torch stream)."""
    import torch
    lib = _lib.load()
    if stream is None:
        handle = torch.cuda.current_stream().cuda_stream
    elif hasattr(stream, "cuda_stream"):
        handle = stream.cuda_stream
    else:
        handle = int(stream)
    st = lib.int4_linear_launch_async(args.X_ptr, args.W_ptr, args.Y_ptr, args.m, args.n, args.k, handle)
    if st != 0:
        raise Int4LinearError(st, "int4_linear_launch_async")


def linear(x_packed, w_packed, k: int | None = None, out=None, stream=None, bias=None):
    """Y = X @ W^T (+ bias) for packed CUDA tensors.

    x_packed: [m, k/2] uint8 (or [m, k/8] int32) on a B200; w_packed likewise with n rows.
    Returns an [m, n] int32 CUDA tensor (written into `out` when given).  Asynchronous
    on the current torch stream; call last_status() after a synchronize to learn
    about device-side failures.  `bias`: optional CUDA int32 tensor [n], added to every row in the
    kernel epilogue (exact)."""
    import torch
    if not (x_packed.is_cuda and w_packed.is_cuda):
        raise ValueError("linear() needs CUDA tensors; there is no CPU implementation")
    # Row width in bytes without materialising views (this function sits on the per-token path).
    if not (x_packed.is_contiguous() and w_packed.is_contiguous()):
        x_packed, w_packed = x_packed.contiguous(), w_packed.contiguous()
    m, n = x_packed.shape[0], w_packed.shape[0]
    xbytes = x_packed.shape[1] * x_packed.element_size()
    wbytes = w_packed.shape[1] * w_packed.element_size()
    if k is None:
        k = xbytes * 2
    if xbytes * 2 != k or wbytes * 2 != k:
        raise ValueError("packed widths do not match k")
    if out is None:
        out = torch.empty((m, n), dtype=torch.int32, device=x_packed.device)
    elif tuple(out.shape) != (m, n) or out.dtype != torch.int32 or not out.is_contiguous():
        raise ValueError("out must be a contiguous int32 tensor of shape [m, n]")
    if m == 0 or n == 0:
        return out  # nothing to compute (a rank whose shard of W is empty)
    if stream is None:
        handle = torch.cuda.current_stream(x_packed.device).cuda_stream
    else:
        handle = stream.cuda_stream if hasattr(stream, "cuda_stream") else int(stream)
    if bias is not None:
        if bias.dtype != torch.int32 or bias.numel() != n or not bias.is_cuda:
            raise ValueError("bias must be a CUDA int32 tensor with n elements")
        bias = bias.contiguous()
    lib = _lib.load()
    dev = x_packed.device.index
    switch = dev is not None and dev != torch.cuda.current_device()
    if switch:
        prev = torch.cuda.current_device()
        torch.cuda.set_device(dev)
    try:
        st = lib.int4_linear_bias_launch_async(x_packed.data_ptr(), w_packed.data_ptr(),
                                               bias.data_ptr() if bias is not None else None,
                                               out.data_ptr(), m, n, k, handle)
    finally:
        if switch:
            torch.cuda.set_device(prev)
    if st != 0:
        raise Int4LinearError(st, "int4_linear_bias_launch_async")
    return out


def linear_decode(x_packed, w_packed, out=None, bias=None, weights_stationary=True, x_not_pending=False, stream=None):
    """Y = X @ W^T (+ bias) for a stream of small-batch launches (int4_linear_decode_launch_async):
    `weights_stationary` promises that nothing queued before this launch writes W, `x_not_pending`
    the same for X; with a promise consecutive launches overlap on the GPU."""
    import torch
    xb = x_packed.contiguous().view(torch.uint8)
    wb = w_packed.contiguous().view(torch.uint8)
    m, n, k = xb.shape[0], wb.shape[0], xb.shape[1] * 2
    if wb.shape[1] * 2 != k:
        raise ValueError("packed widths do not match")
    if x_not_pending and not weights_stationary:
        raise ValueError("x_not_pending is valid only together with weights_stationary")
    if out is None:
        out = torch.empty((m, n), dtype=torch.int32, device=xb.device)
    elif tuple(out.shape) != (m, n) or out.dtype != torch.int32 or not out.is_contiguous():
        raise ValueError("out must be a contiguous int32 tensor of shape [m, n]")
    promises = (1 if weights_stationary else 0) | (2 if x_not_pending else 0)
    handle = (stream or torch.cuda.current_stream(xb.device)).cuda_stream
    with torch.cuda.device(xb.device):
        st = _lib.load().int4_linear_decode_launch_async(
            xb.data_ptr(), wb.data_ptr(), bias.data_ptr() if bias is not None else None, out.data_ptr(),
            m, n, k, promises, handle)
    if st != 0:
        raise Int4LinearError(st, "int4_linear_decode_launch_async")
    return out


def linear_scaled(x_packed, w_packed, row_scale=None, col_scale=None, bias=None, out=None, stream=None, dtype=None):
    """16-bit Y = (X @ W^T) * row_scale[:, None] * col_scale[None, :] + bias (see
    int4_linear_scaled_launch_async).  Scales and bias are CUDA float32 vectors or None; `dtype` is
    torch.bfloat16 (default) or torch.float16 (taken from `out` when that is given)."""
    import torch
    xb = x_packed.contiguous().view(torch.uint8)
    wb = w_packed.contiguous().view(torch.uint8)
    m, n, k = xb.shape[0], wb.shape[0], xb.shape[1] * 2
    if wb.shape[1] * 2 != k:
        raise ValueError("packed widths do not match")
    for name, t, length in (("row_scale", row_scale, m), ("col_scale", col_scale, n), ("bias", bias, n)):
        if t is not None and (t.dtype != torch.float32 or t.numel() != length or not t.is_cuda or not t.is_contiguous()):
            raise ValueError(f"{name} must be a contiguous CUDA float32 tensor with {length} elements")
    if out is None:
        out = torch.empty((m, n), dtype=dtype or torch.bfloat16, device=xb.device)
    if out.dtype not in (torch.bfloat16, torch.float16) or (dtype is not None and out.dtype != dtype):
        raise ValueError("the scaled output is bfloat16 or float16")
    if tuple(out.shape) != (m, n) or not out.is_contiguous() or out.device != xb.device:
        raise ValueError("out must be a contiguous [m, n] tensor on the operands' device")
    handle = (stream or torch.cuda.current_stream(xb.device)).cuda_stream
    ptr = lambda t: t.data_ptr() if t is not None else None  # noqa: E731
    lib = _lib.load()
    fn = lib.int4_linear_scaled_f16_launch_async if out.dtype == torch.float16 else lib.int4_linear_scaled_launch_async
    with torch.cuda.device(xb.device):
        st = fn(xb.data_ptr(), wb.data_ptr(), ptr(row_scale), ptr(col_scale), ptr(bias), out.data_ptr(), m, n, k, handle)
    if st != 0:
        raise Int4LinearError(st, "int4_linear_scaled_launch_async")
    return out


def prepare_weights(w_packed, k: int | None = None, stream=None):
    """Expand packed CUDA weights [n, k/2] once into the [n, k] uint8 layout that
    linear_prepared consumes (see int4_linear_prepare_weights)."""
    import torch
    wb = w_packed.contiguous().view(torch.uint8)
    n = wb.shape[0]
    k = k or wb.shape[1] * 2
    out = torch.empty((n, k), dtype=torch.uint8, device=wb.device)
    handle = (stream or torch.cuda.current_stream(wb.device)).cuda_stream
    with torch.cuda.device(wb.device):
        st = _lib.load().int4_linear_prepare_weights(wb.data_ptr(), out.data_ptr(), n, k, handle)
    if st != 0:
        raise Int4LinearError(st, "int4_linear_prepare_weights")
    return out


def linear_prepared(x_packed, w_expanded, out=None, bias=None, stream=None):
    """Y = X @ W^T (+ bias) with weights from prepare_weights (asynchronous)."""
    import torch
    xb = x_packed.contiguous().view(torch.uint8)
    m, k = xb.shape[0], xb.shape[1] * 2
    n = w_expanded.shape[0]
    if w_expanded.shape[1] != k or w_expanded.dtype != torch.uint8 or not w_expanded.is_contiguous():
        raise ValueError("w_expanded must be the contiguous [n, k] uint8 tensor made by prepare_weights")
    if out is None:
        out = torch.empty((m, n), dtype=torch.int32, device=xb.device)
    elif tuple(out.shape) != (m, n) or out.dtype != torch.int32 or not out.is_contiguous():
        raise ValueError("out must be a contiguous int32 tensor of shape [m, n]")
    handle = (stream or torch.cuda.current_stream(xb.device)).cuda_stream
    with torch.cuda.device(xb.device):
        st = _lib.load().int4_linear_launch_prepared_async(
            xb.data_ptr(), w_expanded.data_ptr(), bias.data_ptr() if bias is not None else None,
            out.data_ptr(), m, n, k, handle)
    if st != 0:
        raise Int4LinearError(st, "int4_linear_launch_prepared_async")
    return out


def linear_expanded(x_expanded, w_expanded, out=None, bias=None, stream=None):
    """Y = X @ W^T (+ bias) with BOTH operands already expanded by prepare_weights ([m, k] and
    [n, k] uint8): the pure 8-bit GEMM of the two-pass path (asynchronous)."""
    import torch
    m, k = x_expanded.shape
    n = w_expanded.shape[0]
    for t in (x_expanded, w_expanded):
        if t.dtype != torch.uint8 or not t.is_contiguous() or t.shape[1] != k or not t.is_cuda:
            raise ValueError("operands must be contiguous CUDA uint8 tensors [rows, k] made by prepare_weights")
    if out is None:
        out = torch.empty((m, n), dtype=torch.int32, device=x_expanded.device)
    elif tuple(out.shape) != (m, n) or out.dtype != torch.int32 or not out.is_contiguous():
        raise ValueError("out must be a contiguous int32 tensor of shape [m, n]")
    handle = (stream or torch.cuda.current_stream(x_expanded.device)).cuda_stream
    with torch.cuda.device(x_expanded.device):
        st = _lib.load().int4_linear_launch_expanded_async(
            x_expanded.data_ptr(), w_expanded.data_ptr(), bias.data_ptr() if bias is not None else None,
            out.data_ptr(), m, n, k, handle)
    if st != 0:
        raise Int4LinearError(st, "int4_linear_launch_expanded_async")
    return out


def linear_host(x_packed: np.ndarray, w_packed: np.ndarray, k: int, out: np.ndarray | None = None,
                w_resident: bool = False) -> np.ndarray:
    """The whole host-side sequence of the reference's correctness program
    (allocate, upload, launch, download; test/test_correctness.cu:53-63) for
    operands in host memory.  Returns (and fills) an [m, n] int32 numpy array."""
    x_packed = np.ascontiguousarray(x_packed)
    w_packed = np.ascontiguousarray(w_packed)
    m, n = x_packed.shape[0], w_packed.shape[0]
    if x_packed.nbytes != m * k // 2 or w_packed.nbytes != n * k // 2:
        raise ValueError("packed sizes do not match k")
    if out is None:
        out = np.empty((m, n), dtype=np.int32)
    st = _lib.load().int4_linear_host(x_packed.ctypes.data, w_packed.ctypes.data, out.ctypes.data,
                                      m, n, k, 1 if w_resident else 0)
    if st != 0:
        raise Int4LinearError(st, "int4_linear_host")
    return out


def last_status() -> int:
    return _lib.load().int4_linear_last_status()


def launch_count() -> int:
    return _lib.load().int4_linear_launch_count()


def set_path(path: int) -> int:
    return _lib.load().int4_linear_set_path(path)


def set_tuning(tile_n: int = 0, direct_store: bool = False, cta_pairs: int = -1) -> None:
    st = _lib.load().int4_linear_set_tuning(tile_n, 1 if direct_store else 0, cta_pairs)
    if st != 0:
        raise Int4LinearError(st, "int4_linear_set_tuning")


def set_two_pass(mode: int) -> int:
    """-1 automatic, 0 never, 1 always for the tensor-memory family (int4_linear_set_two_pass)."""
    st = _lib.load().int4_linear_set_two_pass(mode)
    if st != 0:
        raise Int4LinearError(st, "int4_linear_set_two_pass")
    return st


def set_fewrows(mode: int) -> None:
    """-1 by shape, 0 never, 1 whenever M <= 128: the few-rows kernel with W in tensor memory (int4_linear_set_fewrows)."""
    st = _lib.load().int4_linear_set_fewrows(mode)
    if st != 0:
        raise Int4LinearError(st, "int4_linear_set_fewrows")


def set_tail(mode: int) -> None:
    """-1 automatic, 0 whole tiles, 1 half-width items, 2 last wave cut along K (int4_linear_set_tail)."""
    st = _lib.load().int4_linear_set_tail(mode)
    if st != 0:
        raise Int4LinearError(st, "int4_linear_set_tail")


def set_overlap(mode: int) -> int:
    """0 off, 1 weights stationary, 2 weights and X stationary (see int4_linear_set_overlap)."""
    r = _lib.load().int4_linear_set_overlap(mode)
    if r < 0:
        raise Int4LinearError(-r, "int4_linear_set_overlap")
    return r


def path_for(m: int, n: int, k: int) -> int:
    r = _lib.load().int4_linear_path_for(m, n, k)
    if r < 0:
        raise Int4LinearError(-r, "int4_linear_path_for")
    return r


def linear_gather(x_packed, w_shard_packed, y_full_ptrs, col_offset: int, n_total: int,
                  k: int | None = None, stream=None, bias=None) -> None:
    """This rank's column block of Y = X @ W^T, stored by the kernel's epilogue into the full
    [m, n_total] int32 result of EVERY rank: `y_full_ptrs` lists one device address per rank
    (this rank's own buffer and its peers' buffers mapped into this process).  Asynchronous;
    the full Y is complete on a rank only after all ranks' launches have finished.  No
    reference counterpart (the reference is single-GPU)."""
    import ctypes
    import torch
    if not (x_packed.is_cuda and w_shard_packed.is_cuda):
        raise ValueError("linear_gather() needs CUDA tensors; there is no CPU implementation")
    x_packed, w_shard_packed = x_packed.contiguous(), w_shard_packed.contiguous()
    m, n_local = x_packed.shape[0], w_shard_packed.shape[0]
    xbytes = x_packed.shape[1] * x_packed.element_size()
    if k is None:
        k = xbytes * 2
    if xbytes * 2 != k or w_shard_packed.shape[1] * w_shard_packed.element_size() * 2 != k:
        raise ValueError("packed widths do not match k")
    ptrs = [int(a) for a in y_full_ptrs]
    arr = (ctypes.c_void_p * len(ptrs))(*ptrs)
    if stream is None:
        handle = torch.cuda.current_stream(x_packed.device).cuda_stream
    else:
        handle = stream.cuda_stream if hasattr(stream, "cuda_stream") else int(stream)
    if bias is not None:
        if bias.dtype != torch.int32 or bias.numel() != n_local or not bias.is_cuda:
            raise ValueError("bias must be a CUDA int32 tensor with n_local elements")
        bias = bias.contiguous()
    lib = _lib.load()
    with torch.cuda.device(x_packed.device):
        st = lib.int4_linear_launch_gather_async(x_packed.data_ptr(), w_shard_packed.data_ptr(),
                                                 bias.data_ptr() if bias is not None else None,
                                                 arr, len(ptrs), col_offset, m, n_local, n_total, k, handle)
    if st != 0:
        raise Int4LinearError(st, "int4_linear_launch_gather_async")
