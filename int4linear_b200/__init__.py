"""B200-native INT4 linear layer: Y[M,N] (int32) = X[M,K] (s4) @ W[N,K]^T (s4).

The product is the CUDA library `libint4linear_b200.so` (hand-written sm_100a
kernels behind a C ABI, declared in include/int4linear_b200.h).  This package is
the thin host side over it: the reference's packer and launcher interface, a
seeded operand generator, and the N-sharding driver for several GPUs.  There is
no CPU implementation of the operator here; without the library or without a
B200 the compute calls raise.
"""
from .packer import pack, unpack, pack_bytes, unpack_bytes, pack_device, unpack_device  # noqa: F401
from .data import uniform_s4, uniform_s4_packed  # noqa: F401
from .linear import (  # noqa: F401
    LinearArgs,
    Int4LinearError,
    linear,
    linear_host,
    linear_prepared,
    linear_decode,
    linear_expanded,
    linear_scaled,
    prepare_weights,
    linear_v21_launch,
    last_status,
    launch_count,
    path_for,
    set_path,
    set_overlap,
    set_tail,
    set_fewrows,
    set_two_pass,
    set_tuning,
    PATH_AUTO,
    PATH_TCGEN05,
    PATH_LEGACY,
    PATH_SKINNY,
)

__version__ = "0.1.0"
