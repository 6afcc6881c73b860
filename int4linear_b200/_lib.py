"""ctypes binding of libint4linear_b200.so (the C ABI in include/int4linear_b200.h)."""
from __future__ import annotations

import ctypes
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libint4linear_b200.so")

# Every symbol include/int4linear_b200.h declares, with its ctypes signature.
_VP, _I, _LL = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
SYMBOLS = {
    "int4_linear_launch": (None, [_VP, _VP, _VP, _I, _I, _I]),
    "int4_linear_launch_async": (_I, [_VP, _VP, _VP, _I, _I, _I, _VP]),
    "int4_linear_bias_launch_async": (_I, [_VP, _VP, _VP, _VP, _I, _I, _I, _VP]),
    "int4_linear_decode_launch_async": (_I, [_VP, _VP, _VP, _VP, _I, _I, _I, _I, _VP]),
    "int4_linear_scaled_launch_async": (_I, [_VP, _VP, _VP, _VP, _VP, _VP, _I, _I, _I, _VP]),
    "int4_linear_scaled_f16_launch_async": (_I, [_VP, _VP, _VP, _VP, _VP, _VP, _I, _I, _I, _VP]),
    "int4_linear_launch_gather_async": (_I, [_VP, _VP, _VP, ctypes.POINTER(ctypes.c_void_p), _I, _I, _I, _I, _I, _I, _VP]),
    "int4_linear_prepare_weights": (_I, [_VP, _VP, _I, _I, _VP]),
    "int4_linear_launch_prepared_async": (_I, [_VP, _VP, _VP, _VP, _I, _I, _I, _VP]),
    "int4_linear_launch_expanded_async": (_I, [_VP, _VP, _VP, _VP, _I, _I, _I, _VP]),
    "int4_linear_launch_static_scratch_async": (_I, [_VP, _VP, _VP, _VP, _I, _I, _I, _VP]),
    "int4_linear_host": (_I, [_VP, _VP, _VP, _I, _I, _I, _I]),
    "int4_linear_pack_host": (None, [_VP, _VP, _I, _I]),
    "int4_linear_unpack_host": (None, [_VP, _VP, _I, _I]),
    "int4_linear_pack_i32": (_I, [_VP, _VP, _I, _I, _VP]),
    "int4_linear_pack_i8": (_I, [_VP, _VP, _I, _I, _VP]),
    "int4_linear_unpack_i32": (_I, [_VP, _VP, _I, _I, _VP]),
    "int4_linear_probe_stream_read": (_I, [_VP, ctypes.c_ulonglong, _VP, _VP]),
    "int4_linear_selftest_timeout": (_I, [_I]),
    "int4_linear_last_status": (_I, []),
    "int4_linear_status_string": (ctypes.c_char_p, [_I]),
    "int4_linear_set_path": (_I, [_I]),
    "int4_linear_set_tuning": (_I, [_I, _I, _I]),
    "int4_linear_set_overlap": (_I, [_I]),
    "int4_linear_set_tail": (_I, [_I]),
    "int4_linear_set_fewrows": (_I, [_I]),
    "int4_linear_set_two_pass": (_I, [_I]),
    "int4_linear_path_for": (_I, [_I, _I, _I]),
    "int4_linear_device_info": (_I, [_I]),
    "int4_linear_launch_count": (_LL, []),
    "int4_linear_version": (_I, []),
}

_lib = None


def load() -> ctypes.CDLL:
    """Load the library.  There is no fallback: a missing library is an error."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m int4linear_b200.build` "
                "(needs nvcc); this package has no non-CUDA implementation")
        lib = ctypes.CDLL(LIB_PATH)
        for name, (restype, argtypes) in SYMBOLS.items():
            fn = getattr(lib, name)
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = lib
    return _lib
