"""ctypes binding of ``libmor_b200.so`` (the C ABI declared in ``include/mor_b200.h``).

This is what a host runtime without PyTorch would bind.  The library is loaded from
this directory; if it is missing the import fails -- there is no CPU fallback.
Pointers are plain integers (``tensor.data_ptr()``), the stream is a ``cudaStream_t``
handle as an integer (``torch.cuda.current_stream().cuda_stream``).
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libmor_b200.so")

BF16, FP32 = 0, 1
E4M3, E5M2, E3M2, E2M3 = 0, 1, 2, 3
SF_FP32, SF_E8 = 1, 2
OP_BLOCK_SCALING, OP_CHANNEL_SCALING, OP_E8MX, OP_AMAX_NNZ = 1, 2, 3, 4

# name -> (restype, argtypes); mirrors include/mor_b200.h declaration by declaration
_vp, _i, _i64, _d, _sz = C.c_void_p, C.c_int, C.c_int64, C.c_double, C.c_size_t
SIGNATURES = {
    "mor_b200_version": (_i, []),
    "mor_b200_status_string": (C.c_char_p, [_i]),
    "mor_b200_debug_kernel_selection": (None, [_i]),
    "mor_b200_workspace_bytes": (_sz, [_i, _i64, _i64, _i, _i]),
    "mor_b200_fake_quantize": (_i, [_vp, _vp, _vp, _i, _i64, _i64, _i, _i, _d, _i, _i, _vp]),
    "mor_b200_quant_dequant": (_i, [_vp, _vp, _i64, _i64, _i, _vp]),
    "mor_b200_e4m3_with_e8_scale": (_i, [_vp, _vp, _i64, _i64, _i, _vp]),
    "mor_b200_block_scaling": (_i, [_vp, _vp, _i, _i64, _i64, _i, _i, _d, _i, _vp, _vp, _vp, _i, _vp, _vp, _sz, _vp]),
    "mor_b200_block_scaling_static": (_i, [_vp, _vp, _i, _i64, _i64, _i, _i, _d, _i, _vp, _vp, _vp, _i, _vp, _vp]),
    "mor_b200_channel_scaling": (_i, [_vp, _vp, _i, _i64, _i64, _i, _i, _d, _i, _vp, _vp, _vp, _i, _vp, _vp, _sz, _vp]),
    "mor_b200_e8mx": (_i, [_vp, _vp, _i64, _i64, _i, _i, _vp, _sz, _vp]),
    "mor_b200_fake_quantize_group": (_i, [_vp, _vp, _vp, _i, _i64, _i64, _i, _i, _i, _vp]),
    "mor_b200_quantize_mx": (_i, [_vp, _vp, _vp, _i64, _i64, _i, _i, _vp]),
    "mor_b200_quantize_mx_fp6": (_i, [_vp, _vp, _vp, _i64, _i64, _i, _vp]),
    "mor_b200_quantize_scaled": (_i, [_vp, _vp, _vp, _i, _i64, _i64, _i, _i, _i, _vp, _vp, _vp, _sz, _vp]),
    "mor_b200_block_scaling_delayed": (_i, [_vp, _vp, _i, _i64, _i64, _i, _i, _d, _i, _vp, _vp, _vp, _vp, _i, _vp, _vp, _sz, _vp]),
    "mor_b200_block_scaling_delayed_t": (_i, [_vp, _vp, _vp, _i, _i64, _i64, _i, _i, _d, _i, _vp, _vp, _vp, _vp, _i, _vp, _vp, _sz, _vp]),
    "mor_b200_scaling_amax": (_i, [_i, _vp, _i, _i64, _i64, _i, _i, _vp, _vp, _vp, _sz, _vp]),
    "mor_b200_scaling_cast": (_i, [_i, _vp, _vp, _i, _i64, _i64, _i, _i, _i, _vp, _vp, _vp, _sz, _vp]),
    "mor_b200_scaling_num_errors": (_i64, [_i, _i64, _i64, _i, _i]),
    "mor_b200_scaling_error_stride": (_i, [_i, _i, _i]),
    "mor_b200_scaling_finalize": (_i, [_vp, _i64, _i, _vp, _d, _vp, _vp, _vp, _sz, _vp]),
    "mor_b200_scaling_fallback": (_i, [_vp, _vp, _i64, _vp, _vp]),
    "mor_b200_amax_nnz": (_i, [_vp, _i, _i64, _vp, _vp, _vp, _sz, _vp]),
    "mor_b200_p2p_alloc": (_i, [_i, _sz, _vp, _vp]),
    "mor_b200_p2p_open": (_i, [_i, _vp, _vp]),
    "mor_b200_p2p_close": (_i, [_i, _vp]),
    "mor_b200_p2p_free": (_i, [_i, _vp]),
    "mor_b200_p2p_bytes": (_sz, [_i, _i64]),
    "mor_b200_p2p_set_wait_limit": (None, [C.c_uint32]),
    "mor_b200_p2p_error_offset": (_sz, [_i, _i64, C.c_uint32]),
    "mor_b200_p2p_exchange_scalars": (_i, [_vp, _vp, _vp, _i, _i, C.c_uint32, _vp, _vp, _vp]),
    "mor_b200_scaling_amax_p2p": (_i, [_i, _vp, _i, _i64, _i64, _i, _i, _vp, _sz, _vp, _vp, _i, _i, C.c_uint32, _vp, _vp, _vp]),
    "mor_b200_p2p_exchange_errors": (_i, [_vp, _i64, _vp, _vp, _i, _i, C.c_uint32, _vp, _vp]),
}


ERR_UNSUPPORTED_SHAPE = -2   # MOR_B200_ERR_UNSUPPORTED_SHAPE


class MorB200Error(RuntimeError):
    """A C-ABI call returned a non-zero status."""

    def __init__(self, fn: str, status: int, text: str):
        super().__init__(f"{fn}: {text} (status {status})")
        self.status = status


_lib = None


def lib() -> C.CDLL:
    """Load libmor_b200.so.  Raises if it has not been built: no fallback exists."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python mor_b200/build.py` "
                "(nvcc, sm_100a).  mor_b200 has no CPU or PyTorch fallback.")
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def call(name: str, *args) -> None:
    """Invoke an int-status entry point and raise MorB200Error on failure."""
    rc = getattr(lib(), name)(*args)
    if rc != 0:
        raise MorB200Error(name, rc, lib().mor_b200_status_string(rc).decode())


def workspace_bytes(op: int, rows: int, cols: int, brows: int, bcols: int) -> int:
    return int(lib().mor_b200_workspace_bytes(op, rows, cols, brows, bcols))
