"""ctypes front end of the CPU oracle (``oracle/mor_oracle.c``).  TEST INFRASTRUCTURE.

Only ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline legs of ``bench.py``
may import this module; nothing under ``mor_b200/`` does.  Tensors cross the
boundary as numpy arrays: bf16 data as ``uint16`` bit patterns, fp32 data as
``float32``.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libmor_oracle.so")

FMT_E4M3, FMT_E5M2, FMT_E3M2, FMT_E2M3 = 0, 1, 2, 3
SF_FP32, SF_E8 = 1, 2

ASSERT_E8_EXPONENT, ASSERT_SCALE_1E30, ASSERT_NNZ_ZERO, ASSERT_AMAX_ZERO = 1, 2, 4, 8


def build(force: bool = False) -> str:
    """Compile the oracle with gcc if the library is missing or older than its source."""
    src = os.path.join(_HERE, "mor_oracle.c")
    stale = (not os.path.exists(_LIB_PATH)) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src)
    if force or stale:
        subprocess.run(["make", "-C", _HERE, "all"], check=True, capture_output=True)
    return _LIB_PATH


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(_LIB_PATH)
        f32, i32, i64, dbl, vp = C.c_float, C.c_int, C.c_int64, C.c_double, C.c_void_p
        L.mor_o_bf16_to_fp32.restype = f32
        L.mor_o_bf16_to_fp32.argtypes = [C.c_uint32]
        L.mor_o_fp32_to_bf16.restype = C.c_uint32
        L.mor_o_fp32_to_bf16.argtypes = [f32]
        for name in ("mor_o_quant_dequant_custom", "mor_o_quant_dequant_satfinite"):
            getattr(L, name).restype = f32
            getattr(L, name).argtypes = [f32, i32]
        L.mor_o_sqdd.restype = f32
        L.mor_o_sqdd.argtypes = [f32, f32, i32, i32]
        L.mor_o_sqdd_e8_custom.restype = f32
        L.mor_o_sqdd_e8_custom.argtypes = [f32, f32, i32]
        L.mor_o_scaling_factor.restype = f32
        L.mor_o_scaling_factor.argtypes = [i32, f32, f32]
        L.mor_o_e8m_round.restype = f32
        L.mor_o_e8m_round.argtypes = [f32, i32]
        L.mor_o_e8mx_scale.restype = f32
        L.mor_o_e8mx_scale.argtypes = [f32, i32, i32]
        L.mor_o_assert_flags.restype = i32
        L.mor_o_fake_quantize.argtypes = [vp, vp, vp, i64, i64, i32, i32, dbl, i32, i32]
        L.mor_o_fake_quantize_f32.argtypes = [vp, vp, vp, i64, i64, i32, i32, dbl, i32, i32]
        L.mor_o_block_scaling.argtypes = [vp, vp, i32, i64, i64, i32, i32, dbl, i32, vp, vp, vp, vp, vp, vp, vp]
        L.mor_o_channel_scaling.argtypes = [vp, vp, i32, i64, i64, i32, i32, dbl, i32, vp, vp, vp, vp]
        L.mor_o_e8mx.argtypes = [vp, vp, i64, i64, i32, i32, vp]
        L.mor_o_quant_dequant.argtypes = [vp, vp, i64, i32]
        L.mor_o_e4m3_with_e8_scale.argtypes = [vp, vp, i64, i32]
        L.mor_o_fake_quantize_group.argtypes = [vp, vp, i32, vp, i64, i64, i32, i32, i32, i32]
        L.mor_o_amax_nnz.argtypes = [vp, i32, i64, vp, vp]
        L.mor_o_quantize_mx.argtypes = [vp, vp, vp, i64, i64, i32, i32]
        L.mor_o_dequantize_mx.argtypes = [vp, vp, vp, i64, i64, i32, i32]
        L.mor_o_quantize_scaled.argtypes = [vp, i32, vp, vp, i64, i64, i32, i32, i32, vp, vp]
        L.mor_o_dequantize_scaled.argtypes = [vp, vp, vp, i32, i64, i64, i32, i32]
        L.mor_o_finalize.restype = f32
        L.mor_o_finalize.argtypes = [vp, i64, i32, i64, dbl, vp]
        L.mor_o_num_threads.restype = i32
        L.mor_o_set_num_threads.argtypes = [i32]
        _lib = L
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _check_in(a: np.ndarray):
    if a.dtype == np.uint16:
        return 0
    if a.dtype == np.float32:
        return 1
    raise TypeError("oracle inputs are uint16 (bf16 bits) or float32 arrays")


class OracleError(ValueError):
    """The oracle refuses arguments that the reference rejects or leaves undefined."""


def _rc(rc: int, what: str):
    if rc != 0:
        raise OracleError(f"{what}: oracle status {rc}")


def assert_flags() -> int:
    return lib().mor_o_assert_flags()


def clear_assert_flags() -> None:
    lib().mor_o_clear_assert_flags()


def set_num_threads(n: int) -> None:
    lib().mor_o_set_num_threads(int(n))


def num_threads() -> int:
    return lib().mor_o_num_threads()


# --------------------------------------------------------------------------- ops
def fake_quantize(x: np.ndarray, brows: int, bcols: int, clamp: float, mode: int, sf_type: int):
    """mor.ops.fake_quantize: returns (out, meta)."""
    x = np.ascontiguousarray(x)
    is_f32 = _check_in(x)
    rows, cols = x.shape
    out = np.empty_like(x)
    gy = (rows - 1) // brows + 1
    gx = (cols // 2 - 1) // max(bcols // 2, 1) + 1
    meta = np.full((gy, gx), -1, dtype=np.int32)
    fn = lib().mor_o_fake_quantize_f32 if is_f32 else lib().mor_o_fake_quantize
    _rc(fn(_p(x), _p(out), _p(meta), rows, cols, brows, bcols, float(clamp), mode, sf_type), "fake_quantize")
    return out, meta


def _scaling(fn, x, brows, bcols, thr, ss, extra=()):
    x = np.ascontiguousarray(x)
    is_f32 = _check_in(x)
    rows, cols = x.shape
    out = np.empty_like(x)
    meta = np.zeros(1, np.int32)
    gamax = np.zeros(1, np.float32)
    gnnz = np.zeros(1, np.int64)
    gerr = np.zeros(1, np.float32)
    return x, is_f32, rows, cols, out, meta, gamax, gnnz, gerr


def block_scaling(x, brows, bcols, thr, ss, global_amax=None, want_blocks=False):
    """mor.ops.fake_quantize_block_scaling: returns (out, meta, global_amax, global_nnz, global_error)
    (+ block_amax, block_error when want_blocks).  global_amax overrides the tensor amax
    (row-sharded use)."""
    x, is_f32, rows, cols, out, meta, gamax, gnnz, gerr = _scaling(None, x, brows, bcols, thr, ss)
    ext = None if global_amax is None else np.array([global_amax], np.float32)
    nb = (rows // brows) * (cols // bcols) if brows and bcols else 0
    ba = np.zeros(max(nb, 1), np.float32)
    be = np.zeros(max(nb, 1), np.float32)
    _rc(lib().mor_o_block_scaling(_p(x), _p(out), is_f32, rows, cols, brows, bcols, float(thr), ss, _p(ext),
                                  _p(meta), _p(gamax), _p(gnnz), _p(gerr), _p(ba), _p(be)), "block_scaling")
    res = (out, int(meta[0]), gamax[0], int(gnnz[0]), gerr[0])
    return res + (ba[:nb], be[:nb]) if want_blocks else res


def channel_scaling(x, brows, bcols, thr, ss):
    """mor.ops.fake_quantize_channel_scaling: (out, meta, global_amax, global_nnz, global_error)."""
    x, is_f32, rows, cols, out, meta, gamax, gnnz, gerr = _scaling(None, x, brows, bcols, thr, ss)
    _rc(lib().mor_o_channel_scaling(_p(x), _p(out), is_f32, rows, cols, brows, bcols, float(thr), ss,
                                    _p(meta), _p(gamax), _p(gnnz), _p(gerr)), "channel_scaling")
    return out, int(meta[0]), gamax[0], int(gnnz[0]), gerr[0]


def e8mx(x, qtype, strategy):
    x = np.ascontiguousarray(x)
    assert x.dtype == np.uint16
    rows, cols = x.shape
    out = np.empty_like(x)
    gamax = np.zeros(1, np.float32)
    _rc(lib().mor_o_e8mx(_p(x), _p(out), rows, cols, qtype, strategy, _p(gamax)), "e8mx")
    return out, gamax[0]


def quant_dequant(x, fmt):
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty_like(x)
    _rc(lib().mor_o_quant_dequant(_p(x), _p(out), x.size, fmt), "quant_dequant")
    return out


def e4m3_with_e8_scale(x, rne: bool):
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty_like(x)
    _rc(lib().mor_o_e4m3_with_e8_scale(_p(x), _p(out), x.size, int(bool(rne))), "e4m3_with_e8_scale")
    return out


def fake_quantize_group(x, brows, bcols, fmt, sf_type, want_scales=False):
    x = np.ascontiguousarray(x)
    is_f32 = _check_in(x)
    rows, cols = x.shape
    out = np.empty_like(x)
    nb = (rows // brows) * (cols // bcols)
    scales = np.zeros(nb, np.float32) if want_scales else None
    _rc(lib().mor_o_fake_quantize_group(_p(x), _p(out), is_f32, _p(scales), rows, cols, brows, bcols, fmt, sf_type),
        "fake_quantize_group")
    return (out, scales) if want_scales else out


def quantize_mx(x, bcols, fmt):
    """Real quantized form of ``fake_quantize_group`` with a power-of-two scale: (codes uint8 [rows, cols],
    E8M0 scale bytes uint8 [rows, cols // bcols]); element = decode(code) * 2**(scale - 127)."""
    x = np.ascontiguousarray(x)
    if x.dtype != np.uint16:
        raise TypeError("bf16 bit patterns (uint16) only")
    rows, cols = x.shape
    payload = np.zeros((rows, cols), np.uint8)
    scales = np.zeros((rows, cols // bcols), np.uint8)
    _rc(lib().mor_o_quantize_mx(_p(x), _p(payload), _p(scales), rows, cols, bcols, fmt), "quantize_mx")
    return payload, scales


def pack_fp6(codes):
    """Six-bit codes (one per byte, [rows, cols], cols a multiple of 8) -> [rows, cols * 3 / 4] bytes: every run of
    eight codes is a little-endian 48-bit group with code i in bits [6 i, 6 i + 6)."""
    c = np.ascontiguousarray(codes, dtype=np.uint8)
    rows, cols = c.shape
    g = c.reshape(rows, cols // 8, 8).astype(np.uint64)
    word = np.zeros((rows, cols // 8), np.uint64)
    for i in range(8):
        word |= (g[:, :, i] & np.uint64(63)) << np.uint64(6 * i)
    out = np.zeros((rows, cols // 8, 6), np.uint8)
    for k in range(6):
        out[:, :, k] = ((word >> np.uint64(8 * k)) & np.uint64(255)).astype(np.uint8)
    return out.reshape(rows, cols * 3 // 4)


def dequantize_mx(payload, scales, bcols, fmt):
    payload = np.ascontiguousarray(payload, dtype=np.uint8)
    scales = np.ascontiguousarray(scales, dtype=np.uint8)
    rows, cols = payload.shape
    out = np.zeros((rows, cols), np.uint16)
    _rc(lib().mor_o_dequantize_mx(_p(payload), _p(scales), _p(out), rows, cols, bcols, fmt), "dequantize_mx")
    return out


def quantize_scaled(x, brows, bcols, ss, global_amax=None):
    """Real quantized form of block / channel scaling under a binary32 scale (ss_mode 1, 3 or 4): (E4M3 bytes
    uint8 [rows, cols], scales float32 [rows // brows, cols // bcols], global_amax);
    element = decode(code) / scale."""
    x = np.ascontiguousarray(x)
    is_f32 = _check_in(x)
    rows, cols = x.shape
    payload = np.zeros((rows, cols), np.uint8)
    scales = np.zeros((rows // brows, cols // bcols), np.float32)
    ext = None if global_amax is None else np.array([global_amax], np.float32)
    gamax = np.zeros(1, np.float32)
    _rc(lib().mor_o_quantize_scaled(_p(x), is_f32, _p(payload), _p(scales), rows, cols, brows, bcols, ss, _p(ext),
                                    _p(gamax)), "quantize_scaled")
    return payload, scales, gamax[0]


def dequantize_scaled(payload, scales, brows, bcols, float32=False):
    """decode(code) / scale as bf16 bits (uint16) or float32, rounded as the fake-quantize operators round"""
    payload = np.ascontiguousarray(payload, dtype=np.uint8)
    scales = np.ascontiguousarray(scales, dtype=np.float32)
    rows, cols = payload.shape
    out = np.zeros((rows, cols), np.float32 if float32 else np.uint16)
    _rc(lib().mor_o_dequantize_scaled(_p(payload), _p(scales), _p(out), int(float32), rows, cols, brows, bcols),
        "dequantize_scaled")
    return out


def amax_nnz(x):
    x = np.ascontiguousarray(x)
    is_f32 = _check_in(x)
    a = np.zeros(1, np.float32)
    n = np.zeros(1, np.int64)
    lib().mor_o_amax_nnz(_p(x), is_f32, x.size, _p(a), _p(n))
    return a[0], int(n[0])


def finalize(block_err, stride, nnz, thr):
    """Ordered tensor-level error sum over gathered per-CTA errors: (meta, global_error)."""
    be = np.ascontiguousarray(block_err, dtype=np.float32)
    meta = np.zeros(1, np.int32)
    total = lib().mor_o_finalize(_p(be), be.size, int(stride), int(nnz), float(thr), _p(meta))
    return int(meta[0]), np.float32(total)


# ----------------------------------------------------------------- torch helpers
def bf16_bits(t):
    """torch bf16 CPU tensor -> uint16 numpy view of its bits."""
    import torch

    assert t.dtype == torch.bfloat16 and t.device.type == "cpu"
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def bits_to_bf16(a):
    """uint16 numpy array -> torch bf16 tensor."""
    import torch

    return torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).view(torch.bfloat16)
