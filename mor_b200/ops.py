"""Python operator surface, call-compatible with ``mor/ops.py`` of boryiings/mor.

Every function forwards to ``torch.ops.mor.<name>`` (registered by ``mor_b200._C``
for CUDA tensors) with the reference's positional arguments: ``dim_x`` = rows,
``dim_y`` = columns, ``block_x`` = block rows, ``block_y`` = block columns.  All
operators are fake-quantizers, so the backward is the straight-through estimator:
the incoming gradient is passed to the tensor argument unchanged and every other
argument gets ``None`` (mor/ops.py:15-21 and the registrations that follow it).
"""
from __future__ import annotations

from typing import List

import torch
from torch import Tensor

_ops = torch.ops.mor

__all__ = [
    "fake_quantize", "fake_quantize_no_alloc",
    "fake_quantize_block_scaling", "fake_quantize_block_scaling_inplace",
    "fake_quantize_channel_scaling", "fake_quantize_channel_scaling_inplace",
    "fake_quantize_e8mx", "fake_quantize_e8mx_inplace",
    "quant_dequant_e4m3", "quant_dequant_e5m2", "quant_dequant_e2m3", "quant_dequant_e3m2",
    "e4m3_with_e8_scale_rne", "e4m3_with_e8_scale_rz",
    "fake_quantize_mx",
    "quantize_mx",
    "quantize_mx_fp6",
    "quantize_scaled",
    "fake_quantize_block_scaling_delayed",
    "fake_quantize_block_scaling_delayed_t",
]


# --------------------------------------------------------------------------- MoR / per-block
def fake_quantize(a: Tensor, dim_x: int, dim_y: int, block_x: int, block_y: int, clamp_threshold: float,
                  mode: int, sf_type: int) -> List[Tensor]:
    """Per-block fake-quantize; returns ``[out, meta]``.

    ``mode % 10``: 1 MoR (per-block choice of E2M3 / E4M3 / E5M2 / BF16), 2 E4M3 blocks,
    3 E5M2 blocks, 4 / 5 one given scale (``clamp_threshold``) with E4M3 / E5M2, other
    values copy the tensor.  ``mode >= 100`` makes MoR decide by dynamic range alone.
    ``sf_type``: 1 float scale, 2 power-of-two scale.  ``meta[i, j]`` is the choice for
    block (i, j): 1 E4M3, 2 E5M2, 3 BF16, 4 E2M3, 11 / 12 the "small amax" variants.
    """
    return _ops.fake_quantize.default(a, dim_x, dim_y, block_x, block_y, clamp_threshold, mode, sf_type)


def fake_quantize_no_alloc(a: Tensor, dim_x: int, dim_y: int, block_x: int, block_y: int, clamp_threshold: float,
                           mode: int, sf_type: int, output: Tensor) -> Tensor:
    """``fake_quantize`` into a caller-owned ``output`` (which may be ``a`` itself); returns ``meta``."""
    return _ops.fake_quantize_no_alloc.default(a, dim_x, dim_y, block_x, block_y, clamp_threshold, mode, sf_type,
                                               output)


# --------------------------------------------------------------------------- tensor-scaled E4M3
def fake_quantize_block_scaling(a: Tensor, dim_x: int, dim_y: int, block_x: int, block_y: int,
                                e4m3_threshold: float, ss_mode: int) -> List[Tensor]:
    """E4M3 with a scale per block derived from the block and tensor amax; the whole tensor
    falls back to BF16 when the mean relative error exceeds ``e4m3_threshold``.
    Returns ``[out, meta, global_amax, global_non_zero, global_error]``."""
    return _ops.fake_quantize_block_scaling.default(a, dim_x, dim_y, block_x, block_y, e4m3_threshold, ss_mode)


def fake_quantize_block_scaling_inplace(a: Tensor, dim_x: int, dim_y: int, block_x: int, block_y: int,
                                        e4m3_threshold: float, ss_mode: int) -> List[Tensor]:
    """As above, overwriting ``a``; returns ``[meta, global_amax, global_non_zero, global_error]``."""
    return _ops.fake_quantize_block_scaling_inplace.default(a, dim_x, dim_y, block_x, block_y, e4m3_threshold,
                                                            ss_mode)


def fake_quantize_channel_scaling(a: Tensor, dim_x: int, dim_y: int, block_x: int, block_y: int,
                                  e4m3_threshold: float, ss_mode: int) -> List[Tensor]:
    """Block scaling with 1 x k (``block_x == 1``) or k x 1 (``block_y == 1``) blocks."""
    return _ops.fake_quantize_channel_scaling.default(a, dim_x, dim_y, block_x, block_y, e4m3_threshold, ss_mode)


def fake_quantize_channel_scaling_inplace(a: Tensor, dim_x: int, dim_y: int, block_x: int, block_y: int,
                                          e4m3_threshold: float, ss_mode: int) -> List[Tensor]:
    """In-place form of ``fake_quantize_channel_scaling``."""
    return _ops.fake_quantize_channel_scaling_inplace.default(a, dim_x, dim_y, block_x, block_y, e4m3_threshold,
                                                              ss_mode)


# --------------------------------------------------------------------------- E8Mx
def fake_quantize_e8mx(a: Tensor, dim_x: int, dim_y: int, block_x: int, block_y: int, quantize_type: int,
                       scaling_strategy: int) -> Tensor:
    """Keep the 8-bit exponent, round the mantissa to ``quantize_type`` (1..3) bits;
    ``scaling_strategy == 1`` first scales by the tensor amax."""
    return _ops.fake_quantize_e8mx.default(a, dim_x, dim_y, block_x, block_y, quantize_type, scaling_strategy)


def fake_quantize_e8mx_inplace(a: Tensor, dim_x: int, dim_y: int, block_x: int, block_y: int, quantize_type: int,
                               scaling_strategy: int, output: Tensor) -> None:
    """``fake_quantize_e8mx`` into a caller-owned ``output``.  No autograd registration,
    as in the reference (mor/ops.py:104-106)."""
    return _ops.fake_quantize_e8mx_inplace.default(a, dim_x, dim_y, block_x, block_y, quantize_type,
                                                   scaling_strategy, output)


# --------------------------------------------------------------------------- test operators (float32)
def quant_dequant_e4m3(a: Tensor, dim_x: int, dim_y: int, block_x: int, block_y: int) -> Tensor:
    """float32 -> E4M3 -> float32, unscaled; overflow gives NaN."""
    return _ops.quant_dequant_e4m3.default(a, dim_x, dim_y, block_x, block_y)


def quant_dequant_e5m2(a: Tensor, dim_x: int, dim_y: int, block_x: int, block_y: int) -> Tensor:
    """float32 -> E5M2 -> float32, unscaled; overflow gives NaN."""
    return _ops.quant_dequant_e5m2.default(a, dim_x, dim_y, block_x, block_y)


def quant_dequant_e2m3(a: Tensor, dim_x: int, dim_y: int, block_x: int, block_y: int) -> Tensor:
    """float32 -> E2M3 -> float32, unscaled; overflow clamps to 7.5."""
    return _ops.quant_dequant_e2m3.default(a, dim_x, dim_y, block_x, block_y)


def quant_dequant_e3m2(a: Tensor, dim_x: int, dim_y: int, block_x: int, block_y: int) -> Tensor:
    """float32 -> E3M2 -> float32, unscaled; overflow clamps to 28."""
    return _ops.quant_dequant_e3m2.default(a, dim_x, dim_y, block_x, block_y)


def e4m3_with_e8_scale_rne(a: Tensor, dim_x: int, dim_y: int, block_x: int, block_y: int) -> Tensor:
    """E4M3 with a per-element power-of-two scale, scale exponent rounded to nearest."""
    return _ops.e4m3_with_e8_scale_rne.default(a, dim_x, dim_y, block_x, block_y)


def e4m3_with_e8_scale_rz(a: Tensor, dim_x: int, dim_y: int, block_x: int, block_y: int) -> Tensor:
    """E4M3 with a per-element power-of-two scale, scale exponent truncated."""
    return _ops.e4m3_with_e8_scale_rz.default(a, dim_x, dim_y, block_x, block_y)


# --------------------------------------------------------------------------- addition
def fake_quantize_mx(a: Tensor, dim_x: int, dim_y: int, block_y: int, elem_format: int, sf_type: int) -> List[Tensor]:
    """Single-pass fake-quantize with one scale per 1 x ``block_y`` group (MX: ``block_y = 32``,
    ``sf_type = 2``).  ``elem_format``: 0 E4M3, 1 E5M2, 3 E2M3.  Returns ``[out, scales]``."""
    return _ops.fake_quantize_mx.default(a, dim_x, dim_y, block_y, elem_format, sf_type)


def fake_quantize_block_scaling_delayed(a: Tensor, dim_x: int, dim_y: int, block_x: int, block_y: int,
                                        e4m3_threshold: float, ss_mode: int, amax_in: Tensor) -> List[Tensor]:
    """Block scaling in one pass over the tensor: the scales are built from ``amax_in`` (float32[1] on the
    device, typically the amax that this call returned for the previous step's tensor), each 128 x 128
    block's own amax is taken on chip.  Returns ``[out, meta, amax, non_zero, error]`` of THIS tensor."""
    return _ops.fake_quantize_block_scaling_delayed.default(a, dim_x, dim_y, block_x, block_y, e4m3_threshold, ss_mode, amax_in)


def fake_quantize_block_scaling_delayed_t(a: Tensor, dim_x: int, dim_y: int, block_x: int, block_y: int,
                                          e4m3_threshold: float, ss_mode: int, amax_in: Tensor) -> List[Tensor]:
    """:func:`fake_quantize_block_scaling_delayed` that also returns the result transposed (``[dim_y, dim_x]``, the
    layout a weight-gradient GEMM reads), written from the tile while it is on chip: returns
    ``[out, out_t, meta, amax, non_zero, error]``."""
    return _ops.fake_quantize_block_scaling_delayed_t.default(a, dim_x, dim_y, block_x, block_y, e4m3_threshold, ss_mode, amax_in)


def quantize_mx(a: Tensor, dim_x: int, dim_y: int, block_y: int, elem_format: int) -> List[Tensor]:
    """The real quantized form of :func:`fake_quantize_mx` with a power-of-two scale: returns
    ``[payload, scales]``, both ``uint8``: one narrow-float code per element (fp8 byte for E4M3 / E5M2, the
    6-bit code in a byte for E2M3) and one E8M0 byte per 1 x ``block_y`` group;
    ``element = decode(code) * 2 ** (scale - 127)``.  No gradient."""
    return _ops.quantize_mx.default(a, dim_x, dim_y, block_y, elem_format)


def quantize_mx_fp6(a: Tensor, dim_x: int, dim_y: int, block_y: int) -> List[Tensor]:
    """:func:`quantize_mx` for E2M3 with the codes packed six bits each: ``payload`` is ``uint8 [dim_x, dim_y * 3 / 4]``,
    every run of eight elements a little-endian 48-bit group with code i in bits [6 i, 6 i + 6)."""
    return _ops.quantize_mx_fp6.default(a, dim_x, dim_y, block_y)


def quantize_scaled(a: Tensor, dim_x: int, dim_y: int, block_x: int, block_y: int, ss_mode: int) -> List[Tensor]:
    """The real quantized form of :func:`fake_quantize_block_scaling` / :func:`fake_quantize_channel_scaling` under a
    float scale (``ss_mode`` 1, 3 or 4): returns ``[payload, scales, global_amax]`` -- one E4M3 byte per element
    (``uint8 [dim_x, dim_y]``, viewable as ``torch.float8_e4m3fn``), one ``float32`` scale per block
    (``[dim_x // block_x, dim_y // block_y]``) and the tensor's amax; ``element = decode(code) / scale``.  No gradient."""
    return _ops.quantize_scaled.default(a, dim_x, dim_y, block_x, block_y, ss_mode)


# --------------------------------------------------------------------------- straight-through backward
def _straight_through(n_args: int):
    def backward(ctx, grad, *unused):
        # operators that return a list hand the gradients over as a list: the first
        # entry belongs to the fake-quantized tensor, the rest to integer/scalar outputs
        if isinstance(grad, (list, tuple)):
            grad = grad[0]
        return (grad,) + (None,) * (n_args - 1)
    return backward


def _no_context(ctx, inputs, output):
    return None


for _name, _n in {
    "fake_quantize": 8, "fake_quantize_no_alloc": 9,
    "fake_quantize_block_scaling": 7, "fake_quantize_block_scaling_inplace": 7,
    "fake_quantize_channel_scaling": 7, "fake_quantize_channel_scaling_inplace": 7,
    "fake_quantize_e8mx": 7,
    "quant_dequant_e4m3": 5, "quant_dequant_e5m2": 5, "quant_dequant_e2m3": 5, "quant_dequant_e3m2": 5,
    "e4m3_with_e8_scale_rne": 5, "e4m3_with_e8_scale_rz": 5,
    "fake_quantize_mx": 6,
    "fake_quantize_block_scaling_delayed": 8,
    "fake_quantize_block_scaling_delayed_t": 8,
}.items():
    torch.library.register_autograd(f"mor::{_name}", _straight_through(_n), setup_context=_no_context)
del _name, _n
