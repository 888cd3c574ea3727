"""Fixtures and the torch-CPU computation that the reference's own tests check against.

The reference (boryiings/mor) tests its CUDA operators against a PyTorch CPU
re-computation and a hand-built known-answer matrix; those are restated here so
that the CPU oracle of this repository (and through it the CUDA kernels) is pinned
to the same answers.  Citations are to files of the reference.
"""
from __future__ import annotations

import math
import struct

import numpy as np
import torch


def kat_matrix_bits(rows: int, cols: int, forced=()) -> np.ndarray:
    """Known-answer matrix of test/test_fake_quantize.py:16-24 as bf16 bit patterns.

    Packed word (i, j) is (16256 << 16 | 49024) + i * 65536 + j: element 2j of row i
    has bits 0xBF80 + j (-1.0 and slightly below), element 2j+1 has bits 0x3F80 + i.
    ``forced`` is a list of (row, word, high_bits, low_bits) overrides, the way the
    reference tests plant one outlier word per block.
    """
    w = cols // 2
    i = np.arange(rows, dtype=np.uint32)[:, None]
    j = np.arange(w, dtype=np.uint32)[None, :]
    words = (np.uint32(16256 * 65536 + 49024) + i * np.uint32(65536) + j).astype(np.uint32)
    for (r, c, hi, lo) in forced:
        words[r, c] = np.uint32(hi * 65536 + lo)
    return np.ascontiguousarray(words).view(np.uint16).reshape(rows, cols)


# outlier words used by the reference tests (test_fake_quantize.py:233-239, 323-329)
FORCE_E5M2_DYN = (128, 1, 18200, 50968)    # (38912, -38912): range > 28672
FORCE_E5M2_ERR = (128, 1, 18403, 51171)    # (116224, -116224): range > 114688
FORCE_BF16 = (0, 70, 21000, 53768)         # (1.46e11, -1.46e11): range > 939524096
FORCE_E4M3_DYN = (1, 1, 17262, 50030)      # (238, -238)
FORCE_E4M3_ERR = (1, 1, 17264, 50032)


def bits_to_bf16(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).view(torch.bfloat16)


def bf16_bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def f32(x: float) -> float:
    return struct.unpack("<f", struct.pack("<f", x))[0]


def torch_fake_quantize_to_fp32(block_f32: torch.Tensor, kind: str, amax: float, e8: bool = False) -> torch.Tensor:
    """test/test_fake_quantize.py:33-47.  amax must be a Python scalar so that the
    scale is a true division (the comment at :96-104 of that file explains why)."""
    if kind == "e4m3":
        scale, dt = 448.0 / amax, torch.float8_e4m3fn
    elif kind == "e5m2":
        scale, dt = 57344.0 / amax, torch.float8_e5m2
    elif kind == "e2m3":  # emulated through e4m3, exact while |x * scale| <= 7.5 stays on the e2m3 grid
        scale, dt = 7.5 / amax, torch.float8_e4m3fn
    else:
        raise ValueError(kind)
    scale = f32(scale)
    if e8:
        scale = 2.0 ** math.floor(math.log2(scale))
    return (block_f32 * scale).type(dt).float() / scale


def torch_rel_error(orig: torch.Tensor, q: torch.Tensor) -> torch.Tensor:
    return torch.sum(torch.abs((q - orig) / orig))


def torch_cpu_mor(block: torch.Tensor, dynamic_range: bool, e8: bool = False):
    """test/test_fake_quantize.py:56-143 (cpu_mor_dynamic_range / cpu_mor), with the
    kernel's 28672 in place of that file's 28762 typo.  Returns (bf16 block, code)."""
    bf = block.float()
    ab = bf.abs()
    amax = ab.max().item()
    nz = ab[ab > 0]
    if nz.numel() == 0:
        return block, 4
    rng = f32(amax / nz.min().item())
    e4_range = 28672 if dynamic_range else 28672 * 4
    if rng <= 7.5:
        return torch_fake_quantize_to_fp32(bf, "e2m3", amax, e8).type(torch.bfloat16), 4
    if rng <= e4_range:
        return torch_fake_quantize_to_fp32(bf, "e4m3", amax, e8).type(torch.bfloat16), 1
    if rng <= 939524096:
        if dynamic_range:
            return torch_fake_quantize_to_fp32(bf, "e5m2", amax, e8).type(torch.bfloat16), 2
        q4 = torch_fake_quantize_to_fp32(bf, "e4m3", amax)
        q5 = torch_fake_quantize_to_fp32(bf, "e5m2", amax)
        if torch_rel_error(bf, q4) <= torch_rel_error(bf, q5):
            return q4.type(torch.bfloat16), 1
        return block, 3
    return block, 3


def decompose(v: float):
    b = struct.unpack("<I", struct.pack("<f", v))[0]
    return b >> 31, (b >> 23) & 0xFF, b & 0x7FFFFF


def torch_block_scaling_e4m3(t: torch.Tensor, brows: int, bcols: int, global_mantissa: int):
    """test/test_fake_quantize_block_scaling.py:51-98: per-block scale = block scale with
    the tensor scale's mantissa, halved when that made it larger.  Returns (bf16
    tensor, total relative error as a python float)."""
    out = t.clone()
    total = 0.0
    rows, cols = t.shape
    for x in range(0, rows, brows):
        for y in range(0, cols, bcols):
            blk = t[x:x + brows, y:y + bcols].float()
            bsf = f32(448.0 / blk.abs().max().item())
            s, e, m = decompose(bsf)
            nsf = struct.unpack("<f", struct.pack("<I", s << 31 | e << 23 | global_mantissa))[0]
            sf = nsf if global_mantissa <= m else nsf / 2.0
            deq = (blk * sf).type(torch.float8_e4m3fn).float() / sf
            total += torch.sum(torch.abs((deq - blk) / blk)).item()
            out[x:x + brows, y:y + bcols] = deq.type(torch.bfloat16)
    return out, total


def random_bf16(rows, cols, lo, hi, seed):
    g = torch.Generator().manual_seed(seed)
    return (torch.rand(rows, cols, generator=g) * (hi - lo) + lo).type(torch.bfloat16)
