"""Seeded inputs and operator invocations shared by the golden-vector generator
(``make_gpu_golden.py``, which runs the UNMODIFIED reference extension on a GPU) and by
the tests that replay the same cases through the CPU oracle and the CUDA kernels.

A case is ``(name, op, input_fn, kwargs)``; ``input_fn()`` returns a numpy array, uint16
bf16 bit patterns or float32.  Everything is generated on the CPU from fixed seeds so
that every machine sees identical bits.
"""
from __future__ import annotations

import hashlib
import os
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from ref_fixtures import (FORCE_BF16, FORCE_E4M3_DYN, FORCE_E4M3_ERR, FORCE_E5M2_DYN,  # noqa: E402
                          FORCE_E5M2_ERR, bf16_bits, kat_matrix_bits)


def digest(a: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def _gen(seed):
    return torch.Generator().manual_seed(seed)


def uniform_bf16(seed, lo, hi, rows=256, cols=256):
    t = torch.rand(rows, cols, generator=_gen(seed)) * (hi - lo) + lo
    return bf16_bits(t.to(torch.bfloat16))


def normal_bf16(seed, std=1.0, rows=256, cols=256):
    return bf16_bits((torch.randn(rows, cols, generator=_gen(seed)) * std).to(torch.bfloat16))


def uniform_f32(seed, lo, hi, rows=256, cols=256):
    return (torch.rand(rows, cols, generator=_gen(seed)) * (hi - lo) + lo).numpy().astype(np.float32)


def logspread_bf16(seed, lo_exp, hi_exp, rows=256, cols=256):
    """sign * 10**U(lo_exp, hi_exp): wide dynamic range, no zeros."""
    g = _gen(seed)
    mag = 10.0 ** (torch.rand(rows, cols, generator=g) * (hi_exp - lo_exp) + lo_exp)
    sign = torch.where(torch.rand(rows, cols, generator=g) < 0.5, -1.0, 1.0)
    return bf16_bits((mag * sign).to(torch.bfloat16))


def mixed_blocks_bf16(seed, rows=512, cols=512, block=128, kinds=4):
    """Blocks cycle through N(0,1), Laplace(0,1e-3), log-uniform 1e-6..1e4 and
    log-uniform 1e-3..1e4 (the last one loses the E4M3-vs-E5M2 error comparison)."""
    g = _gen(seed)
    out = torch.empty(rows, cols)
    nbx = cols // block
    for bi in range(rows // block):
        for bj in range(nbx):
            kind = (bi * nbx + bj) % kinds
            if kind == 0:
                blk = torch.randn(block, block, generator=g)
            elif kind == 1:
                u = torch.rand(block, block, generator=g) - 0.5
                blk = -1e-3 * torch.sign(u) * torch.log1p(-2 * u.abs().clamp(max=0.49999997))
            else:
                lo = -6.0 if kind == 2 else -3.0
                mag = 10.0 ** (torch.rand(block, block, generator=g) * (4.0 - lo) + lo)
                blk = mag * torch.where(torch.rand(block, block, generator=g) < 0.5, -1.0, 1.0)
            out[bi * block:(bi + 1) * block, bj * block:(bj + 1) * block] = blk
    return bf16_bits(out.to(torch.bfloat16))


def with_zeros(bits, seed, frac=0.1):
    g = _gen(seed)
    m = torch.rand(*bits.shape, generator=g) < frac
    b = bits.copy()
    b[m.numpy()] = 0
    return b


def scale_for(bits, fmax):
    amax = np.abs((bits.astype(np.uint32) << 16).view(np.float32)).max()
    return float(np.float32(fmax) / np.float32(amax))


KAT_DYN = lambda: kat_matrix_bits(256, 256, [FORCE_E5M2_DYN, FORCE_BF16, FORCE_E4M3_DYN])  # noqa: E731
KAT_ERR = lambda: kat_matrix_bits(256, 256, [FORCE_E5M2_ERR, FORCE_BF16, FORCE_E4M3_ERR])  # noqa: E731
KAT_PLAIN = lambda: kat_matrix_bits(256, 256)  # noqa: E731


def cases():
    """Every golden case.  Ops and keyword names follow mor/ops.py of the reference."""
    c = []

    def fq(name, fn, mode, sf, clamp=1e-15, bx=128, by=128):
        c.append((name, "fake_quantize", fn, dict(block_x=bx, block_y=by, clamp_threshold=clamp, mode=mode, sf_type=sf)))

    # known-answer matrices of test/test_fake_quantize.py
    fq("fq_kat_dyn_fp32", KAT_DYN, 101, 1)
    fq("fq_kat_err_fp32", KAT_ERR, 1, 1)
    fq("fq_kat_dyn_e8", KAT_DYN, 101, 2, clamp=1e-25)
    fq("fq_kat_err_e8", KAT_ERR, 1, 2, clamp=1e-25)
    fq("fq_zero_dyn_e8", lambda: np.zeros((256, 256), np.uint16), 101, 2, clamp=1e-25)
    fq("fq_tiny_dyn_e8", lambda: bf16_bits(torch.ones(256, 256, dtype=torch.bfloat16) * 1e-27), 101, 2, clamp=1e-25)
    for seed in (0, 1):
        u = (lambda s: (lambda: uniform_bf16(s, -53768.0, 53768.0)))(seed)
        for mode, sf in ((1, 1), (101, 1), (1, 2), (101, 2), (2, 1), (2, 2), (3, 1), (3, 2), (7, 1)):
            fq(f"fq_uniform{seed}_m{mode}_sf{sf}", u, mode, sf, clamp=1e-15 if sf == 1 else 1e-25)
    for sf in (1, 2):
        fq(f"fq_mixed_m1_sf{sf}", lambda: mixed_blocks_bf16(7), 1, sf)
        fq(f"fq_mixed_m101_sf{sf}", lambda: mixed_blocks_bf16(7), 101, sf)
    fq("fq_mixed_zeros_m1", lambda: with_zeros(mixed_blocks_bf16(8), 9), 1, 1)
    fq("fq_normal_m1_64x64", lambda: normal_bf16(3), 1, 1, bx=64, by=64)
    fq("fq_logspread_m1_32x64", lambda: logspread_bf16(4, -3, 4), 1, 1, bx=32, by=64)
    fq("fq_logspread_m1_32x32", lambda: logspread_bf16(5, -3, 4), 1, 1, bx=32, by=32)
    fq("fq_small_clamp", lambda: normal_bf16(6, std=1e-3), 1, 1, clamp=1.0)  # *_SMALL codes 11
    fq("fq_small_clamp_dyn", lambda: logspread_bf16(10, -2, 4), 101, 1, clamp=1e6)  # code 12
    # current scaling: the scale travels in clamp_threshold
    for seed in (0, 1):
        bits = (lambda s: (lambda: uniform_bf16(s, -53768.0, 53768.0)))(seed)
        fq(f"fq_current_e4m3_{seed}", bits, 4, 1, clamp=scale_for(bits(), 448.0))
        fq(f"fq_current_e5m2_{seed}", bits, 5, 1, clamp=scale_for(bits(), 57344.0))
        fq(f"fq_current_e4m3_e8_{seed}", bits, 4, 2, clamp=scale_for(bits(), 448.0))
    fq("fq_current_e4m3_normal", lambda: normal_bf16(11), 4, 1, clamp=scale_for(normal_bf16(11), 448.0))

    def scal(op, name, fn, bx, by, thr, ss):
        c.append((name, op, fn, dict(block_x=bx, block_y=by, e4m3_threshold=thr, ss_mode=ss)))

    for ss in (1, 2, 3, 4):
        scal("fake_quantize_block_scaling", f"bs_kat_ss{ss}", KAT_PLAIN, 128, 128, 0.045, ss)
        scal("fake_quantize_block_scaling", f"bs_normal_ss{ss}", lambda: normal_bf16(20), 128, 128, 0.045, ss)
        scal("fake_quantize_block_scaling", f"bs_wide_ss{ss}", lambda: uniform_bf16(21, -53768.0, 53768.0), 128, 128, 0.045, ss)
        scal("fake_quantize_block_scaling", f"bs_zeros_ss{ss}", lambda: with_zeros(normal_bf16(22), 23), 64, 128, 0.045, ss)
        scal("fake_quantize_block_scaling", f"bs_logspread_ss{ss}", lambda: logspread_bf16(24, -4, 4), 128, 128, 0.045, ss)
        scal("fake_quantize_block_scaling", f"bs_logspread_keep_ss{ss}", lambda: logspread_bf16(24, -4, 4), 128, 128, 3e38, ss)
        # full-column groups: the only channel geometry of the shipped reference that is
        # free of out-of-bounds shared-memory accesses (its row-group launches are not)
        scal("fake_quantize_channel_scaling", f"cs_col_kat_ss{ss}", KAT_PLAIN, 256, 1, 0.045, ss)
        scal("fake_quantize_channel_scaling", f"cs_col_normal_ss{ss}", lambda: normal_bf16(25), 256, 1, 0.045, ss)
        scal("fake_quantize_channel_scaling", f"cs_col_wide_ss{ss}", lambda: with_zeros(logspread_bf16(26, -4, 4), 27), 256, 1, 3e38, ss)

    for qt in (1, 2, 3):
        for strat in (1, 3):
            c.append((f"e8m{qt}_s{strat}", "fake_quantize_e8mx", lambda: uniform_bf16(30, -53768.0, 53768.0),
                      dict(block_x=128, block_y=128, quantize_type=qt, scaling_strategy=strat)))
            c.append((f"e8m{qt}_s{strat}_small", "fake_quantize_e8mx", lambda: with_zeros(normal_bf16(31, std=1e-4), 32),
                      dict(block_x=128, block_y=128, quantize_type=qt, scaling_strategy=strat)))

    def unary(op, name, fn):
        c.append((name, op, fn, dict(block_x=128, block_y=128)))

    def nan_probe():
        x = uniform_f32(40, -1000.0, 1000.0)
        x[0, :6] = [463.0, 464.0, 465.0, -464.0, -464.5, 448.0]
        return x

    unary("quant_dequant_e4m3", "qd_e4m3_mid", lambda: uniform_f32(41, -400.0, 400.0))
    unary("quant_dequant_e4m3", "qd_e4m3_sub", lambda: uniform_f32(42, -1.0, 1.0))
    unary("quant_dequant_e4m3", "qd_e4m3_tiny", lambda: uniform_f32(43, -0.02, 0.02))
    unary("quant_dequant_e4m3", "qd_e4m3_nan", nan_probe)
    unary("quant_dequant_e5m2", "qd_e5m2", lambda: uniform_f32(44, -53768.0, 53768.0))
    unary("quant_dequant_e5m2", "qd_e5m2_over", lambda: uniform_f32(45, -70000.0, 70000.0))
    unary("quant_dequant_e5m2", "qd_e5m2_tiny", lambda: uniform_f32(46, -1e-4, 1e-4))
    unary("quant_dequant_e3m2", "qd_e3m2", lambda: uniform_f32(47, -40.0, 100.0))
    unary("quant_dequant_e3m2", "qd_e3m2_sub", lambda: uniform_f32(48, -0.5, 0.5))
    unary("quant_dequant_e2m3", "qd_e2m3", lambda: uniform_f32(49, -10.0, 20.0))
    unary("quant_dequant_e2m3", "qd_e2m3_sub", lambda: uniform_f32(50, -1.0, 1.0))
    unary("e4m3_with_e8_scale_rne", "e8rne", lambda: uniform_f32(51, -1000.0, 1000.0))
    unary("e4m3_with_e8_scale_rz", "e8rz", lambda: uniform_f32(51, -1000.0, 1000.0))
    unary("e4m3_with_e8_scale_rne", "e8rne_small", lambda: uniform_f32(52, -1e-3, 1e-3))
    unary("e4m3_with_e8_scale_rz", "e8rz_small", lambda: uniform_f32(52, -1e-3, 1e-3))
    return c
