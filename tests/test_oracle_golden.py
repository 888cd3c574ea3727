"""Pins the CPU oracle: known-answer matrices and the torch-CPU computation of the
reference's own tests, NVIDIA's conversion headers' semantics via torch's float8 casts,
and outputs recorded from the unmodified reference extension on a B200
(tests/golden/reference_b200.json, written by tests/golden/make_gpu_golden.py)."""
import json
import os

import numpy as np
import pytest
import torch

import oracle
from cases import cases, digest
from ref_fixtures import (FORCE_BF16, FORCE_E4M3_DYN, FORCE_E4M3_ERR, FORCE_E5M2_DYN, FORCE_E5M2_ERR, bf16_bits,
                          bits_to_bf16, decompose, f32, kat_matrix_bits, random_bf16, torch_block_scaling_e4m3,
                          torch_cpu_mor, torch_fake_quantize_to_fp32)
from replay import run_oracle

HERE = os.path.dirname(os.path.abspath(__file__))
GOLDEN = os.path.join(HERE, "golden", "reference_b200.json")


def blocks(t, b=128):
    for i in range(0, t.shape[0], b):
        for j in range(0, t.shape[1], b):
            yield i // b, j // b, t[i:i + b, j:j + b]


# expected meta matrices asserted by test/test_fake_quantize.py:256-269, 346-359, 818-831
@pytest.mark.parametrize("mode,sf,forced,dyn,e8,clamp,expected", [
    (101, 1, [FORCE_E5M2_DYN, FORCE_BF16, FORCE_E4M3_DYN], True, False, 1e-15, [[1, 3], [2, 4]]),
    (1, 1, [FORCE_E5M2_ERR, FORCE_BF16, FORCE_E4M3_ERR], False, False, 1e-15, [[1, 3], [3, 4]]),
    (101, 2, [FORCE_E5M2_DYN, FORCE_BF16, FORCE_E4M3_DYN], True, True, 1e-25, [[1, 3], [2, 4]]),
])
def test_known_answer_matrix(mode, sf, forced, dyn, e8, clamp, expected):
    bits = kat_matrix_bits(256, 256, forced)
    out, meta = oracle.fake_quantize(bits, 128, 128, clamp, mode, sf)
    assert meta.tolist() == expected
    t, o = bits_to_bf16(bits), bits_to_bf16(out)
    for bi, bj, blk in blocks(t):
        exp, code = torch_cpu_mor(blk, dyn, e8)
        assert code == expected[bi][bj]
        assert o[bi * 128:(bi + 1) * 128, bj * 128:(bj + 1) * 128].equal(exp)


def test_zero_and_tiny_blocks():
    # test/test_fake_quantize.py:874-948: all-zero and 1e-27 tensors choose E2M3 (4), output unchanged / exact
    z = np.zeros((256, 256), np.uint16)
    out, meta = oracle.fake_quantize(z, 128, 128, 1e-25, 101, 2)
    assert (meta == 4).all() and (out == 0).all()
    t = torch.ones(256, 256, dtype=torch.bfloat16) * 1e-27
    out, meta = oracle.fake_quantize(bf16_bits(t), 128, 128, 1e-25, 101, 2)
    exp, code = torch_cpu_mor(t[:128, :128], True, True)
    assert (meta == 4).all() and code == 4
    assert bits_to_bf16(out)[:128, :128].equal(exp) and bits_to_bf16(out)[128:, 128:].equal(exp)
    assert oracle.assert_flags() == 0


@pytest.mark.parametrize("seed", range(4))
@pytest.mark.parametrize("mode,sf,dyn,e8,clamp", [(1, 1, False, False, 1e-15), (101, 1, True, False, 1e-15),
                                                  (101, 2, True, True, 1e-25)])
def test_random_matrix_vs_torch_cpu_path(seed, mode, sf, dyn, e8, clamp):
    t = random_bf16(256, 256, -53768.0, 53768.0, seed)
    out, meta = oracle.fake_quantize(bf16_bits(t), 128, 128, clamp, mode, sf)
    o = bits_to_bf16(out)
    for bi, bj, blk in blocks(t):
        exp, code = torch_cpu_mor(blk, dyn, e8)
        assert code == meta[bi, bj]
        assert o[bi * 128:(bi + 1) * 128, bj * 128:(bj + 1) * 128].equal(exp)


@pytest.mark.parametrize("seed", range(3))
def test_current_scaling_vs_torch(seed):
    # test/test_fake_quantize.py:413-461
    t = random_bf16(256, 256, -53768.0, 53768.0, seed)
    amax = t.float().abs().max().item()
    for mode, kind, mx in ((4, "e4m3", 448.0), (5, "e5m2", 57344.0)):
        out, meta = oracle.fake_quantize(bf16_bits(t), 128, 128, f32(mx / amax), mode, 1)
        exp = torch_fake_quantize_to_fp32(t.float(), kind, amax).type(torch.bfloat16)
        assert bits_to_bf16(out).equal(exp)
        assert (meta == (1 if mode == 4 else 2)).all()
    out, meta = oracle.fake_quantize(bf16_bits(t), 128, 128, 1e-15, 7, 1)
    assert (meta == 3).all() and np.array_equal(out, bf16_bits(t))


def test_block_scaling_vs_torch():
    # test/test_fake_quantize_block_scaling.py:100-136: ss_mode 1, bit-equal output, error within rtol 1e-3
    for bits in (kat_matrix_bits(256, 256), bf16_bits(random_bf16(256, 256, 1.0, 3.0, 5))):
        t = bits_to_bf16(bits)
        out, meta, gamax, gnnz, gerr = oracle.block_scaling(bits, 128, 128, 0.045, 1)
        assert meta == 1 and gamax == t.float().abs().max().item() and gnnz == int(torch.count_nonzero(t))
        _, _, gman = decompose(f32(448.0 / float(gamax)))
        exp, total = torch_block_scaling_e4m3(t, 128, 128, gman)
        assert bits_to_bf16(out).equal(exp)
        assert abs(total - gerr) <= 1e-3 * total


def test_block_scaling_bf16_fallback():
    # test_fake_quantize_block_scaling.py:138-175: a wide-range tensor stays BF16 (meta 3, output == input)
    g = torch.Generator().manual_seed(3)
    t = (10.0 ** (torch.rand(256, 256, generator=g) * 8 - 4)).to(torch.bfloat16)
    out, meta, *_ = oracle.block_scaling(bf16_bits(t), 128, 128, 0.045, 1)
    assert meta == 3 and np.array_equal(out, bf16_bits(t))


@pytest.mark.parametrize("bx,by", [(1, 256), (256, 1)])
def test_channel_scaling_vs_torch(bx, by):
    # test_fake_quantize_channel_scaling.py:100-172: full rows / full columns, ss_mode 1
    bits = kat_matrix_bits(256, 256)
    t = bits_to_bf16(bits)
    out, meta, gamax, gnnz, gerr = oracle.channel_scaling(bits, bx, by, 0.045, 1)
    assert meta == 1 and gamax == t.float().abs().max().item() and gnnz == 65536
    _, _, gman = decompose(f32(448.0 / float(gamax)))
    exp, total = torch_block_scaling_e4m3(t, bx, by, gman)
    assert bits_to_bf16(out).equal(exp)
    assert abs(total - gerr) <= 1e-3 * total


def test_unscaled_casts_vs_torch_float8():
    # test_fake_quantize.py:570-709
    g = torch.Generator().manual_seed(0)
    for lo, hi in ((-400.0, 400.0), (-1.0, 1.0), (-0.01, 0.01)):
        x = torch.rand(256, 256, generator=g) * (hi - lo) + lo
        got = torch.from_numpy(oracle.quant_dequant(x.numpy(), oracle.FMT_E4M3).reshape(256, 256))
        assert got.equal(x.type(torch.float8_e4m3fn).float())
    x = torch.rand(256, 256, generator=g) * 2000 - 1000
    x[0, :3] = torch.tensor([463.0, 464.0, 465.0])
    got = torch.from_numpy(oracle.quant_dequant(x.numpy(), oracle.FMT_E4M3).reshape(256, 256))
    exp = x.type(torch.float8_e4m3fn).float()
    assert torch.equal(got.isnan(), exp.isnan()) and got[~exp.isnan()].equal(exp[~exp.isnan()])
    x = torch.rand(256, 256, generator=g) * 107536 - 53768
    got = torch.from_numpy(oracle.quant_dequant(x.numpy(), oracle.FMT_E5M2).reshape(256, 256))
    assert got.equal(x.type(torch.float8_e5m2).float())
    x = torch.rand(256, 256, generator=g) * 99.75 + 0.25
    got = torch.from_numpy(oracle.quant_dequant(x.numpy(), oracle.FMT_E3M2).reshape(256, 256))
    assert got.equal(x.type(torch.float8_e5m2).float().clamp(-28.0, 28.0))
    x = torch.rand(256, 256, generator=g) * 19 + 1
    got = torch.from_numpy(oracle.quant_dequant(x.numpy(), oracle.FMT_E2M3).reshape(256, 256))
    assert got.equal(x.type(torch.float8_e4m3fn).float().clamp(-7.5, 7.5))


def test_saturating_cast_vs_torch_float8_all_bf16():
    """the cuda_fp8.h cast (RNE, satfinite) equals torch's cast wherever torch does not overflow"""
    pats = np.arange(65536, dtype=np.uint32)
    x = (pats << 16).astype(np.uint32).view(np.float32)
    L = oracle.lib()
    for fmt, dt, mx in ((oracle.FMT_E4M3, torch.float8_e4m3fn, 448.0), (oracle.FMT_E5M2, torch.float8_e5m2, 57344.0)):
        for s in (1.0, 0.37, 1.9e-3, 31.0):
            xs = (x * np.float32(s)).astype(np.float32)
            got = np.array([L.mor_o_quant_dequant_satfinite(float(v), fmt) for v in xs[::7]], np.float32)
            t = torch.from_numpy(xs[::7].copy())
            exp = t.type(dt).float().numpy()
            fin = np.isfinite(xs[::7]) & (np.abs(xs[::7]) <= mx)
            assert np.array_equal(got[fin].view(np.uint32), exp[fin].view(np.uint32))
            big = np.isfinite(xs[::7]) & (np.abs(xs[::7]) > mx)
            assert np.array_equal(np.abs(got[big]), np.full(big.sum(), mx, np.float32))


def test_e8_scale_ops_vs_torch():
    # test_fake_quantize.py:712-785
    g = torch.Generator().manual_seed(1)
    v = torch.rand(256, 256, generator=g) * 2000 - 1000
    va = v.abs()
    sc = 448.0 / va
    small = 2 ** torch.floor(torch.log2(sc))
    rz = ((v * small).type(torch.float8_e4m3fn).float() / small)
    got = torch.from_numpy(oracle.e4m3_with_e8_scale(v.numpy(), False).reshape(256, 256))
    assert got.equal(rz)
    large = small * 2
    e8 = torch.where((va - va * small) / va <= (va * large - va) / va, small, large)
    e8 = torch.where(va * large <= 464, e8, small)
    rne = ((v * e8).type(torch.float8_e4m3fn).float() / e8)
    got = torch.from_numpy(oracle.e4m3_with_e8_scale(v.numpy(), True).reshape(256, 256))
    assert (got != rne).float().mean() < 0.02  # the torch formula of that test is itself approximate at ties


def test_e8mx_python_model():
    """test/test_e8mx.py:34-129: keep the exponent, RNE on the mantissa with the reference's thresholds"""
    L = oracle.lib()
    rng = np.random.default_rng(0)
    vals = rng.standard_normal(4000).astype(np.float32) * 100
    for m in (1, 2, 3):
        for v in vals:
            b = np.array([v], np.float32).view(np.uint32)[0]
            e, man = (b >> 23) & 0xFF, b & 0x7FFFFF
            step = 0x800000 >> m
            k = (man + step // 2) // step
            if (man + step // 2) % step == 0 and k % 2 == 1 and (man & 0xFFFF) == 0:
                k -= 1  # ties to even
            # the reference ladder only looks at 7 mantissa bits for the tie: recompute exactly
            lims = [j * step + step // 2 - (65536 if j & 1 else 0) for j in range(1 << m)]
            k = next((j for j, lim in enumerate(lims) if man <= lim), 1 << m)
            if k == (1 << m):
                e2, man2 = e + 1, 0
            else:
                e2, man2 = e, k * step
            exp = np.array([(b & 0x80000000) | (e2 << 23) | man2], np.uint32).view(np.float32)[0]
            assert L.mor_o_e8m_round(float(v), m) == exp


def test_recorded_reference_outputs():
    """Outputs of the unmodified reference extension on a B200, replayed through the oracle."""
    if not os.path.exists(GOLDEN):
        pytest.skip("tests/golden/reference_b200.json has not been recorded yet")
    rec = json.load(open(GOLDEN))["cases"]
    checked = 0
    for name, op, fn, kw in cases():
        r = rec.get(name)
        if r is None or "skipped" in r:
            continue
        x = fn()
        assert digest(x) == r["input_sha256"], f"{name}: input bits differ from the recording"
        got = run_oracle(op, x, kw)
        out = got["out"]
        if out.dtype == np.float32:
            out = out.copy()
            out[np.isnan(out)] = np.float32(np.nan)
            out = out.view(np.uint32)
        assert digest(out) == r["out_sha256"], f"{name}: oracle output differs from the reference's"
        if "meta" in r:
            assert np.asarray(got["meta"]).reshape(-1).tolist() == r["meta"], name
        for k in ("gamax", "gerr"):
            if k + "_bits" in r:
                assert int(np.array([got[k]], np.float32).view(np.uint32)[0]) == r[k + "_bits"], f"{name}: {k}"
        if "gnnz" in r:
            assert got["gnnz"] == r["gnnz"], name
        checked += 1
    assert checked >= 90


@pytest.mark.parametrize("fmt", [0, 1, 3])
@pytest.mark.parametrize("by", [8, 32, 128])
def test_quantize_mx_round_trip(fmt, by):
    """The real quantized form (codes + E8M0 scale bytes) decodes to the fake-quantized tensor bit for
    bit, except where a code of zero meets a scale below one: fake quantization returns 2^(-e8-127)
    there (its exponent-field arithmetic, fake_quantize.cu:296-305), the decoded payload zero."""
    g = torch.Generator().manual_seed(fmt * 10 + by)
    t = torch.randn(96, 512, generator=g) * torch.where(torch.rand(96, 512, generator=g) < 0.01, 3000.0, 1.0)
    t[3] = 0.0
    t[5, 40:50] = 0.0
    t[7] *= 1e-20
    x = t.to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    codes, scales = oracle.quantize_mx(x, by, fmt)
    assert oracle.assert_flags() == 0
    deq = oracle.dequantize_mx(codes, scales, by, fmt)
    fq = oracle.fake_quantize_group(x, 1, by, fmt, 2)
    zero_code = (codes & (0x1F if fmt == 3 else 0x7F)) == 0
    scale_below_one = np.repeat(scales > 127, by, axis=1)
    diff = deq != fq
    assert not (diff & ~(zero_code & scale_below_one)).any()
    assert (scales[3] == 127).all() and (codes[3] == 0).all()
    # codes are valid for the format: E2M3 uses six bits, E4M3 never the NaN code for finite input
    if fmt == 3:
        assert (codes < 64).all()
    if fmt == 0:
        assert ((codes & 0x7F) != 0x7F).all()


def test_pack_fp6_layout():
    codes = np.arange(64, dtype=np.uint8).reshape(2, 32)
    p = oracle.pack_fp6(codes)
    assert p.shape == (2, 24)
    # first group 0..7: 0 | 1<<6 | 2<<12 | 3<<18 | 4<<24 | 5<<30 | 6<<36 | 7<<42
    word = sum(i << (6 * i) for i in range(8))
    assert bytes(p[0, :6]) == word.to_bytes(6, "little")
    back = np.zeros_like(codes)
    for gi in range(8):
        w = int.from_bytes(bytes(p.reshape(-1)[6 * gi:6 * gi + 6]), "little")
        back.reshape(-1)[8 * gi:8 * gi + 8] = [(w >> (6 * i)) & 63 for i in range(8)]
    assert np.array_equal(back, codes)


@pytest.mark.parametrize("brows,bcols", [(128, 128), (32, 64), (1, 256), (64, 1)])
@pytest.mark.parametrize("ss", [1, 3, 4])
@pytest.mark.parametrize("dtype", ["bf16", "f32"])
def test_quantize_scaled_round_trip(brows, bcols, ss, dtype):
    """E4M3 bytes + binary32 scales: decode(code) / scale is the fake-quantized tensor, bit for bit"""
    g = torch.Generator().manual_seed(brows + bcols + ss)
    t = torch.randn(256, 512, generator=g) * 10.0 ** (torch.rand(256, 512, generator=g) * 4 - 2)
    t[5, 7] = 0.0
    t[9, 11] = -0.0
    x = t.numpy().copy() if dtype == "f32" else oracle.bf16_bits(t.to(torch.bfloat16))
    payload, scales, gamax = oracle.quantize_scaled(x, brows, bcols, ss)
    fn = oracle.channel_scaling if (brows == 1 or bcols == 1) else oracle.block_scaling
    fq = fn(x, brows, bcols, 3e38, ss)
    assert np.float32(gamax) == np.float32(fq[2])
    deq = oracle.dequantize_scaled(payload, scales, brows, bcols, float32=(dtype == "f32"))
    assert np.array_equal(deq.view(np.uint8), np.ascontiguousarray(fq[0]).view(np.uint8))
    assert payload[5, 7] == 0 and payload[9, 11] == 0
    # the bytes are what torch's own E4M3 type holds for the scaled values
    xf = t.numpy() if dtype == "f32" else t.to(torch.bfloat16).float().numpy()
    s_full = np.repeat(np.repeat(scales, brows, axis=0), bcols, axis=1)
    ref = (torch.from_numpy(xf * s_full).clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8).numpy())
    nz = xf != 0
    assert np.array_equal(payload[nz], ref[nz])
