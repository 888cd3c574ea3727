"""Bit-exact parity of the CUDA kernels (through the C ABI) with the CPU oracle.

bf16 outputs, meta matrices, amax, non-zero counts and error sums must be identical
bit for bit; float32 outputs likewise except that NaNs compare by position (payloads of
NaNs are not defined by the reference).  No tolerance is used anywhere in this file.
"""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import oracle
from cases import cases
from replay import run_oracle

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def canon(a):
    a = np.asarray(a)
    if a.dtype == np.float32:
        b = a.copy()
        b[np.isnan(b)] = np.float32(np.nan)
        return b.view(np.uint32)
    return a


def f32_bits(v):
    return int(np.array([v], np.float32).view(np.uint32)[0])


def assert_same(got: dict, exp: dict, what: str):
    a, b = canon(got["out"]).reshape(-1), canon(exp["out"]).reshape(-1)
    bad = np.nonzero(a != b)[0]
    assert bad.size == 0, f"{what}: {bad.size}/{a.size} outputs differ, first at {bad[:8].tolist()}: cuda {a[bad[:8]].tolist()} oracle {b[bad[:8]].tolist()}"
    if "meta" in exp:
        assert np.array_equal(np.asarray(got["meta"]).reshape(-1), np.asarray(exp["meta"]).reshape(-1)), \
            f"{what}: meta cuda {np.asarray(got['meta']).reshape(-1)[:32]} oracle {np.asarray(exp['meta']).reshape(-1)[:32]}"
    for k in ("gamax", "gerr"):
        if k in exp:
            assert f32_bits(got[k]) == f32_bits(exp[k]), f"{what}: {k} cuda {got[k]!r} oracle {float(exp[k])!r}"
    if "gnnz" in exp:
        assert got["gnnz"] == exp["gnnz"], f"{what}: nnz cuda {got['gnnz']} oracle {exp['gnnz']}"


ALL_CASES = cases()


@pytest.fixture(params=[0, 2], ids=["single-launch", "launch-sequence"])
def selection(request):
    """Small block-scaled tensors take the single-launch kernel by default; mask 2 sends them through the
    sequence of launches that large tensors use, so that both are compared with the oracle on the same input."""
    from mor_b200 import cabi
    cabi.lib().mor_b200_debug_kernel_selection(request.param)
    yield request.param
    cabi.lib().mor_b200_debug_kernel_selection(0)


@pytest.mark.parametrize("case", ALL_CASES, ids=[c[0] for c in ALL_CASES])
def test_golden_case_matches_oracle(case, selection):
    if selection and case[1] != "fake_quantize_block_scaling":
        pytest.skip("one kernel only")
    import gpu_harness as H
    name, op, fn, kw = case
    x = fn()
    assert_same(H.run_case(op, x, kw), run_oracle(op, x, kw), name)


# ------------------------------------------------------------------ exhaustive element sweeps
def all_bf16_patterns(finite_only: bool) -> np.ndarray:
    p = np.arange(65536, dtype=np.uint32).astype(np.uint16)
    if finite_only:
        p = p.copy()
        p[(p & 0x7F80) == 0x7F80] = 0
    return p.reshape(256, 256)


SWEEP_SCALES = [1.0, 448.0 / 240.0, 0.37, 3.0e-3, 7.0e4, 2.0 ** -20, 1.0e-30, 5.1e27, 0.99999994, 57344.0 / 3.0]


@pytest.mark.parametrize("mode,sf", [(4, 1), (5, 1), (4, 2), (5, 2)])
def test_every_bf16_pattern_uniform_scale(mode, sf):
    import gpu_harness as H
    x = all_bf16_patterns(finite_only=(sf == 2))
    for s in SWEEP_SCALES:
        if sf == 2 and not (1e-20 < s < 1e20):
            continue  # exponent-field arithmetic leaves the reference's asserted domain
        oracle.clear_assert_flags()
        exp = dict(zip(("out", "meta"), oracle.fake_quantize(x, 128, 128, s, mode, sf)))
        if oracle.assert_flags():
            continue
        assert_same(H.fake_quantize(x, 128, 128, s, mode, sf), exp, f"mode {mode} sf {sf} scale {s}")


@pytest.mark.parametrize("fmt", [oracle.FMT_E4M3, oracle.FMT_E5M2, oracle.FMT_E2M3])
@pytest.mark.parametrize("sf", [1, 2])
def test_every_bf16_pattern_group_scaled(fmt, sf):
    """65536 patterns shuffled into 1 x 32 groups and into full rows: every pattern meets many scales."""
    import gpu_harness as H
    rng = np.random.default_rng(123)
    pats = all_bf16_patterns(finite_only=True).reshape(-1)
    for rep in range(3):
        x = rng.permutation(pats).reshape(256, 256)
        if sf == 2:
            # keep each group's dynamic range inside the exponent field: sort so neighbours are similar
            x = np.sort(x.reshape(-1) & 0x7FFF).astype(np.uint16).reshape(256, 256) | (x & 0x8000)
        for by in (32, 256):
            oracle.clear_assert_flags()
            out, scales = oracle.fake_quantize_group(x, 1, by, fmt, sf, want_scales=True)
            if oracle.assert_flags():
                continue
            got = H.fake_quantize_group(x, by, fmt, sf)
            assert_same(got, {"out": out}, f"group fmt {fmt} sf {sf} by {by} rep {rep}")
            assert np.array_equal(got["scales"].view(np.uint32), scales.view(np.uint32))


@pytest.mark.parametrize("by", [32, 256, 1024])
def test_group_scaled_with_nan_and_inf_elements(by):
    """a NaN is skipped by the group amax (fmaxf) and comes out as 0x8000; the other elements are unaffected"""
    import gpu_harness as H
    x = rand_bits(700 + by, 64, 2048, "normal")
    x[3, 5] = 0x7FC0
    x[3, 700] = 0xFFC1
    x[40, 100] = 0x7F80   # +inf: the group's scale becomes 0
    for fmt in (oracle.FMT_E4M3, oracle.FMT_E5M2):
        out, scales = oracle.fake_quantize_group(x, 1, by, fmt, 1, want_scales=True)
        got = H.fake_quantize_group(x, by, fmt, 1)
        assert_same(got, {"out": out}, f"group with NaN fmt {fmt} by {by}")
    # power-of-two scales: non-finite values are outside the reference's domain (it asserts);
    # here they must not fault, and groups without them must still be exact
    clean = np.ones(x.shape, bool)
    for r, c in ((3, 5), (3, 700), (40, 100)):
        clean[r, (c // by) * by:(c // by + 1) * by] = False
    for fmt in (oracle.FMT_E4M3, oracle.FMT_E2M3):
        out = oracle.fake_quantize_group(x, 1, by, fmt, 2)
        got = H.fake_quantize_group(x, by, fmt, 2, want_scales=False)["out"]
        assert np.array_equal(got[clean], out[clean])
    assert torch.zeros(1, device="cuda").item() == 0.0


@pytest.mark.parametrize("qtype", [1, 2, 3])
@pytest.mark.parametrize("strategy", [0, 1])
@pytest.mark.parametrize("top", [0x7F7F, 0x4680, 0x3F80, 0x0200])
def test_e8mx_every_bf16_pattern(qtype, strategy, top, selection):
    """E8Mx on every finite bf16 pattern up to a largest magnitude `top` (which sets the tensor scale under strategy 1):
    the tabulated offsets of the fast path, the literal path at both ends of the exponent range, zeros of both signs;
    through the single launch that small tensors take and through the amax kernel + element kernel"""
    import gpu_harness as H
    mags = np.arange(0, top + 1, dtype=np.uint32)
    pats = np.concatenate([mags, mags | 0x8000]).astype(np.uint16)
    pad = (-pats.size) % 512
    x = np.concatenate([pats, np.zeros(pad, np.uint16)]).reshape(-1, 512)
    oracle.clear_assert_flags()
    exp, _ = oracle.e8mx(x, qtype, strategy)
    if oracle.assert_flags():
        pytest.skip("the reference asserts on this input")
    got = H.e8mx(x, qtype, strategy)["out"]
    bad = np.nonzero(got.reshape(-1) != exp.reshape(-1))[0]
    assert bad.size == 0, f"e8m{qtype} strategy {strategy}: {bad.size} differ, e.g. in {x.reshape(-1)[bad[:5]]} got {got.reshape(-1)[bad[:5]]} want {exp.reshape(-1)[bad[:5]]}"


@pytest.mark.parametrize("rows,cols", [(1000, 520), (148 * 7 * 4, 4096), (148 * 7 * 4 + 1, 4096), (3, 8)])
def test_e8mx_single_launch_sizes(rows, cols, selection):
    """the single-launch E8Mx kernel keeps up to 148 x 7 chunks of 32 KiB in shared memory: a ragged last chunk,
    exactly the capacity, one row more (the launch sequence takes over), a tensor smaller than one chunk"""
    import gpu_harness as H
    from ref_fixtures import bf16_bits
    g = torch.Generator().manual_seed(rows)
    x = bf16_bits((torch.randn(rows, cols, generator=g) * 3.0).to(torch.bfloat16))
    x[0, 0] = 0x0000; x[0, 1] = 0x8000; x[rows - 1, cols - 1] = 0x4680   # zeros of both signs; the largest magnitude last
    exp, _ = oracle.e8mx(x, 3, 1)
    got = H.e8mx(x, 3, 1)["out"]
    assert np.array_equal(got, exp), f"e8m3 {rows}x{cols}"


def test_unscaled_casts_every_bf16_pattern_and_neighbours():
    """quant_dequant_*: all bf16 patterns widened to float32, plus values just off the rounding ties."""
    import gpu_harness as H
    base = (all_bf16_patterns(False).astype(np.uint32) << 16)
    for delta in (0, 1, 0x7FFF, 0x8000, 0x8001, 0xFFFF):
        x = (base + np.uint32(delta)).view(np.float32)
        for fmt in (oracle.FMT_E4M3, oracle.FMT_E5M2, oracle.FMT_E3M2, oracle.FMT_E2M3):
            exp = oracle.quant_dequant(x, fmt).reshape(x.shape)
            # the custom cast has no defined result for NaN inputs of E4M3/E5M2 beyond "NaN"
            assert_same(H.quant_dequant(x, fmt), {"out": exp}, f"quant_dequant fmt {fmt} delta {delta:#x}")


def test_exact_division_building_blocks():
    """Hardware fp8/fp6 conversions agree with the oracle's casts on a dense float32 sweep."""
    import gpu_harness as H
    rng = np.random.default_rng(5)
    # dense around every binade boundary and tie of the formats, both signs
    mant = rng.integers(0, 1 << 23, size=1 << 18, dtype=np.uint32)
    expo = rng.integers(127 - 20, 127 + 18, size=1 << 18, dtype=np.uint32)
    sign = rng.integers(0, 2, size=1 << 18, dtype=np.uint32)
    x = ((sign << 31) | (expo << 23) | mant).view(np.float32).reshape(512, 512)
    xb = (x.view(np.uint32) >> 16).astype(np.uint16)  # as bf16
    for fmt in (oracle.FMT_E4M3, oracle.FMT_E5M2, oracle.FMT_E2M3):
        for sf in (1, 2):
            exp = oracle.fake_quantize_group(xb, 1, 512, fmt, sf)
            got = H.fake_quantize_group(xb, 512, fmt, sf, want_scales=False)
            assert_same(got, {"out": exp}, f"row-group fmt {fmt} sf {sf}")


# ------------------------------------------------------------------ shapes, aliasing, dtypes
def rand_bits(seed, rows, cols, kind="normal"):
    g = torch.Generator().manual_seed(seed)
    if kind == "normal":
        t = torch.randn(rows, cols, generator=g)
    elif kind == "wide":
        t = 10.0 ** (torch.rand(rows, cols, generator=g) * 8 - 4) * torch.where(torch.rand(rows, cols, generator=g) < 0.5, -1.0, 1.0)
    else:
        t = torch.rand(rows, cols, generator=g) * 2 - 1
    z = torch.rand(rows, cols, generator=g) < 0.05
    t = torch.where(z, 0.0, t)
    return t.to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)


@pytest.mark.parametrize("rows,cols,bx,by", [(200, 136, 128, 128), (250, 130, 96, 64), (64, 66, 32, 32),
                                              (33, 64, 32, 64), (256, 256, 4, 16), (128, 128, 2, 32),
                                              (384, 640, 128, 128), (96, 192, 32, 64)])
@pytest.mark.parametrize("mode", [1, 101, 2, 3])
def test_fake_quantize_ragged_and_odd_blocks(rows, cols, bx, by, mode):
    import gpu_harness as H
    x = rand_bits(rows * 7 + cols + mode, rows, cols, "wide" if mode in (1, 101) else "normal")
    for sf in (1, 2):
        oracle.clear_assert_flags()
        try:
            exp = dict(zip(("out", "meta"), oracle.fake_quantize(x, bx, by, 1e-15, mode, sf)))
        except oracle.OracleError:
            from mor_b200 import cabi
            with pytest.raises(cabi.MorB200Error):
                H.fake_quantize(x, bx, by, 1e-15, mode, sf)
            continue
        if oracle.assert_flags():
            continue
        assert_same(H.fake_quantize(x, bx, by, 1e-15, mode, sf), exp, f"{rows}x{cols} block {bx}x{by} mode {mode} sf {sf}")


@pytest.mark.parametrize("shift", [-118, -112, -104, -96, 90])
@pytest.mark.parametrize("sf", [1, 2])
def test_mor_error_pass_with_extreme_magnitudes(shift, sf):
    """blocks scaled by 2^-96 / 2^90 leave the range of the short exact quotient: the IEEE division takes over;
    below that the quotients q / scale turn denormal, where the error table's binade folding does not hold"""
    import gpu_harness as H
    from cases import mixed_blocks_bf16
    from ref_fixtures import bits_to_bf16, bf16_bits
    t = bits_to_bf16(mixed_blocks_bf16(7)).float() * (2.0 ** shift)
    x = bf16_bits(t.to(torch.bfloat16))
    oracle.clear_assert_flags()
    exp = dict(zip(("out", "meta"), oracle.fake_quantize(x, 128, 128, 1e-38, 1, sf)))
    if oracle.assert_flags():
        pytest.skip("outside the reference's asserted domain")
    assert_same(H.fake_quantize(x, 128, 128, 1e-38, 1, sf), exp, f"MoR shift {shift} sf {sf}")


@pytest.mark.parametrize("by", [8, 16, 32, 64, 128, 256, 1024, 4096])
@pytest.mark.parametrize("mode", [2, 3])
def test_fake_quantize_row_groups(by, mode):
    """fixed-format modes with 1 x k blocks run on the single-pass group kernels"""
    import gpu_harness as H
    x = rand_bits(by + mode, 64, 4096, "wide")
    for sf in (1, 2):
        oracle.clear_assert_flags()
        exp = dict(zip(("out", "meta"), oracle.fake_quantize(x, 1, by, 1e-15, mode, sf)))
        if oracle.assert_flags():
            continue
        assert_same(H.fake_quantize(x, 1, by, 1e-15, mode, sf), exp, f"1x{by} mode {mode} sf {sf}")


@pytest.mark.parametrize("mode,sf", [(1, 1), (101, 2), (2, 1), (4, 1), (7, 1)])
def test_fake_quantize_in_place(mode, sf):
    import gpu_harness as H
    from cases import mixed_blocks_bf16
    x = mixed_blocks_bf16(77)
    clamp = 0.5 if mode == 4 else 1e-15
    exp = dict(zip(("out", "meta"), oracle.fake_quantize(x, 128, 128, clamp, mode, sf)))
    assert_same(H.fake_quantize(x, 128, 128, clamp, mode, sf, inplace=True), exp, f"in place mode {mode}")


@pytest.fixture(params=[0, 1], ids=["single-pass", "two-pass"])
def channel_passes(request):
    """1 x k groups under strategies 2 and 3 run in one pass by default; mask 1 sends them through the amax
    pass and the generic kernels, so that both are compared with the oracle on the same input."""
    from mor_b200 import cabi
    cabi.lib().mor_b200_debug_kernel_selection(request.param)
    yield request.param
    cabi.lib().mor_b200_debug_kernel_selection(0)


@pytest.mark.parametrize("by", [8, 16, 32, 64, 128, 256, 512])
@pytest.mark.parametrize("ss", [1, 2, 3, 4])
def test_channel_scaling_row_groups(by, ss, channel_passes):
    import gpu_harness as H
    if channel_passes and ss not in (2, 3):
        pytest.skip("strategies 1 and 4 always run two passes")
    x = rand_bits(by * 10 + ss, 96, 512, "wide" if ss != 2 else "normal")
    for thr in (0.045, 3e38):
        oracle.clear_assert_flags()
        exp = dict(zip(("out", "meta", "gamax", "gnnz", "gerr"), oracle.channel_scaling(x, 1, by, thr, ss)))
        if oracle.assert_flags():
            continue
        exp["meta"] = np.array([exp["meta"]])
        assert_same(H.channel_scaling(x, 1, by, thr, ss), exp, f"1x{by} ss {ss} thr {thr}")


@pytest.mark.parametrize("by", [8, 16, 32, 64])
@pytest.mark.parametrize("kind", ["dense", "dense_large", "sparse_large", "tiny_rows"])
@pytest.mark.parametrize("rows,cols", [(33, 384), (520, 640)])
def test_channel_scaling_small_groups_power_of_two(by, kind, rows, cols, channel_passes):
    """1 x k groups with k < 128 and a power-of-two scale (ss_mode 2): tensors without zeros, groups whose
    amax exceeds the format maximum (scale below one), ragged ends (vector count 16 mod 32, partial chunks)."""
    import gpu_harness as H
    g = torch.Generator().manual_seed(by + rows)
    t = torch.randn(rows, cols, generator=g)
    t = torch.where(t == 0, torch.ones_like(t), t)
    if kind in ("dense_large", "sparse_large"):
        t = t * torch.where(torch.rand(rows, cols, generator=g) < 0.3, 3000.0, 1.0)
    if kind == "sparse_large":
        t = torch.where(torch.rand(rows, cols, generator=g) < 0.1, 0.0, t)
    if kind == "tiny_rows":
        t[::3] *= 1e-30     # group maxima below 1e-35 * 2^12 leave the short form's domain
    x = t.to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    for thr in (0.045, 3e38):
        oracle.clear_assert_flags()
        exp = dict(zip(("out", "meta", "gamax", "gnnz", "gerr"), oracle.channel_scaling(x, 1, by, thr, 2)))
        if oracle.assert_flags():
            continue
        exp["meta"] = np.array([exp["meta"]])
        assert_same(H.channel_scaling(x, 1, by, thr, 2), exp, f"{kind} {rows}x{cols} 1x{by} thr {thr}")


@pytest.mark.parametrize("by", [4096, 8192])
def test_channel_rows_with_mixed_magnitudes(by):
    """Long rows under their own binary32 scale: rows whose elements are all normal E4M3 numbers under the row's
    scale, rows that mix them with E4M3 denormals and zeros, rows at both ends of the bf16 exponent range, an
    all-zero row, a row with a single non-zero element"""
    import gpu_harness as H
    from ref_fixtures import bf16_bits
    g = torch.Generator().manual_seed(by)
    x = torch.randn(32, 8192, generator=g)
    x[1] *= 2.0 ** -112                      # amax below 2^-100
    x[2] *= 2.0 ** 100                       # a large scale exponent the other way
    x[3, ::64] *= 2.0 ** -16                 # one element of every step below the normal range
    x[4, 100:164] = 0.0                      # a step of zeros, and a step that straddles them
    x[5] = 0.0                               # nothing but zeros
    x[6] = 0.0; x[6, 77] = -3.0              # a single non-zero element
    x[7, :4096] *= 2.0 ** -20                # half a row of E4M3 denormals and zeros after the cast
    x[8] = x[8].abs() * 2.0 ** -126          # bf16 denormals and the smallest normals
    x[9, 5] = 3.0e38                         # the largest finite magnitudes
    bits = bf16_bits(x.to(torch.bfloat16))
    oracle.clear_assert_flags()
    exp = dict(zip(("out", "meta", "gamax", "gnnz", "gerr"), oracle.channel_scaling(bits, 1, by, 3e38, 3)))
    assert not oracle.assert_flags()
    exp["meta"] = np.array([exp["meta"]])
    assert_same(H.channel_scaling(bits, 1, by, 3e38, 3), exp, f"1x{by} rows with mixed magnitudes")


@pytest.mark.parametrize("by", [2048, 4096, 8192])
@pytest.mark.parametrize("ss", [1, 2, 3, 4])
@pytest.mark.parametrize("kind", ["normal", "wide", "nan"])
def test_channel_scaling_long_rows(by, ss, kind, channel_passes):
    """1 x k blocks of 4 KiB and more: the amax pass streams every block through one warp's ring"""
    import gpu_harness as H
    if kind == "nan" and ss == 2:
        pytest.skip("non-finite inputs are outside the reference's domain for power-of-two scales")
    x = rand_bits(by + ss, 24, 8192, "wide" if kind == "wide" else "normal")
    x[5] = (x[5] & 0x8000) | ((x[5] & 0x7FFF) | 1)        # a row without a single zero
    if kind == "nan":
        x[7, 4000] = 0x7FC0
    oracle.clear_assert_flags()
    exp = dict(zip(("out", "meta", "gamax", "gnnz", "gerr"), oracle.channel_scaling(x, 1, by, 3e38, ss)))
    if oracle.assert_flags():
        pytest.skip("the reference asserts on this input")
    exp["meta"] = np.array([exp["meta"]])
    got = H.channel_scaling(x, 1, by, 3e38, ss)
    if kind == "nan":
        assert np.isnan(got["gerr"]) and np.isnan(exp["gerr"])
        got["gerr"] = exp["gerr"] = 0.0
    assert_same(got, exp, f"{kind} 1x{by} ss {ss}")


@pytest.mark.parametrize("bx,rows", [(256, 256), (64, 256), (16, 64), (128, 384)])
@pytest.mark.parametrize("ss", [1, 2, 3, 4])
def test_channel_scaling_column_groups(bx, rows, ss):
    import gpu_harness as H
    x = rand_bits(bx + rows + ss, rows, 192, "normal")
    for thr in (0.045, 3e38):
        oracle.clear_assert_flags()
        exp = dict(zip(("out", "meta", "gamax", "gnnz", "gerr"), oracle.channel_scaling(x, bx, 1, thr, ss)))
        if oracle.assert_flags():
            continue
        exp["meta"] = np.array([exp["meta"]])
        assert_same(H.channel_scaling(x, bx, 1, thr, ss), exp, f"{bx}x1 ss {ss} thr {thr}")


@pytest.mark.parametrize("kind", ["block", "row", "col"])
@pytest.mark.parametrize("thr", [0.045, 1e-6])
def test_scaling_in_place(kind, thr, selection):
    """in place: the input must survive until the tensor-level BF16 decision (thr=1e-6 forces it)"""
    import gpu_harness as H
    if selection and kind != "block":
        pytest.skip("one kernel only")
    x = rand_bits(91, 256, 256, "normal")
    if kind == "block":
        exp = oracle.block_scaling(x, 128, 128, thr, 1)
        got = H.block_scaling(x, 128, 128, thr, 1, inplace=True)
    elif kind == "row":
        exp = oracle.channel_scaling(x, 1, 256, thr, 1)
        got = H.channel_scaling(x, 1, 256, thr, 1, inplace=True)
    else:
        exp = oracle.channel_scaling(x, 256, 1, thr, 1)
        got = H.channel_scaling(x, 256, 1, thr, 1, inplace=True)
    e = dict(zip(("out", "meta", "gamax", "gnnz", "gerr"), exp))
    e["meta"] = np.array([e["meta"]])
    assert e["meta"][0] == (3 if thr < 1e-3 else 1)
    assert_same(got, e, f"in place {kind} thr {thr}")


@pytest.mark.parametrize("kind", ["tiny", "huge", "nan"])
@pytest.mark.parametrize("ss", [1, 2, 3, 4])
def test_scaling_with_extreme_magnitudes(kind, ss, selection):
    """values outside [2^-90, 2^90) (or a NaN) switch the error quotient to the IEEE division: same bits"""
    import gpu_harness as H
    x = rand_bits(300 + ss, 256, 256, "normal")
    if kind == "tiny":
        x[7, 9] = 0x0081      # 1.2e-38
        x[130, 200] = 0x8F00  # -6.3e-30
    elif kind == "huge":
        x[:128, :128] = rand_bits(301, 128, 128, "normal") + np.uint16(0x3000)  # times 2^96
    else:
        if ss == 2:
            pytest.skip("non-finite inputs are outside the reference's domain for power-of-two scales")
        x[3, 3] = 0x7FC0
    for (op, h, bx, by) in ((oracle.block_scaling, H.block_scaling, 128, 128), (oracle.channel_scaling, H.channel_scaling, 1, 256),
                            (oracle.channel_scaling, H.channel_scaling, 1, 32)):
        oracle.clear_assert_flags()
        e = dict(zip(("out", "meta", "gamax", "gnnz", "gerr"), op(x, bx, by, 3e38, ss)))
        if oracle.assert_flags():
            continue
        e["meta"] = np.array([e["meta"]])
        got = h(x, bx, by, 3e38, ss)
        if kind == "nan":   # the error sum is NaN on both sides; compare everything else exactly
            assert np.isnan(got["gerr"]) and np.isnan(e["gerr"])
            got["gerr"] = e["gerr"] = 0.0
        assert_same(got, e, f"{kind} ss {ss} {bx}x{by}")


@pytest.mark.parametrize("ss", [1, 2, 3, 4])
def test_block_scaling_float32(ss, selection):
    import gpu_harness as H
    g = torch.Generator().manual_seed(50 + ss)
    x = torch.randn(256, 512, generator=g).numpy()
    x[5, 7] = 0.0
    for bx, by in ((128, 128), (32, 64)):
        e = dict(zip(("out", "meta", "gamax", "gnnz", "gerr"), oracle.block_scaling(x, bx, by, 0.045, ss)))
        e["meta"] = np.array([e["meta"]])
        assert_same(H.block_scaling(x, bx, by, 0.045, ss), e, f"float32 block scaling ss {ss} {bx}x{by}")


def test_group_and_generic_float32():
    import gpu_harness as H
    g = torch.Generator().manual_seed(60)
    x = (torch.randn(64, 1024, generator=g) * 3).numpy()
    for fmt in (oracle.FMT_E4M3, oracle.FMT_E5M2, oracle.FMT_E2M3):
        for sf in (1, 2):
            for by in (32, 1024):
                out, sc = oracle.fake_quantize_group(x, 1, by, fmt, sf, want_scales=True)
                got = H.fake_quantize_group(x, by, fmt, sf)
                assert_same(got, {"out": out}, f"float32 group fmt {fmt} sf {sf} by {by}")
                assert np.array_equal(got["scales"].view(np.uint32), sc.view(np.uint32))
    for mode in (1, 101, 2, 3):
        exp = dict(zip(("out", "meta"), oracle.fake_quantize(x, 32, 64, 1e-15, mode, 1)))
        assert_same(H.fake_quantize(x, 32, 64, 1e-15, mode, 1), exp, f"float32 generic mode {mode}")


def test_generic_block_kernel_matches_tile_kernel():
    """mor_b200_debug_kernel_selection(1) routes 128x128 blocks (and the block pipeline) through the generic kernels;
    same bits expected."""
    import gpu_harness as H
    from cases import mixed_blocks_bf16
    from mor_b200 import cabi
    x = mixed_blocks_bf16(7)
    cabi.lib().mor_b200_debug_kernel_selection(1)
    try:
        for mode, sf in ((1, 1), (101, 1), (1, 2), (2, 1), (3, 2)):
            out, meta = oracle.fake_quantize(x, 128, 128, 1e-15, mode, sf)
            g = H.fake_quantize(x, 128, 128, 1e-15, mode, sf)
            assert np.array_equal(g["out"], out) and np.array_equal(g["meta"], meta), (mode, sf)
        for ss in (1, 2, 3, 4):
            exp = dict(zip(("out", "meta", "gamax", "gnnz", "gerr"), oracle.block_scaling(x, 128, 128, 0.045, ss)))
            exp["meta"] = np.array([exp["meta"]])
            assert_same(H.block_scaling(x, 128, 128, 0.045, ss), exp, f"generic block pipeline ss {ss}")
    finally:
        cabi.lib().mor_b200_debug_kernel_selection(0)


@pytest.mark.parametrize("stride", [1, 4, 64])
@pytest.mark.parametrize("n", [1, 1000, 32768, 65536, 65537, 200001, 1 << 20])
def test_ordered_error_sum_of_long_arrays(n, stride):
    """The tensor-level error sum is order-sensitive (ref: 1178-1241); arrays above 65536 entries
    take the path that spreads the independent sequential sums over CTAs."""
    from mor_b200 import cabi
    rng = np.random.default_rng(n * 7 + stride)
    err = (rng.random(n, dtype=np.float32) * np.float32(10.0) ** rng.integers(-6, 3, n).astype(np.float32)).astype(np.float32)
    nnz = int(n) * 100
    want_meta, want_total = oracle.finalize(err, stride, nnz, 0.045)
    d_err = torch.from_numpy(err).cuda()
    d_nnz = torch.tensor([nnz], dtype=torch.int64, device="cuda")
    meta = torch.zeros(1, dtype=torch.int32, device="cuda")
    total = torch.zeros(1, dtype=torch.float32, device="cuda")
    wsb = cabi.workspace_bytes(cabi.OP_AMAX_NNZ, 1, 1, 1, 1)
    ws = torch.zeros(wsb, dtype=torch.uint8, device="cuda")  # the head carries flags of the earlier phases
    cabi.call("mor_b200_scaling_finalize", d_err.data_ptr(), n, stride, d_nnz.data_ptr(), 0.045, meta.data_ptr(),
              total.data_ptr(), ws.data_ptr(), wsb, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert total.cpu().numpy().view(np.uint32)[0] == np.float32(want_total).view(np.uint32)
    assert int(meta.item()) == int(want_meta)


@pytest.mark.parametrize("fmt", [0, 1, 3])
@pytest.mark.parametrize("by", [8, 16, 32, 64, 128, 256])
def test_quantize_mx_codes_and_scales(fmt, by):
    """codes and E8M0 scale bytes of the real quantized output against the oracle, bit for bit"""
    import gpu_harness as H
    g = torch.Generator().manual_seed(fmt * 100 + by)
    rows, cols = 72, 1024
    t = torch.randn(rows, cols, generator=g) * torch.where(torch.rand(rows, cols, generator=g) < 0.01, 3000.0, 1.0)
    t[3] = 0.0
    t[5, 40:50] = 0.0
    t[7] *= 1e-20
    t[9] *= 1e-36      # subnormal bf16 values: scale exponents outside the short form's range
    t[11] *= 1e30
    x = t.to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    oracle.clear_assert_flags()
    codes, scales = oracle.quantize_mx(x, by, fmt)
    assert oracle.assert_flags() == 0
    got = H.quantize_mx(x, by, fmt)
    assert np.array_equal(got["scales"], scales), f"scale bytes fmt {fmt} 1x{by}"
    bad = np.argwhere(got["payload"] != codes)
    assert bad.size == 0, f"codes fmt {fmt} 1x{by}: first mismatch at {bad[0]}: {got['payload'][tuple(bad[0])]:#x} vs {codes[tuple(bad[0])]:#x}"


@pytest.mark.parametrize("by", [8, 32, 128])
def test_quantize_mx_fp6_packed(by):
    """E2M3 codes packed six bits each equal the oracle's codes packed on the CPU"""
    import gpu_harness as H
    g = torch.Generator().manual_seed(by)
    t = torch.randn(40, 1024, generator=g) * torch.where(torch.rand(40, 1024, generator=g) < 0.01, 300.0, 1.0)
    t[3] = 0.0
    x = t.to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    oracle.clear_assert_flags()
    codes, scales = oracle.quantize_mx(x, by, 3)
    assert oracle.assert_flags() == 0
    got = H.quantize_mx_fp6(x, by)
    assert np.array_equal(got["scales"], scales)
    assert np.array_equal(got["payload"], oracle.pack_fp6(codes))


@pytest.mark.parametrize("bx,by", [(128, 128), (32, 64), (1, 256), (1, 2048), (64, 1), (256, 1)])
@pytest.mark.parametrize("ss", [1, 3, 4])
@pytest.mark.parametrize("dtype", ["bf16", "f32"])
def test_quantize_scaled_codes_and_scales(bx, by, ss, dtype):
    """E4M3 bytes and binary32 scales of the block / channel pipelines: equal to the oracle's, with this tensor's amax
    and with a larger one handed in (row sharding)"""
    import gpu_harness as H
    g = torch.Generator().manual_seed(bx + by + ss)
    t = torch.randn(256, 2048, generator=g) * 10.0 ** (torch.rand(256, 2048, generator=g) * 4 - 2)
    t[5, 7] = 0.0
    t[9, 11] = -0.0
    t[128:, :512] = 0.0
    x = t.numpy().copy() if dtype == "f32" else oracle.bf16_bits(t.to(torch.bfloat16))
    for amax_in in (None, 3.0e4):
        payload, scales, gamax = oracle.quantize_scaled(x, bx, by, ss, global_amax=amax_in)
        got = H.quantize_scaled(x, bx, by, ss, amax_in)
        assert np.array_equal(got["scales"].view(np.uint32), scales.view(np.uint32)), f"scales, amax_in {amax_in}"
        bad = np.nonzero(got["payload"] != payload)
        assert bad[0].size == 0, f"{bad[0].size} codes differ, first at {bad[0][:4]}, {bad[1][:4]}"
        assert np.float32(got["gamax"]) == np.float32(gamax)


def test_quantize_mx_round_trip_full_size():
    """configuration 3 at full size (16384 x 8192, 1 x 32 groups): decode(code) * 2^(scale - 127) equals the
    fake-quantized tensor wherever the code is non-zero or the scale is at least one"""
    import mor
    from mor_b200 import workloads
    x = workloads.config3(device="cuda")
    r, c = x.shape
    for fmt, lut_bits in ((0, None), (3, None)):
        payload, scales = mor.ops.quantize_mx(x, r, c, 32, fmt)
        fq, _ = mor.ops.fake_quantize_mx(x, r, c, 32, fmt, 2)
        if fmt == 0:
            dec = payload.view(torch.float8_e4m3fn).to(torch.float32)
        else:   # E2M3: sign, two exponent bits (bias 1), three mantissa bits
            p = payload.to(torch.int32)
            e, m = (p >> 3) & 3, (p & 7).to(torch.float32)
            mag = torch.where(e == 0, m * 0.125, (1.0 + m * 0.125) * torch.exp2((e - 1).to(torch.float32)))
            dec = torch.where((p & 32) != 0, -mag, mag)
        deq = (dec.view(r, c // 32, 32) * torch.exp2(scales.to(torch.float32) - 127.0).unsqueeze(-1)).view(r, c)
        same = deq.to(torch.bfloat16).view(torch.int16) == fq.view(torch.int16)
        zero_code = (payload & (0x7F if fmt == 0 else 0x1F)) == 0
        below_one = (scales > 127).repeat_interleave(32, dim=1)
        assert bool((same | (zero_code & below_one)).all())
        assert float(same.float().mean()) > 0.9


@pytest.mark.parametrize("dtype", ["bf16", "f32"])
@pytest.mark.parametrize("ss", [1, 2, 3, 4])
@pytest.mark.parametrize("kind", ["same", "stale_small", "stale_large", "zeros", "nan", "tiny"])
def test_block_scaling_delayed_amax(dtype, ss, kind):
    """single-pass block scaling with the tensor amax of an earlier step: output, meta, count and error equal
    the two-pass arithmetic run with that amax; the reported amax is this tensor's"""
    import gpu_harness as H
    g = torch.Generator().manual_seed(ss * 7 + len(kind))
    t = torch.randn(384, 512, generator=g) * 3.0
    if kind == "zeros":
        t = torch.where(torch.rand(384, 512, generator=g) < 0.2, 0.0, t)
        t[:128, :128] = 0.0
    if kind == "tiny":
        t[128:256, 128:256] *= 1e-30
    if dtype == "bf16":
        x = t.to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16).copy()
        if kind == "nan":
            if ss == 2:
                pytest.skip("non-finite inputs are outside the reference's domain for power-of-two scales")
            x[200, 300] = 0x7FC0
    else:
        x = t.numpy().copy()
        if kind == "nan":
            pytest.skip("covered by the bf16 case")
    true_amax, _ = oracle.amax_nnz(x)
    amax_in = {"stale_small": float(true_amax) * 0.37, "stale_large": float(true_amax) * 5.0}.get(kind, float(true_amax))
    amax_in = float(np.float32(amax_in))
    oracle.clear_assert_flags()
    out, meta, _, nnz, err = oracle.block_scaling(x, 128, 128, 0.045, ss, global_amax=amax_in)
    if oracle.assert_flags():
        pytest.skip("the reference asserts on this input")
    got = H.block_scaling_delayed(x, 0.045, ss, amax_in)
    assert np.array_equal(got["out"].view(np.uint8), np.ascontiguousarray(out).view(np.uint8))
    assert int(got["meta"][0]) == meta and got["gnnz"] == nnz
    if kind == "nan":
        assert np.isnan(got["gerr"]) and np.isnan(err)
    else:
        assert np.float32(got["gerr"]).view(np.uint32) == np.float32(err).view(np.uint32)
    assert np.float32(got["gamax"]) == np.float32(true_amax)


@pytest.mark.parametrize("dtype", ["bf16", "f32"])
@pytest.mark.parametrize("ss", [1, 2, 3, 4])
@pytest.mark.parametrize("thr,want_out", [(0.045, True), (1e-6, True), (0.045, False)])
def test_block_scaling_delayed_transposed(dtype, ss, thr, want_out):
    """the single-pass operator's transposed output equals the oracle's result transposed (or the transposed
    input when the tensor stays BF16), with and without the regular output, on a non-square tensor"""
    import gpu_harness as H
    g = torch.Generator().manual_seed(ss * 11 + 3)
    t = torch.randn(384, 640, generator=g) * 3.0
    t = torch.where(torch.rand(384, 640, generator=g) < 0.1, 0.0, t)
    x = t.numpy().copy() if dtype == "f32" else oracle.bf16_bits(t.to(torch.bfloat16))
    amax, _ = oracle.amax_nnz(x)
    amax_in = float(np.float32(amax) * np.float32(0.75))
    out, meta, _, nnz, err = oracle.block_scaling(x, 128, 128, thr, ss, global_amax=amax_in)
    assert meta == (3 if thr < 1e-3 else 1)
    got = H.block_scaling_delayed_t(x, thr, ss, amax_in, want_out)
    assert np.array_equal(got["out_t"].view(np.uint8), np.ascontiguousarray(out.T).view(np.uint8)), "transposed output"
    if want_out:
        assert np.array_equal(got["out"].view(np.uint8), np.ascontiguousarray(out).view(np.uint8))
    assert int(got["meta"][0]) == meta and got["gnnz"] == nnz
    assert np.float32(got["gerr"]).view(np.uint32) == np.float32(err).view(np.uint32)
    assert np.float32(got["gamax"]) == np.float32(amax)


def test_peer_exchange_wait_runs_out():
    """A rank whose peer never shows up: the exchange kernels give up after their bounded wait, flag the
    workspace, and the ordered sum then reports meta = -1.  The absent peer is a second local buffer that
    nothing writes flags into; the limit is lowered so that the wait lasts milliseconds."""
    import ctypes
    from mor_b200 import cabi
    L = cabi.lib()
    n_err = 64
    nbytes = int(L.mor_b200_p2p_bytes(2, n_err))
    bufs, handle = [], (ctypes.c_ubyte * 64)()
    for _ in range(2):
        p = ctypes.c_void_p()
        cabi.call("mor_b200_p2p_alloc", 0, nbytes, ctypes.byref(p), handle)
        bufs.append(int(p.value))
    peers = (ctypes.c_void_p * 2)(*bufs)
    wsb = cabi.workspace_bytes(cabi.OP_AMAX_NNZ, 1, 1, 1, 1)
    ws = torch.zeros(wsb, dtype=torch.uint8, device="cuda")
    amax = torch.zeros(1, dtype=torch.float32, device="cuda")
    nnz = torch.ones(1, dtype=torch.int64, device="cuda")
    err = torch.rand(n_err, device="cuda")
    meta = torch.zeros(1, dtype=torch.int32, device="cuda")
    total = torch.zeros(1, dtype=torch.float32, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    L.mor_b200_p2p_set_wait_limit(1 << 12)
    try:
        cabi.call("mor_b200_p2p_exchange_scalars", ws.data_ptr(), bufs[0], peers, 0, 2, 1, amax.data_ptr(), nnz.data_ptr(), st)
        torch.cuda.synchronize()
        assert ws[28:32].view(torch.int32).item() == 1          # the time-out flag of the workspace head
        ws.zero_()
        cabi.call("mor_b200_p2p_exchange_errors", err.data_ptr(), n_err, bufs[0], peers, 0, 2, 1, ws.data_ptr(), st)
        torch.cuda.synchronize()
        assert ws[28:32].view(torch.int32).item() == 1
        nnz.fill_(1000)
        cabi.call("mor_b200_scaling_finalize", err.data_ptr(), n_err, 1, nnz.data_ptr(), 0.045, meta.data_ptr(),
                  total.data_ptr(), ws.data_ptr(), wsb, st)
        torch.cuda.synchronize()
        assert meta.item() == -1
    finally:
        L.mor_b200_p2p_set_wait_limit(1 << 25)
        torch.cuda.synchronize()
        for b in bufs:
            L.mor_b200_p2p_free(0, b)


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_amax_kernel_with_built_in_exchange(dtype):
    """mor_b200_scaling_amax_p2p: the last CTA of the amax kernel exchanges the slab's amax and count itself.  One GPU:
    the rank's own slot travels through its own buffer, the second rank is played by the host (its slot is written
    with a plain copy before the kernel starts, so nothing on this GPU waits for another kernel).  Shapes without a
    built-in exchange answer MOR_B200_ERR_UNSUPPORTED_SHAPE and launch nothing."""
    import ctypes
    import struct
    from mor_b200 import cabi
    L = cabi.lib()
    rt = ctypes.CDLL("libcudart.so.12")
    rt.cudaMemcpy.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int]
    rows, cols, world = 512, 768, 2
    dt = getattr(torch, dtype)
    x = (torch.randn(rows, cols, generator=torch.Generator().manual_seed(3)) * 2.0).to(dt).cuda()
    x[7, 9] = 0.0
    code = cabi.BF16 if dt == torch.bfloat16 else cabi.FP32
    wsb = cabi.workspace_bytes(cabi.OP_BLOCK_SCALING, rows, cols, 128, 128)
    n_err = 24
    nbytes = int(L.mor_b200_p2p_bytes(world, n_err))
    bufs, handle = [], (ctypes.c_ubyte * 64)()
    for _ in range(world):
        p = ctypes.c_void_p()
        cabi.call("mor_b200_p2p_alloc", 0, nbytes, ctypes.byref(p), handle)
        bufs.append(int(p.value))
    peers = (ctypes.c_void_p * world)(*bufs)
    st = torch.cuda.current_stream().cuda_stream
    amax = torch.zeros(1, dtype=torch.float32, device="cuda")
    nnz = torch.zeros(1, dtype=torch.int64, device="cuda")
    try:
        for epoch, (peer_amax, peer_nnz) in enumerate([(1.0, 10), (1000.0, 7), (0.5, 0)], start=1):
            ws = torch.zeros(wsb, dtype=torch.uint8, device="cuda")
            slot = struct.pack("<IIQI12x", int(np.float32(peer_amax).view(np.uint32)), 0, peer_nnz, epoch)
            assert rt.cudaMemcpy(bufs[0] + ((epoch & 1) * 16 + 1) * 32, slot, len(slot), 1) == 0
            cabi.call("mor_b200_scaling_amax_p2p", cabi.OP_BLOCK_SCALING, x.data_ptr(), code, rows, cols, 128, 128,
                      ws.data_ptr(), wsb, bufs[0], peers, 0, world, epoch, amax.data_ptr(), nnz.data_ptr(), st)
            torch.cuda.synchronize()
            assert ws[28:32].view(torch.int32).item() == 0, "no wait ran out"
            assert amax.item() == max(x.float().abs().max().item(), peer_amax)
            assert nnz.item() == int((x != 0).sum().item()) + peer_nnz
        ws = torch.zeros(wsb, dtype=torch.uint8, device="cuda")
        rc = L.mor_b200_scaling_amax_p2p(cabi.OP_CHANNEL_SCALING, x.data_ptr(), code, rows, cols, rows, 1, ws.data_ptr(),
                                         cabi.workspace_bytes(cabi.OP_CHANNEL_SCALING, rows, cols, rows, 1), bufs[0], peers,
                                         0, world, 4, amax.data_ptr(), nnz.data_ptr(), st)
        assert rc == cabi.ERR_UNSUPPORTED_SHAPE
    finally:
        torch.cuda.synchronize()
        for b in bufs:
            L.mor_b200_p2p_free(0, b)


def test_peer_exchange_recovers_with_new_buffers():
    """After a wait ran out (meta = -1) the documented recovery is to drop the exchange buffers and set new ones up,
    with the call counter back at 1.  The absent peer is played by the host here: no second kernel waits on this
    GPU -- the peer's slot (amax, count, epoch flag) is written with a plain copy before the exchange kernel starts."""
    import ctypes
    import struct
    from mor_b200 import cabi
    L = cabi.lib()
    rt = ctypes.CDLL("libcudart.so.12")
    rt.cudaMemcpy.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int]
    n_err, world = 64, 2
    nbytes = int(L.mor_b200_p2p_bytes(world, n_err))
    wsb = cabi.workspace_bytes(cabi.OP_AMAX_NNZ, 1, 1, 1, 1)
    st = torch.cuda.current_stream().cuda_stream
    x = torch.randn(4096, device="cuda")
    amax = torch.zeros(1, dtype=torch.float32, device="cuda")
    nnz = torch.zeros(1, dtype=torch.int64, device="cuda")

    def fresh_buffers():
        bufs, handle = [], (ctypes.c_ubyte * 64)()
        for _ in range(world):
            p = ctypes.c_void_p()
            cabi.call("mor_b200_p2p_alloc", 0, nbytes, ctypes.byref(p), handle)
            bufs.append(int(p.value))
        return bufs

    def one_call(bufs, epoch, peer_present):
        ws = torch.zeros(wsb, dtype=torch.uint8, device="cuda")
        cabi.call("mor_b200_amax_nnz", x.data_ptr(), cabi.FP32, x.numel(), amax.data_ptr(), nnz.data_ptr(), ws.data_ptr(), wsb, st)
        torch.cuda.synchronize()
        if peer_present:   # rank 1's slot in rank 0's buffer: 32 bytes at ((epoch & 1) * 16 + 1) * 32
            slot = struct.pack("<IIQI12x", int(np.float32(7.5).view(np.uint32)), 0, 1000, epoch)
            assert rt.cudaMemcpy(bufs[0] + ((epoch & 1) * 16 + 1) * 32, slot, len(slot), 1) == 0
        peers = (ctypes.c_void_p * world)(*bufs)
        cabi.call("mor_b200_p2p_exchange_scalars", ws.data_ptr(), bufs[0], peers, 0, world, epoch, amax.data_ptr(), nnz.data_ptr(), st)
        torch.cuda.synchronize()
        return ws[28:32].view(torch.int32).item(), amax.item(), nnz.item()

    L.mor_b200_p2p_set_wait_limit(1 << 12)
    bufs = fresh_buffers()
    try:
        timed_out, _, _ = one_call(bufs, 1, peer_present=False)
        assert timed_out == 1                                    # the call that would report meta = -1
        for b in bufs:
            L.mor_b200_p2p_free(0, b)
        bufs = fresh_buffers()                                   # recovery: new buffers, epoch back to 1
        for epoch in (1, 2, 3):
            timed_out, a, n = one_call(bufs, epoch, peer_present=True)
            assert timed_out == 0
            assert a == max(7.5, float(x.abs().max().item())) and n == 1000 + int((x != 0).sum().item())
    finally:
        L.mor_b200_p2p_set_wait_limit(1 << 25)
        torch.cuda.synchronize()
        for b in bufs:
            L.mor_b200_p2p_free(0, b)


def test_host_pipeline_matches_device_call():
    """HostScaling (pinned host in/out, double-buffered copies) gives the bits of the device-side call,
    call after call, with a different tensor in every call"""
    from mor_b200.sharded import HostScaling, ShardedScaling, KIND_BLOCK
    dev = torch.device("cuda", 0)
    rows, cols = 512, 1024
    host = HostScaling(rows, cols, 128, 128, torch.float32, dev, KIND_BLOCK)
    direct = ShardedScaling(rows, cols, 128, 128, torch.float32, dev, KIND_BLOCK)
    g = torch.Generator().manual_seed(77)
    xs = [torch.randn(rows, cols, generator=g) * (10.0 ** i) for i in range(5)]
    outs_h = [torch.empty(rows, cols, pin_memory=True) for _ in xs]
    scal_h = [torch.empty(2, pin_memory=True) for _ in xs]
    pinned = [x.pin_memory() for x in xs]
    for xp, oh, sh in zip(pinned, outs_h, scal_h):
        host(xp, oh, sh, 1, 0.045)
    host.synchronize()
    for x, oh, sh in zip(xs, outs_h, scal_h):
        xd = x.to(dev)
        od = torch.empty_like(xd)
        r = direct(xd, od, 1, 0.045)
        torch.cuda.synchronize()
        assert torch.equal(od.cpu().view(torch.int32), oh.view(torch.int32))
        assert sh[0].item() == r.global_amax.item() and sh[1].item() == r.global_error.item()


def test_pipelined_calls_match_plain_calls():
    """ShardedScaling(overlap=True): the post-cast chain of a call runs on a second stream under the next call's amax
    pass, with two alternating sets of scratch; a different tensor in every call (one of them falls back to BF16),
    one output buffer reused by every call"""
    from mor_b200.sharded import ShardedScaling, KIND_BLOCK
    dev = torch.device("cuda", 0)
    rows, cols = 1024, 1024
    piped = ShardedScaling(rows, cols, 128, 128, torch.float32, dev, KIND_BLOCK, overlap=True)
    plain = ShardedScaling(rows, cols, 128, 128, torch.float32, dev, KIND_BLOCK)
    g = torch.Generator().manual_seed(78)
    xs = [torch.randn(rows, cols, generator=g) * (10.0 ** i) for i in range(6)]
    xs[2] = xs[2] * 10.0 ** (torch.rand(rows, cols, generator=g) * 8 - 4)
    xd = [x.to(dev) for x in xs]
    out = torch.empty(rows, cols, device=dev)
    kept, metas = [], []
    for x in xd:
        r = piped(x, out, 1, 0.045)
        r.wait()                                           # the current stream waits; the host does not
        kept.append((out.clone(), r.meta.clone(), r.global_amax.clone(), r.global_nnz.clone(), r.global_error.clone()))
    torch.cuda.synchronize()
    for x, k in zip(xd, kept):
        o = torch.empty_like(x)
        r = plain(x, o, 1, 0.045)
        torch.cuda.synchronize()
        assert torch.equal(o.view(torch.int32), k[0].view(torch.int32))
        assert r.meta.item() == k[1].item() and r.global_nnz.item() == k[3].item()
        assert r.global_amax.item() == k[2].item() and r.global_error.item() == k[4].item()
        metas.append(r.meta.item())
    assert set(metas) == {1, 3}


def test_invalid_arguments_are_status_codes_not_faults():
    import gpu_harness as H
    from mor_b200 import cabi
    x = rand_bits(1, 64, 64)
    with pytest.raises(cabi.MorB200Error):
        H.fake_quantize(x, 32, 33, 1.0, 1, 1)          # odd block width
    with pytest.raises(cabi.MorB200Error):
        H.fake_quantize(x, 32, 32, 1.0, 1, 3)          # unknown sf_type
    with pytest.raises(cabi.MorB200Error):
        H.block_scaling(x, 32, 64, 0.045, 5)           # ss_mode out of range
    with pytest.raises(AssertionError):
        H.block_scaling(x, 16, 16, 0.045, 1)           # block shape the pipeline does not cover
    with pytest.raises(cabi.MorB200Error):
        H.e8mx(x, 4, 1)                                # quantize_type out of range
    # the context is still healthy
    assert torch.zeros(1, device="cuda").item() == 0.0
