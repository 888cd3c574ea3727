"""The five benchmark configurations on their own seeded inputs (mor_b200/workloads.py, drawn
on the CPU so that every machine sees the same bits): every operator that bench.py times on a
configuration is fed that configuration's tensor through the C ABI and compared with the CPU
oracle -- outputs, meta, amax, non-zero count and the bit pattern of the error sum.  No
tolerance.  Sizes are the full ones (the oracle needs about a second per operator); the
float32 configuration is checked on its first 1 GiB slab and on two slabs handled the way two
ranks handle them.
"""
import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu

BIG = 3e38  # a threshold no tensor exceeds: the quantized output is kept


def bits(t):
    return oracle.bf16_bits(t.contiguous())


def f32_bits(v):
    return int(np.array([v], np.float32).view(np.uint32)[0])


def same_bytes(a, b, what):
    a = np.ascontiguousarray(a).reshape(-1).view(np.uint8)
    b = np.ascontiguousarray(b).reshape(-1).view(np.uint8)
    if a.size != b.size or not np.array_equal(a, b):
        bad = np.nonzero(a != b)[0] if a.size == b.size else np.array([-1])
        raise AssertionError(f"{what}: {bad.size} of {a.size} bytes differ, first at {bad[:8].tolist()}")


def check_scaling(got, exp, what):
    out, meta, gamax, gnnz, gerr = exp
    same_bytes(got["out"], out, what)
    assert int(np.asarray(got["meta"]).reshape(-1)[0]) == meta, f"{what}: meta {got['meta']} vs {meta}"
    assert f32_bits(got["gamax"]) == f32_bits(gamax), f"{what}: amax {got['gamax']!r} vs {float(gamax)!r}"
    assert got["gnnz"] == gnnz, f"{what}: nnz {got['gnnz']} vs {gnnz}"
    assert f32_bits(got["gerr"]) == f32_bits(gerr), f"{what}: error sum {got['gerr']!r} vs {float(gerr)!r}"


@pytest.fixture(scope="module")
def c1():
    from mor_b200 import workloads
    return bits(workloads.config1())


@pytest.fixture(scope="module")
def c2():
    from mor_b200 import workloads
    return bits(workloads.config2())


@pytest.fixture(scope="module")
def c3():
    from mor_b200 import workloads
    return bits(workloads.config3())


@pytest.fixture(scope="module")
def c4():
    from mor_b200 import workloads
    return bits(workloads.config4())


# ------------------------------------------------------------------ configuration 1
def test_config1_per_tensor_scale_given(c1):
    import gpu_harness as H
    amax, _ = oracle.amax_nnz(c1)
    scale = float(np.float32(448.0) / np.float32(amax))          # binary32 division, as the cast kernels do
    exp_out, exp_meta = oracle.fake_quantize(c1, 128, 128, scale, 4, 1)
    got = H.fake_quantize(c1, 128, 128, scale, 4, 1)
    same_bytes(got["out"], exp_out, "config 1, fake_quantize mode 4")
    assert np.array_equal(got["meta"], exp_meta)


@pytest.mark.parametrize("ss", [4, 1])
@pytest.mark.parametrize("thr", [BIG, 0.045])
def test_config1_block_scaling(c1, ss, thr):
    import gpu_harness as H
    check_scaling(H.block_scaling(c1, 128, 128, thr, ss), oracle.block_scaling(c1, 128, 128, thr, ss),
                  f"config 1, block_scaling ss {ss} thr {thr}")


def test_config1_block_scaling_in_place(c1):
    import gpu_harness as H
    check_scaling(H.block_scaling(c1.copy(), 128, 128, BIG, 4, inplace=True), oracle.block_scaling(c1, 128, 128, BIG, 4),
                  "config 1, block_scaling ss 4 in place")


# ------------------------------------------------------------------ configuration 2
@pytest.mark.parametrize("mode", [2, 3])
def test_config2_per_row_single_pass(c2, mode):
    import gpu_harness as H
    rows, cols = c2.shape
    exp_out, exp_meta = oracle.fake_quantize(c2, 1, cols, 0.0, mode, 1)
    got = H.fake_quantize(c2, 1, cols, 0.0, mode, 1)
    same_bytes(got["out"], exp_out, f"config 2, fake_quantize mode {mode} 1x{cols}")
    assert np.array_equal(got["meta"], exp_meta)


@pytest.mark.parametrize("ss", [3, 1, 2])
@pytest.mark.parametrize("thr", [BIG, 0.045])
def test_config2_channel_pipeline(c2, ss, thr):
    import gpu_harness as H
    rows, cols = c2.shape
    check_scaling(H.channel_scaling(c2, 1, cols, thr, ss), oracle.channel_scaling(c2, 1, cols, thr, ss),
                  f"config 2, channel_scaling 1x{cols} ss {ss} thr {thr}")


# ------------------------------------------------------------------ configuration 3
@pytest.mark.parametrize("fmt", [oracle.FMT_E4M3, oracle.FMT_E2M3])
def test_config3_mx_groups(c3, fmt):
    import gpu_harness as H
    exp_out, exp_scales = oracle.fake_quantize_group(c3, 1, 32, fmt, oracle.SF_E8, want_scales=True)
    got = H.fake_quantize_group(c3, 32, fmt, oracle.SF_E8)
    same_bytes(got["out"], exp_out, f"config 3, fake_quantize_mx format {fmt}")
    same_bytes(got["scales"], exp_scales, f"config 3, group scales format {fmt}")


def test_config3_quantize_mx(c3):
    import gpu_harness as H
    payload, scales = oracle.quantize_mx(c3, 32, oracle.FMT_E4M3)
    got = H.quantize_mx(c3, 32, oracle.FMT_E4M3)
    same_bytes(got["payload"], payload, "config 3, quantize_mx codes")
    same_bytes(got["scales"], scales, "config 3, quantize_mx scale bytes")


@pytest.mark.parametrize("thr", [BIG, 0.045])
def test_config3_channel_pipeline_1x32(c3, thr):
    """4 194 304 groups -> 2^20 error entries: the one workload whose ordered error sum goes through the
    chained partial sums behind a real cast"""
    import gpu_harness as H
    check_scaling(H.channel_scaling(c3, 1, 32, thr, 2), oracle.channel_scaling(c3, 1, 32, thr, 2),
                  f"config 3, channel_scaling 1x32 ss 2 thr {thr}")


# ------------------------------------------------------------------ configuration 4
@pytest.mark.parametrize("mode", [1, 101])
def test_config4_mor_choice(c4, mode):
    import gpu_harness as H
    exp_out, exp_meta = oracle.fake_quantize(c4, 128, 128, 1e-15, mode, 1)
    got = H.fake_quantize(c4, 128, 128, 1e-15, mode, 1)
    same_bytes(got["out"], exp_out, f"config 4, MoR mode {mode}")
    assert np.array_equal(got["meta"], exp_meta)
    kinds = set(np.unique(exp_meta).tolist())
    assert {1, 3} <= kinds and (mode == 1 or 2 in kinds), f"representations chosen: {sorted(kinds)}"


def test_config4_blocks_that_lose_the_error_comparison():
    """sign * 10^U(-3, 4) blocks: range admits E4M3/E5M2 but the E4M3 error sum exceeds the E5M2 one, so the
    relative-error criterion keeps BF16 (a branch configuration 4 itself never takes); mixed with the
    configuration's three kinds so that every outcome sits in one tensor"""
    import gpu_harness as H
    from mor_b200 import workloads
    g = torch.Generator().manual_seed(3003)
    base = workloads.config4(scale=8).float()                       # 4096 x 1024, all three kinds
    rows, cols = base.shape
    lose = torch.where(torch.rand(rows, cols, generator=g) < 0.5, -1.0, 1.0) * 10.0 ** (torch.rand(rows, cols, generator=g) * 7.0 - 3.0)
    bi = torch.arange(rows)[:, None] // 128
    bj = torch.arange(cols)[None, :] // 128
    x = bits(torch.where((bi + bj) % 4 == 3, lose, base).to(torch.bfloat16))
    exp_out, exp_meta = oracle.fake_quantize(x, 128, 128, 1e-15, 1, 1)
    # the losing blocks are BF16 by comparison, not by range: in dynamic-range mode the same blocks are E5M2
    _, dyn_meta = oracle.fake_quantize(x, 128, 128, 1e-15, 101, 1)
    lost = (exp_meta == 3) & ((dyn_meta == 2) | (dyn_meta == 12))
    assert lost.sum() >= 32, "the input does not exercise the comparison-loses branch"
    got = H.fake_quantize(x, 128, 128, 1e-15, 1, 1)
    same_bytes(got["out"], exp_out, "MoR mode 1 with blocks that lose the comparison")
    assert np.array_equal(got["meta"], exp_meta)


@pytest.mark.parametrize("thr", [BIG, 0.045])
def test_config4_block_scaling_pipeline(c4, thr):
    import gpu_harness as H
    check_scaling(H.block_scaling(c4, 128, 128, thr, 1), oracle.block_scaling(c4, 128, 128, thr, 1),
                  f"config 4, block_scaling ss 1 thr {thr}")


def test_config4_block_scaling_delayed(c4):
    import gpu_harness as H
    amax, _ = oracle.amax_nnz(c4)
    stale = float(np.float32(amax) * np.float32(0.5))
    out, meta, _, nnz, err = oracle.block_scaling(c4, 128, 128, BIG, 1, global_amax=stale)
    got = H.block_scaling_delayed(c4, BIG, 1, stale)
    same_bytes(got["out"], out, "config 4, delayed block scaling")
    assert int(got["meta"][0]) == meta and got["gnnz"] == nnz and f32_bits(got["gerr"]) == f32_bits(err)
    assert f32_bits(got["gamax"]) == f32_bits(amax)


def test_config4_quantize_scaled_round_trip(c4):
    """real quantized form at full size: decode(code) / scale equals the fake-quantized tensor"""
    import gpu_harness as H
    got = H.quantize_scaled(c4, 128, 128, 1)
    payload, scales, gamax = oracle.quantize_scaled(c4, 128, 128, 1)
    same_bytes(got["payload"], payload, "config 4, quantize_scaled codes")
    same_bytes(got["scales"], scales, "config 4, quantize_scaled scales")
    fq = H.block_scaling(c4, 128, 128, BIG, 1)
    same_bytes(oracle.dequantize_scaled(got["payload"], got["scales"], 128, 128), fq["out"], "config 4, decode / scale")


def test_config2_quantize_scaled_per_row(c2):
    import gpu_harness as H
    rows, cols = c2.shape
    got = H.quantize_scaled(c2, 1, cols, 3)
    payload, scales, _ = oracle.quantize_scaled(c2, 1, cols, 3)
    same_bytes(got["payload"], payload, "config 2, per-row codes")
    same_bytes(got["scales"], scales, "config 2, per-row scales")


# ------------------------------------------------------------------ configuration 5
@pytest.mark.parametrize("ss", [1, 4])
def test_config5_first_slab(ss):
    import gpu_harness as H
    from mor_b200 import workloads
    x = workloads.config5_slab(0).numpy()
    check_scaling(H.block_scaling(x, 128, 128, 0.045, ss), oracle.block_scaling(x, 128, 128, 0.045, ss),
                  f"config 5 slab 0, block_scaling ss {ss}")


@pytest.mark.parametrize("ss", [1, 4])
def test_config5_two_slabs_as_two_ranks(ss):
    """Slabs 0 and 1 (a quarter of their columns, to bound the run time) handled as two ranks handle them: amax per
    slab, the larger one given to both casts, the error sums gathered in row order and summed once -- equal
    to the oracle on the two slabs stacked."""
    from mor_b200 import cabi, workloads
    import gpu_harness as H
    slabs = [np.ascontiguousarray(workloads.config5_slab(s).numpy()[:, :4096]) for s in (0, 1)]
    rows, cols = slabs[0].shape
    whole = np.concatenate(slabs, axis=0)
    exp_out, exp_meta, exp_amax, exp_nnz, exp_err = oracle.block_scaling(whole, 128, 128, 0.045, ss)
    wsb = cabi.workspace_bytes(cabi.OP_BLOCK_SCALING, rows, cols, 128, 128)
    n_err = int(cabi.lib().mor_b200_scaling_num_errors(cabi.OP_BLOCK_SCALING, rows, cols, 128, 128))
    st = H.stream()
    dev = [H.to_dev(s) for s in slabs]
    outs = [torch.empty_like(d) for d in dev]
    wss = [torch.empty(wsb, dtype=torch.uint8, device="cuda") for _ in dev]
    amax = [torch.zeros(1, dtype=torch.float32, device="cuda") for _ in dev]
    nnz = [torch.zeros(1, dtype=torch.int64, device="cuda") for _ in dev]
    for d, w, a, n in zip(dev, wss, amax, nnz):
        cabi.call("mor_b200_scaling_amax", cabi.OP_BLOCK_SCALING, d.data_ptr(), cabi.FP32, rows, cols, 128, 128,
                  a.data_ptr(), n.data_ptr(), w.data_ptr(), wsb, st)
    gamax = torch.maximum(amax[0], amax[1])
    gnnz = nnz[0] + nnz[1]
    all_err = torch.zeros(2 * n_err, dtype=torch.float32, device="cuda")
    for r, (d, o, w) in enumerate(zip(dev, outs, wss)):
        cabi.call("mor_b200_scaling_cast", cabi.OP_BLOCK_SCALING, d.data_ptr(), o.data_ptr(), cabi.FP32, rows, cols,
                  128, 128, ss, gamax.data_ptr(), all_err[r * n_err:].data_ptr(), w.data_ptr(), wsb, st)
    meta = torch.zeros(1, dtype=torch.int32, device="cuda")
    gerr = torch.zeros(1, dtype=torch.float32, device="cuda")
    cabi.call("mor_b200_scaling_finalize", all_err.data_ptr(), 2 * n_err, 1, gnnz.data_ptr(), 0.045, meta.data_ptr(),
              gerr.data_ptr(), wss[0].data_ptr(), wsb, st)
    for d, o in zip(dev, outs):
        cabi.call("mor_b200_scaling_fallback", d.data_ptr(), o.data_ptr(), d.numel() * 4, meta.data_ptr(), st)
    torch.cuda.synchronize()
    got = {"out": np.concatenate([H.to_np(o) for o in outs], axis=0), "meta": H.to_np(meta), "gamax": gamax.item(),
           "gnnz": int(gnnz.item()), "gerr": gerr.item()}
    check_scaling(got, (exp_out, exp_meta, exp_amax, exp_nnz, exp_err), f"config 5, two slabs as two ranks, ss {ss}")
