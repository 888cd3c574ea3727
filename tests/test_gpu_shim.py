"""Every operator of the reference's surface called the way the reference's users call it --
``mor.ops.<name>(cuda tensor, ...)`` through the registered torch operators -- and compared bit
for bit with the CPU oracle: the allocation paths of the shim, ``result`` aliasing the input,
in-place operators on a non-contiguous input (packed, processed, copied back), the int32 / int64
non-zero count, and one backward pass through every operator that registers a gradient.
"""
import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu

R, C = 256, 384


def bf16_input(seed, kind="normal", rows=R, cols=C):
    g = torch.Generator().manual_seed(seed)
    t = torch.randn(rows, cols, generator=g)
    if kind == "wide":
        t = t * 10.0 ** (torch.rand(rows, cols, generator=g) * 8 - 4)
    return t.to(torch.bfloat16)


def bits(t):
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().view(np.uint16)
    if t.dtype == torch.float32:
        a = t.numpy().copy()
        a[np.isnan(a)] = np.float32(np.nan)
        return a.view(np.uint32)
    return t.numpy()


def same(t, expected, what):
    a, b = bits(t).reshape(-1), np.asarray(expected).reshape(-1)
    if b.dtype == np.float32:
        b = b.copy()
        b[np.isnan(b)] = np.float32(np.nan)
        b = b.view(np.uint32)
    bad = np.nonzero(a != b)[0]
    assert bad.size == 0, f"{what}: {bad.size} of {a.size} differ, first at {bad[:6].tolist()}"


def f32_bits(v):
    return int(np.array([v], np.float32).view(np.uint32)[0])


@pytest.mark.parametrize("mode,sf,bx,by,clamp", [(1, 1, 128, 128, 1e-15), (101, 1, 128, 128, 1e-15), (1, 2, 128, 128, 1e-25),
                                                 (2, 1, 32, 64, 0.0), (3, 2, 64, 32, 0.0), (4, 1, 128, 128, 37.5),
                                                 (5, 1, 128, 128, 900.0), (9, 1, 128, 128, 0.0)])
def test_fake_quantize_and_no_alloc(mode, sf, bx, by, clamp):
    import mor
    x = bf16_input(mode, "wide" if mode in (1, 101) else "normal")
    xb = oracle.bf16_bits(x)
    exp_out, exp_meta = oracle.fake_quantize(xb, bx, by, clamp, mode, sf)
    xd = x.cuda()
    out, meta = mor.ops.fake_quantize(xd, R, C, bx, by, clamp, mode, sf)
    same(out, exp_out, f"fake_quantize mode {mode}")
    assert meta.dtype == torch.int32 and np.array_equal(meta.cpu().numpy(), exp_meta)
    same(xd, xb, "input untouched")
    # caller-owned result, then result aliasing the input (the reference's test_inplace)
    res = torch.full_like(xd, 7.0)
    meta2 = mor.ops.fake_quantize_no_alloc(xd, R, C, bx, by, clamp, mode, sf, res)
    same(res, exp_out, "no_alloc result")
    assert np.array_equal(meta2.cpu().numpy(), exp_meta)
    meta3 = mor.ops.fake_quantize_no_alloc(xd, R, C, bx, by, clamp, mode, sf, xd)
    same(xd, exp_out, "no_alloc with result = input")
    assert np.array_equal(meta3.cpu().numpy(), exp_meta)


@pytest.mark.parametrize("op,bx,by", [("block", 128, 128), ("block", 64, 64), ("channel", 1, 384), ("channel", 1, 32),
                                      ("channel", 256, 1)])
@pytest.mark.parametrize("ss", [1, 2, 3, 4])
@pytest.mark.parametrize("thr", [0.045, 1e-6])
def test_scaling_and_inplace(op, bx, by, ss, thr):
    import mor
    x = bf16_input(10 * ss + bx % 7)
    xb = oracle.bf16_bits(x)
    fn = oracle.block_scaling if op == "block" else oracle.channel_scaling
    oracle.clear_assert_flags()
    exp = fn(xb, bx, by, thr, ss)
    if oracle.assert_flags():
        pytest.skip("the reference asserts on this input")
    name = f"fake_quantize_{op}_scaling"
    xd = x.cuda()
    out, meta, gamax, gnnz, gerr = getattr(mor.ops, name)(xd, R, C, bx, by, thr, ss)
    same(out, exp[0], name)
    assert meta.dtype == torch.int32 and gnnz.dtype == torch.int32 and gamax.dtype == torch.float32
    assert meta.item() == exp[1] and gnnz.item() == exp[3]
    assert f32_bits(gamax.item()) == f32_bits(exp[2]) and f32_bits(gerr.item()) == f32_bits(exp[4])
    same(xd, xb, "input untouched")
    # in place on a NON-contiguous view: every second column of a wider tensor
    wide = torch.zeros(R, 2 * C, dtype=torch.bfloat16, device="cuda")
    wide[:, ::2] = xd
    wide[:, 1::2] = 3.0
    view = wide[:, ::2]
    assert not view.is_contiguous()
    meta, gamax, gnnz, gerr = getattr(mor.ops, name + "_inplace")(view, R, C, bx, by, thr, ss)
    same(wide[:, ::2], exp[0], name + "_inplace on a strided view")
    assert bool((wide[:, 1::2] == 3.0).all()), "the columns between were touched"
    assert meta.item() == exp[1] and gnnz.item() == exp[3] and f32_bits(gerr.item()) == f32_bits(exp[4])
    # and on a contiguous tensor
    xc = x.cuda()
    getattr(mor.ops, name + "_inplace")(xc, R, C, bx, by, thr, ss)
    same(xc, exp[0], name + "_inplace")


def test_scaling_float32_reports_int64_count():
    import mor
    g = torch.Generator().manual_seed(5)
    x = torch.randn(R, C, generator=g)
    exp = oracle.block_scaling(x.numpy(), 128, 128, 0.045, 1)
    out, meta, gamax, gnnz, gerr = mor.ops.fake_quantize_block_scaling(x.cuda(), R, C, 128, 128, 0.045, 1)
    assert gnnz.dtype == torch.int64 and gnnz.item() == exp[3]
    same(out, exp[0], "float32 block scaling")
    assert f32_bits(gerr.item()) == f32_bits(exp[4])


@pytest.mark.parametrize("qt", [1, 2, 3])
@pytest.mark.parametrize("strategy", [0, 1])
def test_e8mx_and_inplace(qt, strategy):
    import mor
    x = bf16_input(20 + qt)
    xb = oracle.bf16_bits(x)
    exp, _ = oracle.e8mx(xb, qt, strategy)
    xd = x.cuda()
    same(mor.ops.fake_quantize_e8mx(xd, R, C, 128, 128, qt, strategy), exp, f"e8m{qt}")
    res = torch.zeros_like(xd)
    assert mor.ops.fake_quantize_e8mx_inplace(xd, R, C, 128, 128, qt, strategy, res) is None
    same(res, exp, f"e8m{qt} into result")
    mor.ops.fake_quantize_e8mx_inplace(xd, R, C, 128, 128, qt, strategy, xd)
    same(xd, exp, f"e8m{qt} with result = input")


@pytest.mark.parametrize("name,fmt", [("quant_dequant_e4m3", 0), ("quant_dequant_e5m2", 1), ("quant_dequant_e3m2", 2),
                                      ("quant_dequant_e2m3", 3)])
def test_unscaled_casts(name, fmt):
    import mor
    g = torch.Generator().manual_seed(fmt)
    x = torch.randn(R, C, generator=g) * 10.0 ** (torch.rand(R, C, generator=g) * 8 - 5)
    same(getattr(mor.ops, name)(x.cuda(), R, C, 128, 128), oracle.quant_dequant(x.numpy(), fmt), name)


@pytest.mark.parametrize("rne", [True, False])
def test_e8_scale_ops(rne):
    import mor
    g = torch.Generator().manual_seed(3)
    x = torch.randn(R, C, generator=g) * 10.0 ** (torch.rand(R, C, generator=g) * 6 - 3)
    fn = mor.ops.e4m3_with_e8_scale_rne if rne else mor.ops.e4m3_with_e8_scale_rz
    same(fn(x.cuda(), R, C, 128, 128), oracle.e4m3_with_e8_scale(x.numpy(), rne), f"e8 scale rne={rne}")


def test_additional_operators():
    import mor
    x = bf16_input(31)
    xb = oracle.bf16_bits(x)
    xd = x.cuda()
    out, scales = mor.ops.fake_quantize_mx(xd, R, C, 32, 0, 2)
    eo, es = oracle.fake_quantize_group(xb, 1, 32, 0, 2, want_scales=True)
    same(out, eo, "fake_quantize_mx")
    same(scales, es, "fake_quantize_mx scales")
    payload, sb = mor.ops.quantize_mx(xd, R, C, 32, 0)
    ep, eb = oracle.quantize_mx(xb, 32, 0)
    same(payload, ep, "quantize_mx codes")
    same(sb, eb, "quantize_mx scale bytes")
    pq, sq, aq = mor.ops.quantize_scaled(xd, R, C, 128, 128, 1)
    ep, es, ea = oracle.quantize_scaled(xb, 128, 128, 1)
    same(pq, ep, "quantize_scaled codes")
    same(sq, es, "quantize_scaled scales")
    assert aq.item() == float(ea) and pq.dtype == torch.uint8 and sq.shape == (R // 128, C // 128)
    # the bytes are torch's float8_e4m3fn: dividing by the scale gives the fake-quantized tensor
    fq = mor.ops.fake_quantize_block_scaling(xd, R, C, 128, 128, 3e38, 1)[0]
    deq = pq.view(torch.float8_e4m3fn).float() / sq.repeat_interleave(128, 0).repeat_interleave(128, 1)
    assert torch.equal(deq.to(torch.bfloat16).view(torch.int16)[xd != 0], fq.view(torch.int16)[xd != 0])
    amax_in = xd.float().abs().max().reshape(1)
    o, ot, m, am, nz, er = mor.ops.fake_quantize_block_scaling_delayed_t(xd, R, C, 128, 128, 3e38, 1, amax_in)
    assert ot.shape == (C, R) and torch.equal(ot.view(torch.int16), o.t().contiguous().view(torch.int16))
    same(o, oracle.block_scaling(xb, 128, 128, 3e38, 1)[0], "delayed_t regular output")
    p6, sb6 = mor.ops.quantize_mx_fp6(xd, R, C, 32)
    c6, e6 = oracle.quantize_mx(xb, 32, 3)
    same(p6, oracle.pack_fp6(c6), "quantize_mx_fp6 payload")
    same(sb6, e6, "quantize_mx_fp6 scale bytes")


GRAD_OPS = [
    ("fake_quantize", lambda m, x: m.fake_quantize(x, R, C, 128, 128, 1e-15, 1, 1)[0]),
    ("fake_quantize_no_alloc", None),   # returns meta only: exercised through its registration below
    ("fake_quantize_block_scaling", lambda m, x: m.fake_quantize_block_scaling(x, R, C, 128, 128, 0.045, 1)[0]),
    ("fake_quantize_channel_scaling", lambda m, x: m.fake_quantize_channel_scaling(x, R, C, 1, C, 0.045, 1)[0]),
    ("fake_quantize_e8mx", lambda m, x: m.fake_quantize_e8mx(x, R, C, 128, 128, 2, 1)),
    ("fake_quantize_mx", lambda m, x: m.fake_quantize_mx(x, R, C, 32, 0, 2)[0]),
    ("fake_quantize_block_scaling_delayed",
     lambda m, x: m.fake_quantize_block_scaling_delayed(x, R, C, 128, 128, 0.045, 1, torch.ones(1, device="cuda"))[0]),
    ("fake_quantize_block_scaling_delayed_t",
     lambda m, x: m.fake_quantize_block_scaling_delayed_t(x, R, C, 128, 128, 0.045, 1, torch.ones(1, device="cuda"))[0]),
]


@pytest.mark.parametrize("name,call", [g for g in GRAD_OPS if g[1] is not None], ids=[g[0] for g in GRAD_OPS if g[1] is not None])
def test_straight_through_backward(name, call):
    import mor
    x = bf16_input(40).cuda().requires_grad_(True)
    y = call(mor.ops, x)
    w = torch.randn_like(y)
    (y * w).sum().backward()
    assert x.grad is not None and torch.equal(x.grad, w), f"{name}: the gradient must pass through unchanged"


@pytest.mark.parametrize("name", ["quant_dequant_e4m3", "quant_dequant_e5m2", "quant_dequant_e2m3", "quant_dequant_e3m2",
                                  "e4m3_with_e8_scale_rne", "e4m3_with_e8_scale_rz"])
def test_straight_through_backward_float32_ops(name):
    import mor
    x = torch.randn(R, C, device="cuda", requires_grad=True)
    y = getattr(mor.ops, name)(x, R, C, 128, 128)
    w = torch.randn_like(y)
    (torch.nan_to_num(y) * w).sum().backward()
    assert x.grad is not None and x.grad.shape == x.shape


def test_argument_errors_raise_runtime_error():
    import mor
    x = bf16_input(1).cuda()
    with pytest.raises(RuntimeError):
        mor.ops.fake_quantize(x, R, C, 128, 127, 1.0, 1, 1)                 # odd block width
    with pytest.raises(RuntimeError):
        mor.ops.fake_quantize_block_scaling(x, R, C, 128, 128, 0.045, 7)    # ss_mode out of range
    with pytest.raises(RuntimeError):
        mor.ops.fake_quantize_channel_scaling(x, R, C, 2, 2, 0.045, 1)      # neither 1 x k nor k x 1
    with pytest.raises(RuntimeError):
        mor.ops.fake_quantize(x.float().double(), R, C, 128, 128, 1.0, 1, 1)
    with pytest.raises(RuntimeError):
        mor.ops.fake_quantize_no_alloc(x, R, C, 128, 128, 1.0, 1, 1, torch.zeros(4, 4, dtype=torch.bfloat16, device="cuda"))
    assert torch.zeros(1, device="cuda").item() == 0.0
