"""Calls the C ABI of libmor_b200 (through mor_b200.cabi / ctypes) on numpy inputs.

Device memory and the stream come from torch; the operators themselves are reached
exactly as a non-PyTorch host would reach them: raw pointers, sizes, a workspace.
"""
from __future__ import annotations

import numpy as np
import torch

from mor_b200 import cabi


def to_dev(a: np.ndarray) -> torch.Tensor:
    a = np.ascontiguousarray(a)
    if a.dtype == np.uint16:
        return torch.from_numpy(a.view(np.int16)).view(torch.bfloat16).cuda()
    return torch.from_numpy(a).cuda()


def to_np(t: torch.Tensor) -> np.ndarray:
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().view(np.uint16)
    return t.numpy()


def stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def dtype_of(a: np.ndarray) -> int:
    return cabi.FP32 if a.dtype == np.float32 else cabi.BF16


def meta_shape(rows, cols, bx, by):
    return ((rows - 1) // bx + 1, (cols // 2 - 1) // (by // 2) + 1)


def fake_quantize(x, bx, by, clamp, mode, sf, inplace=False):
    rows, cols = x.shape
    d = to_dev(x)
    out = d if inplace else torch.empty_like(d)
    meta = torch.full(meta_shape(rows, cols, bx, by), -1, dtype=torch.int32, device="cuda")
    cabi.call("mor_b200_fake_quantize", d.data_ptr(), out.data_ptr(), meta.data_ptr(), dtype_of(x), rows, cols,
              bx, by, float(clamp), mode, sf, stream())
    torch.cuda.synchronize()
    return {"out": to_np(out), "meta": to_np(meta)}


def _scaling(fn_name, op, x, bx, by, thr, ss, inplace=False):
    rows, cols = x.shape
    d = to_dev(x)
    out = d if inplace else torch.empty_like(d)
    wsb = cabi.workspace_bytes(op, rows, cols, bx, by)
    assert wsb > 0, "unsupported shape"
    ws = torch.empty(wsb, dtype=torch.uint8, device="cuda")
    f32 = x.dtype == np.float32
    meta = torch.zeros(1, dtype=torch.int32, device="cuda")
    gamax = torch.zeros(1, dtype=torch.float32, device="cuda")
    gnnz = torch.zeros(1, dtype=torch.int64 if f32 else torch.int32, device="cuda")
    gerr = torch.zeros(1, dtype=torch.float32, device="cuda")
    cabi.call(fn_name, d.data_ptr(), out.data_ptr(), dtype_of(x), rows, cols, bx, by, float(thr), ss,
              meta.data_ptr(), gamax.data_ptr(), gnnz.data_ptr(), 1 if f32 else 0, gerr.data_ptr(), ws.data_ptr(),
              wsb, stream())
    torch.cuda.synchronize()
    return {"out": to_np(out), "meta": to_np(meta), "gamax": gamax.item(), "gnnz": int(gnnz.item()),
            "gerr": gerr.item()}


def block_scaling(x, bx, by, thr, ss, inplace=False):
    return _scaling("mor_b200_block_scaling", cabi.OP_BLOCK_SCALING, x, bx, by, thr, ss, inplace)


def channel_scaling(x, bx, by, thr, ss, inplace=False):
    return _scaling("mor_b200_channel_scaling", cabi.OP_CHANNEL_SCALING, x, bx, by, thr, ss, inplace)


def e8mx(x, qtype, strategy, inplace=False):
    rows, cols = x.shape
    d = to_dev(x)
    out = d if inplace else torch.empty_like(d)
    wsb = cabi.workspace_bytes(cabi.OP_E8MX, rows, cols, 0, 0)
    ws = torch.empty(wsb, dtype=torch.uint8, device="cuda")
    cabi.call("mor_b200_e8mx", d.data_ptr(), out.data_ptr(), rows, cols, qtype, strategy, ws.data_ptr(), wsb, stream())
    torch.cuda.synchronize()
    return {"out": to_np(out)}


def quant_dequant(x, fmt):
    rows, cols = x.shape
    d = to_dev(x)
    out = torch.empty_like(d)
    cabi.call("mor_b200_quant_dequant", d.data_ptr(), out.data_ptr(), rows, cols, fmt, stream())
    torch.cuda.synchronize()
    return {"out": to_np(out)}


def e4m3_with_e8_scale(x, rne):
    rows, cols = x.shape
    d = to_dev(x)
    out = torch.empty_like(d)
    cabi.call("mor_b200_e4m3_with_e8_scale", d.data_ptr(), out.data_ptr(), rows, cols, int(rne), stream())
    torch.cuda.synchronize()
    return {"out": to_np(out)}


def fake_quantize_group(x, by, fmt, sf, want_scales=True):
    rows, cols = x.shape
    d = to_dev(x)
    out = torch.empty_like(d)
    scales = torch.zeros(rows * (cols // by), dtype=torch.float32, device="cuda") if want_scales else None
    cabi.call("mor_b200_fake_quantize_group", d.data_ptr(), out.data_ptr(), scales.data_ptr() if want_scales else None,
              dtype_of(x), rows, cols, by, fmt, sf, stream())
    torch.cuda.synchronize()
    return {"out": to_np(out), "scales": to_np(scales) if want_scales else None}


def block_scaling_delayed(x, thr, ss, amax_in):
    rows, cols = x.shape
    d = to_dev(x)
    out = torch.empty_like(d)
    wsb = cabi.workspace_bytes(cabi.OP_BLOCK_SCALING, rows, cols, 128, 128)
    ws = torch.empty(wsb, dtype=torch.uint8, device="cuda")
    f32 = x.dtype == np.float32
    meta = torch.zeros(1, dtype=torch.int32, device="cuda")
    gamax = torch.zeros(1, dtype=torch.float32, device="cuda")
    gerr = torch.zeros(1, dtype=torch.float32, device="cuda")
    gnnz = torch.zeros(1, dtype=torch.int64 if f32 else torch.int32, device="cuda")
    ain = torch.tensor([amax_in], dtype=torch.float32, device="cuda")
    cabi.call("mor_b200_block_scaling_delayed", d.data_ptr(), out.data_ptr(), dtype_of(x), rows, cols, 128, 128, float(thr),
              ss, ain.data_ptr(), meta.data_ptr(), gamax.data_ptr(), gnnz.data_ptr(), 1 if f32 else 0, gerr.data_ptr(),
              ws.data_ptr(), wsb, stream())
    torch.cuda.synchronize()
    return {"out": to_np(out), "meta": to_np(meta), "gamax": float(gamax.item()), "gnnz": int(gnnz.item()),
            "gerr": float(gerr.item())}


def block_scaling_delayed_t(x, thr, ss, amax_in, want_out=True):
    rows, cols = x.shape
    d = to_dev(x)
    out = torch.empty_like(d) if want_out else None
    out_t = torch.empty(cols, rows, dtype=d.dtype, device="cuda")
    wsb = cabi.workspace_bytes(cabi.OP_BLOCK_SCALING, rows, cols, 128, 128)
    ws = torch.empty(wsb, dtype=torch.uint8, device="cuda")
    f32 = x.dtype == np.float32
    meta = torch.zeros(1, dtype=torch.int32, device="cuda")
    gamax = torch.zeros(1, dtype=torch.float32, device="cuda")
    gerr = torch.zeros(1, dtype=torch.float32, device="cuda")
    gnnz = torch.zeros(1, dtype=torch.int64 if f32 else torch.int32, device="cuda")
    ain = torch.tensor([amax_in], dtype=torch.float32, device="cuda")
    cabi.call("mor_b200_block_scaling_delayed_t", d.data_ptr(), out.data_ptr() if want_out else None, out_t.data_ptr(),
              dtype_of(x), rows, cols, 128, 128, float(thr), ss, ain.data_ptr(), meta.data_ptr(), gamax.data_ptr(),
              gnnz.data_ptr(), 1 if f32 else 0, gerr.data_ptr(), ws.data_ptr(), wsb, stream())
    torch.cuda.synchronize()
    return {"out": to_np(out) if want_out else None, "out_t": to_np(out_t), "meta": to_np(meta), "gamax": float(gamax.item()),
            "gnnz": int(gnnz.item()), "gerr": float(gerr.item())}


def quantize_mx(x, by, fmt):
    rows, cols = x.shape
    d = to_dev(x)
    payload = torch.zeros(rows, cols, dtype=torch.uint8, device="cuda")
    scales = torch.zeros(rows, cols // by, dtype=torch.uint8, device="cuda")
    cabi.call("mor_b200_quantize_mx", d.data_ptr(), payload.data_ptr(), scales.data_ptr(), rows, cols, by, fmt, stream())
    torch.cuda.synchronize()
    return {"payload": payload.cpu().numpy(), "scales": scales.cpu().numpy()}


def quantize_mx_fp6(x, by):
    rows, cols = x.shape
    d = to_dev(x)
    payload = torch.zeros(rows, cols * 3 // 4, dtype=torch.uint8, device="cuda")
    scales = torch.zeros(rows, cols // by, dtype=torch.uint8, device="cuda")
    cabi.call("mor_b200_quantize_mx_fp6", d.data_ptr(), payload.data_ptr(), scales.data_ptr(), rows, cols, by, stream())
    torch.cuda.synchronize()
    return {"payload": payload.cpu().numpy(), "scales": scales.cpu().numpy()}


def quantize_scaled(x, bx, by, ss, amax_in=None):
    rows, cols = x.shape
    d = to_dev(x)
    op = cabi.OP_CHANNEL_SCALING if (bx == 1 or by == 1) else cabi.OP_BLOCK_SCALING
    wsb = cabi.workspace_bytes(op, rows, cols, bx, by)
    assert wsb > 0, "unsupported shape"
    ws = torch.empty(wsb, dtype=torch.uint8, device="cuda")
    payload = torch.zeros(rows, cols, dtype=torch.uint8, device="cuda")
    scales = torch.zeros(rows // bx, cols // by, dtype=torch.float32, device="cuda")
    gamax = torch.zeros(1, dtype=torch.float32, device="cuda")
    ain = None if amax_in is None else torch.tensor([amax_in], dtype=torch.float32, device="cuda")
    cabi.call("mor_b200_quantize_scaled", d.data_ptr(), payload.data_ptr(), scales.data_ptr(), dtype_of(x), rows, cols, bx, by,
              ss, None if ain is None else ain.data_ptr(), gamax.data_ptr(), ws.data_ptr(), wsb, stream())
    torch.cuda.synchronize()
    return {"payload": payload.cpu().numpy(), "scales": scales.cpu().numpy(), "gamax": float(gamax.item())}


_FMT = {"quant_dequant_e4m3": cabi.E4M3, "quant_dequant_e5m2": cabi.E5M2, "quant_dequant_e3m2": cabi.E3M2,
        "quant_dequant_e2m3": cabi.E2M3}


def run_case(op: str, x: np.ndarray, kw: dict) -> dict:
    """Runs a golden case (tests/golden/cases.py) through the C ABI."""
    if op == "fake_quantize":
        return fake_quantize(x, kw["block_x"], kw["block_y"], kw["clamp_threshold"], kw["mode"], kw["sf_type"])
    if op == "fake_quantize_block_scaling":
        return block_scaling(x, kw["block_x"], kw["block_y"], kw["e4m3_threshold"], kw["ss_mode"])
    if op == "fake_quantize_channel_scaling":
        return channel_scaling(x, kw["block_x"], kw["block_y"], kw["e4m3_threshold"], kw["ss_mode"])
    if op == "fake_quantize_e8mx":
        return e8mx(x, kw["quantize_type"], kw["scaling_strategy"])
    if op in _FMT:
        return quant_dequant(x, _FMT[op])
    if op == "e4m3_with_e8_scale_rne":
        return e4m3_with_e8_scale(x, True)
    if op == "e4m3_with_e8_scale_rz":
        return e4m3_with_e8_scale(x, False)
    raise ValueError(op)
