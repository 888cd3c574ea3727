"""Replays a golden case (see cases.py) through the CPU oracle."""
from __future__ import annotations

import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
import oracle  # noqa: E402

_FMT = {"quant_dequant_e4m3": oracle.FMT_E4M3, "quant_dequant_e5m2": oracle.FMT_E5M2,
        "quant_dequant_e3m2": oracle.FMT_E3M2, "quant_dequant_e2m3": oracle.FMT_E2M3}


def run_oracle(op: str, x: np.ndarray, kw: dict) -> dict:
    if op == "fake_quantize":
        out, meta = oracle.fake_quantize(x, kw["block_x"], kw["block_y"], kw["clamp_threshold"], kw["mode"], kw["sf_type"])
        return {"out": out, "meta": meta}
    if op == "fake_quantize_block_scaling":
        out, meta, gamax, gnnz, gerr = oracle.block_scaling(x, kw["block_x"], kw["block_y"], kw["e4m3_threshold"], kw["ss_mode"])
        return {"out": out, "meta": np.array([meta], np.int32), "gamax": gamax, "gnnz": gnnz, "gerr": gerr}
    if op == "fake_quantize_channel_scaling":
        out, meta, gamax, gnnz, gerr = oracle.channel_scaling(x, kw["block_x"], kw["block_y"], kw["e4m3_threshold"], kw["ss_mode"])
        return {"out": out, "meta": np.array([meta], np.int32), "gamax": gamax, "gnnz": gnnz, "gerr": gerr}
    if op == "fake_quantize_e8mx":
        out, _ = oracle.e8mx(x, kw["quantize_type"], kw["scaling_strategy"])
        return {"out": out}
    if op in _FMT:
        return {"out": oracle.quant_dequant(x, _FMT[op]).reshape(x.shape)}
    if op == "e4m3_with_e8_scale_rne":
        return {"out": oracle.e4m3_with_e8_scale(x, True).reshape(x.shape)}
    if op == "e4m3_with_e8_scale_rz":
        return {"out": oracle.e4m3_with_e8_scale(x, False).reshape(x.shape)}
    raise ValueError(op)
