"""Training-loop callers of the fake-quantization operators.

``MoRLinear`` applies the operators to the input, the weight and (optionally) the incoming
gradient of a linear layer, with the straight-through gradients that ``mor_b200.ops``
registers (mor/ops.py:15-156 of the reference), and can emit one log line per quantized
tensor in the format that the reference's log tooling parses
(train_logs/process_example_logs.py:38-72):

    <rank>: Tensor <name> at counter <c> step <s> tensor dimension: <R>x<C>
    global_non_zero: <n> global_error: <e> relative_error: <e / n> histogram [h0, ..., h12]

The histogram counts 128 x 128 blocks by their mean relative error in bins of 0.005 (the
tooling labels bin i with (i + 1) * 0.005 and uses the first twelve); the last bin
collects everything from 0.060 up.  The numbers in the line come from the operator itself
(``global_nnz``, ``global_error``); the histogram is computed from input and output with
ordinary tensor operations and is a logging aid, not part of the bit-exact path.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, List, Optional

import torch
from torch import Tensor

from . import ops

HIST_BINS = 13
HIST_WIDTH = 0.005


@dataclass
class QuantConfig:
    """``kind``: "block" (block scaling, global-mantissa scale by default), "block_delayed" (the same in one
    pass over the tensor, with the tensor amax of the previous call: delayed scaling), "row" (one scale per
    row), "mx" (1 x 32 groups, E8M0 scale, single pass), "mor" (per-block format choice), "none"."""
    kind: str = "block"
    block_rows: int = 128
    block_cols: int = 128
    ss_mode: int = 1
    threshold: float = 0.045
    elem_format: int = 0          # mx: 0 E4M3, 1 E5M2, 3 E2M3
    mor_mode: int = 1             # mor: 1 relative-error criterion, 101 dynamic range
    clamp_threshold: float = 1e-15


@dataclass
class QuantStats:
    meta: Optional[Tensor] = None
    global_amax: Optional[Tensor] = None
    global_nnz: Optional[Tensor] = None
    global_error: Optional[Tensor] = None


def fake_quantize_tensor(t: Tensor, cfg: QuantConfig, state: Optional[dict] = None):
    """Fake-quantizes a tensor of any rank >= 1 (viewed as ``[-1, last]``); returns ``(out, QuantStats)``.
    ``state`` carries the amax from call to call for the "block_delayed" kind (first call: two passes)."""
    if cfg.kind == "none":
        return t, QuantStats()
    x = t.reshape(-1, t.shape[-1])
    if not x.is_contiguous():
        x = x.contiguous()
    r, c = x.shape
    if cfg.kind == "block":
        out, meta, amax, nnz, err = ops.fake_quantize_block_scaling(x, r, c, cfg.block_rows, cfg.block_cols,
                                                                    cfg.threshold, cfg.ss_mode)
        st = QuantStats(meta, amax, nnz, err)
    elif cfg.kind == "block_delayed":
        prev = None if state is None else state.get("amax")
        if prev is None:   # nothing to go by yet: the two-pass form, whose amax seeds the next call
            out, meta, amax, nnz, err = ops.fake_quantize_block_scaling(x, r, c, 128, 128, cfg.threshold, cfg.ss_mode)
        else:
            out, meta, amax, nnz, err = ops.fake_quantize_block_scaling_delayed(x, r, c, 128, 128, cfg.threshold,
                                                                                cfg.ss_mode, prev)
        if state is not None:
            state["amax"] = amax.detach()
        st = QuantStats(meta, amax, nnz, err)
    elif cfg.kind == "row":
        out, meta, amax, nnz, err = ops.fake_quantize_channel_scaling(x, r, c, 1, c, cfg.threshold, cfg.ss_mode)
        st = QuantStats(meta, amax, nnz, err)
    elif cfg.kind == "mx":
        out, _ = ops.fake_quantize_mx(x, r, c, 32, cfg.elem_format, 2)
        st = QuantStats()
    elif cfg.kind == "mor":
        out, meta = ops.fake_quantize(x, r, c, cfg.block_rows, cfg.block_cols, cfg.clamp_threshold, cfg.mor_mode, 1)
        st = QuantStats(meta=meta)
    else:
        raise ValueError(f"unknown quantization kind {cfg.kind!r}")
    return out.reshape(t.shape), st


def block_error_histogram(x: Tensor, out: Tensor, block_rows: int = 128, block_cols: int = 128) -> List[int]:
    """Counts blocks by mean relative error |(out - x) / x| over their non-zero elements, bins of 0.005."""
    x2 = x.reshape(-1, x.shape[-1]).float()
    o2 = out.reshape(-1, out.shape[-1]).float()
    r, c = x2.shape
    br, bc = min(block_rows, r), min(block_cols, c)
    r2, c2 = (r // br) * br, (c // bc) * bc
    x2, o2 = x2[:r2, :c2], o2[:r2, :c2]
    nz = x2 != 0
    rel = torch.where(nz, ((o2 - x2) / torch.where(nz, x2, torch.ones_like(x2))).abs(), torch.zeros_like(x2))
    blocks = lambda a: a.reshape(r2 // br, br, c2 // bc, bc).sum(dim=(1, 3))  # noqa: E731
    mean = blocks(rel) / blocks(nz.float()).clamp(min=1.0)
    idx = (mean / HIST_WIDTH).floor().clamp(0, HIST_BINS - 1).long().flatten()
    return torch.bincount(idx, minlength=HIST_BINS).tolist()


def format_log_line(rank: int, name: str, counter: int, step: int, rows: int, cols: int, global_nnz: int,
                    global_error: float, histogram: List[int]) -> str:
    """One line in the format parsed by train_logs/process_example_logs.py:38-72 (plain decimals only)."""
    rel = global_error / global_nnz if global_nnz else 0.0
    return (f"{rank}: Tensor {name} at counter {counter} step {step} tensor dimension: {rows}x{cols} "
            f"global_non_zero: {global_nnz} global_error: {global_error:.6f} relative_error: {rel:.10f} "
            f"histogram [{', '.join(str(int(h)) for h in histogram)}]")


class TensorLogger:
    """Collects log lines; ``sink`` receives each line (``print`` by default).  Logging synchronises the
    stream (it reads scalars back), so enable it for the steps you want to look at, not for every step."""

    def __init__(self, sink: Callable[[str], None] = print, rank: int = 0, every: int = 1):
        self.sink, self.rank, self.every = sink, rank, max(1, every)
        self.step = 0
        self.counter = 0

    def wants(self) -> bool:
        return self.step % self.every == 0

    def log(self, name: str, x: Tensor, out: Tensor, st: QuantStats, cfg: QuantConfig) -> Optional[str]:
        if st.global_nnz is None or not self.wants():
            return None
        x2 = x.reshape(-1, x.shape[-1])
        line = format_log_line(self.rank, name, self.counter, self.step, x2.shape[0], x2.shape[1],
                               int(st.global_nnz.item()), float(st.global_error.item()),
                               block_error_histogram(x, out, cfg.block_rows, cfg.block_cols))
        self.counter += 1
        self.sink(line)
        return line


class _QuantizeGrad(torch.autograd.Function):
    """Identity in the forward pass; fake-quantizes the gradient that flows back."""

    @staticmethod
    def forward(ctx, x: Tensor, layer: "MoRLinear") -> Tensor:
        ctx.layer = layer
        return x.view_as(x)

    @staticmethod
    def backward(ctx, grad: Tensor):
        layer = ctx.layer
        g = grad.contiguous()
        gq, st = fake_quantize_tensor(g, layer.grad_cfg, layer._state["grad"])
        if layer.logger is not None:
            layer.logger.log(f"{layer.log_name}.grad_output", g, gq, st, layer.grad_cfg)
        return gq, None


class MoRLinear(torch.nn.Linear):
    """``torch.nn.Linear`` whose input, weight and (optionally) output gradient are fake-quantized.

    Tensors must be CUDA bfloat16 (float32 is accepted by the block and row kinds) with dimensions that the
    chosen block shape divides; the matrix product itself is torch's."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True, device=None, dtype=torch.bfloat16,
                 input_cfg: Optional[QuantConfig] = None, weight_cfg: Optional[QuantConfig] = None,
                 grad_cfg: Optional[QuantConfig] = None, logger: Optional[TensorLogger] = None, name: str = "linear"):
        super().__init__(in_features, out_features, bias=bias, device=device, dtype=dtype)
        self.input_cfg = input_cfg or QuantConfig()
        self.weight_cfg = weight_cfg or QuantConfig()
        self.grad_cfg = grad_cfg or QuantConfig(kind="none")
        self.logger = logger
        self.log_name = name
        self._state = {"input": {}, "weight": {}, "grad": {}}   # amax carried between calls (delayed scaling)

    def forward(self, x: Tensor) -> Tensor:
        xq, sx = fake_quantize_tensor(x, self.input_cfg, self._state["input"])
        wq, sw = fake_quantize_tensor(self.weight, self.weight_cfg, self._state["weight"])
        if self.logger is not None:
            self.logger.log(f"{self.log_name}.input", x, xq, sx, self.input_cfg)
            self.logger.log(f"{self.log_name}.weight", self.weight, wq, sw, self.weight_cfg)
        y = torch.nn.functional.linear(xq, wq, self.bias)
        if self.grad_cfg.kind != "none" and torch.is_grad_enabled():
            y = _QuantizeGrad.apply(y, self)
        return y
