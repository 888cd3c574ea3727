"""Callers either side of the hot path: the .bin tensor dumps of the reference's prototypes and the
linear-layer wrapper with its log line (format of train_logs/process_example_logs.py:38-72)."""
import os
import re
import struct
import sys

import numpy as np
import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def test_bin_round_trip(tmp_path):
    from mor_b200 import binio
    t = torch.randn(37, 53)
    p = str(tmp_path / "t.bin")
    binio.write_bin(p, t)
    raw = open(p, "rb").read()
    assert struct.unpack("<ii", raw[:8]) == (37, 53) and len(raw) == 8 + 4 * 37 * 53
    assert np.array_equal(np.frombuffer(raw[8:], "<f4").reshape(37, 53), t.numpy())
    assert torch.equal(binio.read_bin(p), t)
    assert binio.read_bin(p, torch.bfloat16).dtype == torch.bfloat16
    with open(p, "ab") as f:
        f.write(b"\0\0\0\0")
    with pytest.raises(ValueError):
        binio.read_bin(p)
    with pytest.raises(ValueError):
        binio.write_bin(p, torch.zeros(3))


# the patterns with which the reference's tooling takes a log line apart
PATTERNS = {
    "tensor": r"Tensor\s+([\w\.]+)\s+at\s+counter\s+(\d+)\s+step\s+(\d+)",
    "dimension": r"tensor dimension:\s+([\dx]+)",
    "non_zero": r"global_non_zero:\s+(\d+)",
    "global_error": r"global_error:\s+([\d\.]+)",
    "relative_error": r"relative_error:\s+([\d\.]+)",
    "histogram": r"histogram\s+\[([\d,\s]+)\]",
}


def parse(line):
    out = {k: re.search(p, line) for k, p in PATTERNS.items()}
    assert all(out.values()), line
    return {
        "node": int(line.split(":")[0].strip()), "name": out["tensor"].group(1), "counter": int(out["tensor"].group(2)),
        "step": int(out["tensor"].group(3)), "dim": out["dimension"].group(1), "nnz": int(out["non_zero"].group(1)),
        "err": float(out["global_error"].group(1)), "rel": float(out["relative_error"].group(1)),
        "hist": [int(v) for v in out["histogram"].group(1).split(",")],
    }


def test_log_line_is_parsed_by_the_reference_patterns():
    from mor_b200.nn import HIST_BINS, format_log_line
    line = format_log_line(3, "decoder.layers.7.mlp.fc1.weight", 12, 400, 4096, 1024, 4194000, 61234.5, list(range(HIST_BINS)))
    d = parse(line)
    assert d == {"node": 3, "name": "decoder.layers.7.mlp.fc1.weight", "counter": 12, "step": 400, "dim": "4096x1024",
                 "nnz": 4194000, "err": 61234.5, "rel": pytest.approx(61234.5 / 4194000, abs=1e-9),
                 "hist": list(range(HIST_BINS))}
    tiny = parse(format_log_line(0, "w", 0, 0, 128, 128, 16384, 1e-7, [0] * HIST_BINS))   # no exponent notation
    assert tiny["err"] == 0.0 and tiny["rel"] == pytest.approx(1e-7 / 16384, abs=1e-10)


def test_block_error_histogram_bins():
    from mor_b200.nn import HIST_BINS, block_error_histogram
    x = torch.ones(256, 256)
    out = x.clone()
    out[:128, :128] *= 1.012      # bin 2
    out[:128, 128:] *= 1.0        # bin 0
    out[128:, :128] *= 0.9        # 0.1 -> last bin
    x[128:, 128:] = 0.0           # no non-zero element: error 0 -> bin 0
    h = block_error_histogram(x, out)
    assert len(h) == HIST_BINS and sum(h) == 4
    assert h[0] == 2 and h[2] == 1 and h[HIST_BINS - 1] == 1


@pytest.mark.gpu
def test_linear_wrapper_forward_backward_and_log():
    import mor
    from mor_b200.nn import MoRLinear, QuantConfig, TensorLogger
    torch.manual_seed(0)
    lines = []
    log = TensorLogger(sink=lines.append, rank=1)
    layer = MoRLinear(512, 256, bias=True, device="cuda", input_cfg=QuantConfig("block"), weight_cfg=QuantConfig("row"),
                      grad_cfg=QuantConfig("mx"), logger=log, name="blk0.fc")
    x = torch.randn(4, 64, 512, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    y = layer(x)
    # forward = torch's linear on the fake-quantized operands
    xq = mor.ops.fake_quantize_block_scaling(x.detach().reshape(256, 512), 256, 512, 128, 128, 0.045, 1)[0]
    wq = mor.ops.fake_quantize_channel_scaling(layer.weight.detach(), 256, 512, 1, 512, 0.045, 1)[0]
    want = torch.nn.functional.linear(xq.reshape(4, 64, 512), wq, layer.bias)
    assert torch.allclose(y.float(), want.float(), rtol=1e-2, atol=1e-2)
    g = torch.randn_like(y)
    y.backward(g)
    # straight-through: gradients are those of a plain linear layer fed the quantized operands and gradient
    gq = mor.ops.fake_quantize_mx(g.reshape(256, 256), 256, 256, 32, 0, 2)[0].reshape(4, 64, 256)
    assert torch.allclose(x.grad.float(), (gq.reshape(256, 256) @ wq).reshape(4, 64, 512).float(), rtol=2e-2, atol=2e-2)
    assert torch.allclose(layer.weight.grad.float(), (gq.reshape(256, 256).t() @ xq).float(), rtol=2e-2, atol=2e-2)
    parsed = [parse(l) for l in lines]
    assert [p["name"] for p in parsed] == ["blk0.fc.input", "blk0.fc.weight"]   # the mx gradient has no tensor-level error
    assert parsed[0]["node"] == 1 and parsed[0]["dim"] == "256x512" and parsed[0]["nnz"] == int((x != 0).sum())
    assert sum(parsed[0]["hist"]) == 2 * 4 and parsed[0]["rel"] < 0.045


@pytest.mark.gpu
def test_linear_wrapper_delayed_scaling():
    """the first call seeds the amax with the two-pass form; later calls quantize in one pass with the
    amax of the call before"""
    import mor
    from mor_b200.nn import MoRLinear, QuantConfig
    torch.manual_seed(1)
    layer = MoRLinear(256, 128, bias=False, device="cuda", input_cfg=QuantConfig("block_delayed"),
                      weight_cfg=QuantConfig("none"))
    x1 = torch.randn(128, 256, device="cuda", dtype=torch.bfloat16)
    x2 = x1 * 3.0
    y1 = layer(x1)
    want1 = mor.ops.fake_quantize_block_scaling(x1, 128, 256, 128, 128, 0.045, 1)
    assert torch.equal(y1, torch.nn.functional.linear(want1[0], layer.weight))
    y2 = layer(x2)
    want2 = mor.ops.fake_quantize_block_scaling_delayed(x2, 128, 256, 128, 128, 0.045, 1, want1[2])
    assert torch.equal(y2, torch.nn.functional.linear(want2[0], layer.weight))
    assert layer._state["input"]["amax"].item() == x2.float().abs().max().item()


@pytest.mark.gpu
def test_bin_file_replays_through_the_operator(tmp_path):
    import mor
    from mor_b200 import binio
    t = torch.randn(256, 384)
    p = str(tmp_path / "capture.bin")
    binio.write_bin(p, t)
    x = binio.read_bin(p, torch.bfloat16).cuda()
    out, meta = mor.ops.fake_quantize(x, 256, 384, 128, 128, 1e-15, 1, 1)
    assert out.shape == x.shape and meta.shape == (2, 3)
