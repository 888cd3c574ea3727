"""Record golden vectors from the UNMODIFIED reference extension on a CUDA GPU.

    oracle/build_ref.sh                      # builds oracle/_ref/mor_ref_C.so (needs the reference sources)
    python tests/golden/make_gpu_golden.py [--out-dir DIR]   # on a machine with a GPU

Loads ``oracle/_ref/mor_ref_C.so`` -- the reference's two translation units compiled
as they are -- in this process only (it registers ``torch.ops.mor.*``, so the
repository's own extension must not be imported here), runs every case of
``cases.py`` through the reference operators, and writes

    tests/golden/reference_b200.json   per case: sha256 of the output bits, the meta
                                       matrix and the scalar outputs (as bit patterns)
    <out-dir>/golden_report.txt            case-by-case comparison with the CPU oracle

Before a case runs on the GPU the CPU oracle evaluates it: a case on which a
device-side assert() of the reference would fire (the reference is built with asserts
on) is skipped and listed, never launched.
"""
from __future__ import annotations

import json
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, HERE)

import oracle  # noqa: E402
from cases import cases, digest  # noqa: E402
from replay import run_oracle  # noqa: E402


def to_dev(a: np.ndarray) -> torch.Tensor:
    if a.dtype == np.uint16:
        return torch.from_numpy(a.view(np.int16)).view(torch.bfloat16).cuda()
    return torch.from_numpy(a).cuda()


def to_np(t: torch.Tensor) -> np.ndarray:
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().view(np.uint16)
    return t.numpy()


def f32_bits(v) -> int:
    return int(np.array([v], np.float32).view(np.uint32)[0])


def run_reference(op: str, x: np.ndarray, kw: dict) -> dict:
    rows, cols = x.shape
    fn = getattr(torch.ops.mor, op).default
    d = to_dev(x)
    if op == "fake_quantize":
        out, meta = fn(d, rows, cols, kw["block_x"], kw["block_y"], kw["clamp_threshold"], kw["mode"], kw["sf_type"])
        return {"out": to_np(out), "meta": to_np(meta)}
    if op in ("fake_quantize_block_scaling", "fake_quantize_channel_scaling"):
        out, meta, gamax, gnnz, gerr = fn(d, rows, cols, kw["block_x"], kw["block_y"], kw["e4m3_threshold"], kw["ss_mode"])
        return {"out": to_np(out), "meta": to_np(meta), "gamax": float(gamax.item()), "gnnz": int(gnnz.item()),
                "gerr": float(gerr.item())}
    if op == "fake_quantize_e8mx":
        out = fn(d, rows, cols, kw["block_x"], kw["block_y"], kw["quantize_type"], kw["scaling_strategy"])
        return {"out": to_np(out)}
    out = fn(d, rows, cols, kw["block_x"], kw["block_y"])
    return {"out": to_np(out)}


def canon(out: np.ndarray) -> np.ndarray:
    """float32 outputs: NaNs compare by position only (payloads differ between host and device)."""
    if out.dtype == np.float32:
        o = out.copy()
        o[np.isnan(o)] = np.float32(np.nan)
        return o.view(np.uint32)
    return out


def main() -> int:
    import argparse
    ap = argparse.ArgumentParser()
    ap.add_argument("--out-dir", default=os.path.join(ROOT, "golden_out"),
                    help="folder for the report, mismatch dumps and a copy of the golden file")
    out_dir = ap.parse_args().out_dir
    ref_so = os.path.join(ROOT, "oracle", "_ref", "mor_ref_C.so")
    if not os.path.exists(ref_so):
        print(f"{ref_so} missing: run oracle/build_ref.sh where the reference sources are", file=sys.stderr)
        return 2
    if not torch.cuda.is_available():
        print("no CUDA device", file=sys.stderr)
        return 2
    torch.ops.load_library(ref_so)
    os.makedirs(out_dir, exist_ok=True)
    report = open(os.path.join(out_dir, "golden_report.txt"), "w")
    golden = {"device": torch.cuda.get_device_name(0), "torch": torch.__version__, "cases": {}}
    n_bad = 0
    for name, op, fn, kw in cases():
        x = fn()
        oracle.clear_assert_flags()
        try:
            exp = run_oracle(op, x, kw)
        except oracle.OracleError as e:
            report.write(f"{name}: oracle refuses ({e}); not run\n")
            continue
        flags = oracle.assert_flags()
        if flags:
            report.write(f"{name}: SKIPPED, reference assert would fire (flags {flags})\n")
            golden["cases"][name] = {"skipped": f"reference device assert, oracle flags {flags}"}
            continue
        got = run_reference(op, x, kw)
        torch.cuda.synchronize()
        rec = {"op": op, "input_sha256": digest(x), "out_sha256": digest(canon(got["out"]))}
        if "meta" in got:
            rec["meta"] = got["meta"].astype(int).reshape(-1).tolist()
        for k in ("gamax", "gerr"):
            if k in got:
                rec[k + "_bits"] = f32_bits(got[k])
        if "gnnz" in got:
            rec["gnnz"] = got["gnnz"]
        golden["cases"][name] = rec
        # diagnostics against the oracle, here where both are at hand
        same_out = np.array_equal(canon(got["out"]), canon(exp["out"]))
        msgs = []
        if not same_out:
            a, b = canon(got["out"]).reshape(-1), canon(exp["out"]).reshape(-1)
            bad = np.nonzero(a != b)[0]
            msgs.append(f"out differs at {bad.size} of {a.size}; first idx {bad[:5].tolist()} "
                        f"ref {a[bad[:5]].tolist()} oracle {b[bad[:5]].tolist()} in {x.reshape(-1)[bad[:5]].tolist()}")
            np.savez_compressed(os.path.join(out_dir, f"golden_mismatch_{name}.npz"), x=x,
                                ref=got["out"], oracle=exp["out"])
        if "meta" in got and not np.array_equal(got["meta"].reshape(-1), np.asarray(exp["meta"]).reshape(-1)):
            msgs.append(f"meta ref {got['meta'].reshape(-1).tolist()} oracle {np.asarray(exp['meta']).reshape(-1).tolist()}")
        for k in ("gamax", "gerr"):
            if k in got and f32_bits(got[k]) != f32_bits(exp[k]):
                msgs.append(f"{k} ref {got[k]!r} oracle {float(exp[k])!r}")
        if "gnnz" in got and got["gnnz"] != exp["gnnz"]:
            msgs.append(f"gnnz ref {got['gnnz']} oracle {exp['gnnz']}")
        n_bad += bool(msgs)
        report.write(f"{name}: {'OK' if not msgs else 'MISMATCH ' + '; '.join(msgs)}\n")
        report.flush()
    with open(os.path.join(HERE, "reference_b200.json"), "w") as f:
        json.dump(golden, f, indent=1, sort_keys=True)
    # a copy in the folder that travels back from a remote GPU run
    with open(os.path.join(out_dir, "reference_b200.json"), "w") as f:
        json.dump(golden, f, indent=1, sort_keys=True)
    report.write(f"cases {len(golden['cases'])}, oracle mismatches {n_bad}\n")
    report.close()
    print(f"recorded {len(golden['cases'])} cases, {n_bad} differ from the oracle")
    return 0


if __name__ == "__main__":
    sys.exit(main())
