"""Benchmark of the fake-quantization hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W]            one JSON line on stdout
    python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N ...
    python bench.py --impl reference ...                           CPU arm (the oracle on the host cores)
    python bench.py --suite                                        also times every kernel family on
                                                                   configurations 1-5 (table in <run-output folder>/suite.json)

Workload: configuration 5 -- a float32 131072 x 16384 tensor (8 GiB, N(0,1), synthetic),
row-sharded over the N ranks, fake-quantized to E4M3 with 128 x 128 block scaling under
the global-mantissa rule (ss_mode 1): slab amax kernel, amax/nnz all-reduce, scale +
cast + error kernel, error all-gather, ordered error sum and BF16-fallback decision.
Total work is fixed as N grows ("strong" scaling).  A step is one pass over the tensor.

Metric: algorithmic GB/s, whole job = 12 bytes per element (two reads and one write of
float32, the accounting of the reference authors' own harness) / step time; inputs are
resident in HBM when the timed region starts and are far larger than L2, so no flush
is needed.  `e2e` is the same metric from pinned HOST buffers through the same call
with both copies inside the timed region.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

ROWS, COLS, BLOCK = 131072, 16384, 128
BYTES_PER_ELEM_TWO_PASS = 12   # 2 x 4-byte reads + 1 x 4-byte write
THRESHOLD = 0.045              # the reference tests' e4m3_threshold
SS_MODE = 1
FALLBACK_HBM_GBS = 6650.0      # used only when MEASURED_PEAKS.json is absent
# dram read + write bytes of the dominant kernel per algorithmic byte, from one ncu capture of a
# 1 GiB slab (profiles/block_tile128_fp32_config5.md: 2.0914 GB moved for 2.1475 GB algorithmic);
# one CTA per block and no reuse across blocks, so traffic grows in proportion to the elements
TRAFFIC_PER_ALGORITHMIC_BYTE = 2.0914 / 2.1475


def measured_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons, sampled every 200 ms while running."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu, self.rows, self.proc = gpu_index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.gpu)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *a):
        if self.proc:
            time.sleep(0.25)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[1])); mx.append(float(r[2]))
                for n, v in zip(names, r[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
            except Exception:
                continue
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


def cpu_baseline(rows_sample_hint=None, budget_s=12.0, steps=1, warmup=0):
    """Times the CPU oracle (a port of the reference arithmetic, OpenMP over blocks) on a
    bounded row sample of the workload: same columns, same block scaling, all host threads."""
    import numpy as np
    import oracle
    # all the host cores this process may use, whatever OMP_NUM_THREADS says (torchrun sets it to 1)
    try:
        avail = len(os.sched_getaffinity(0))
    except AttributeError:
        avail = os.cpu_count() or 1
    oracle.set_num_threads(avail)
    threads = oracle.num_threads()
    rng = np.random.default_rng(4000)
    probe = rng.standard_normal((BLOCK * 2, COLS), dtype=np.float32)
    t0 = time.perf_counter()
    oracle.block_scaling(probe, BLOCK, BLOCK, THRESHOLD, SS_MODE)
    dt = max(time.perf_counter() - t0, 1e-4)
    rate = probe.size / dt
    rows = rows_sample_hint or int(min(16384, max(256, (rate * budget_s / max(steps + warmup, 1)) // COLS // BLOCK * BLOCK)))
    x = rng.standard_normal((rows, COLS), dtype=np.float32)
    for _ in range(warmup):
        oracle.block_scaling(x, BLOCK, BLOCK, THRESHOLD, SS_MODE)
    t0 = time.perf_counter()
    for _ in range(max(steps, 1)):
        oracle.block_scaling(x, BLOCK, BLOCK, THRESHOLD, SS_MODE)
    dt = (time.perf_counter() - t0) / max(steps, 1)
    gbs = x.size * BYTES_PER_ELEM_TWO_PASS / dt / 1e9
    return {"value": gbs, "unit": "GB/s", "cores": threads, "kind": "port",
            "sample": f"{rows} of {ROWS} rows x {COLS} float32, block scaling ss_mode 1, {threads} OpenMP threads, "
                      f"{dt * 1e3:.0f} ms per pass",
            "elements_per_s": x.size / dt, "ms_per_step": dt * 1e3}


def reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    b = cpu_baseline(budget_s=20.0, steps=args.steps, warmup=args.warmup)
    line = {
        "impl": "reference", "metric": "fake_quantize_throughput", "value": b["value"], "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": b["ms_per_step"],
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "config5: float32 131072x16384, 128x128 block scaling ss_mode 1 (bounded row sample)"},
        "cpu_baseline": {k: b[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": b["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "elements_per_s": b["elements_per_s"], "gpu_launches": 0,
    }
    print(json.dumps(line))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--suite", action="store_true", help="also time configurations 1-4 (single GPU)")
    ap.add_argument("--scale", type=int, default=1, help="divide the row count (development only; reported)")
    ap.add_argument("--no-main", action="store_true", help="skip the configuration-5 workload (profiling the suite)")
    ap.add_argument("--suite-only", default="", help="substring filter on suite entry names")
    ap.add_argument("--suite-iters", type=int, default=10)
    ap.add_argument("--suite-impl", choices=["ours", "reference"], default="ours",
                    help="reference: time the unmodified reference CUDA extension (oracle/_ref) on the configurations it supports")
    ap.add_argument("--suite-graph", action="store_true", help="also time the suite calls replayed as one CUDA graph")
    ap.add_argument("--suite-out", default=None, help="where --suite writes its table (default: suite.json in the run-output folder)")
    ap.add_argument("--exchange", choices=["auto", "nccl", "p2p"], default="auto",
                    help="how ranks exchange amax / non-zero count / error sums (N > 1): NCCL collectives or peer stores")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        return reference_arm(args)

    import torch
    import torch.distributed as dist

    if args.no_main and args.suite_impl == "reference":
        # the reference extension registers the same torch.ops.mor.* names as the repository's shim: this
        # process loads the workload generators by file and never imports the mor_b200 package
        import importlib.util
        spec = importlib.util.spec_from_file_location("_workloads", os.path.join(ROOT, "mor_b200", "workloads.py"))
        wl = importlib.util.module_from_spec(spec)
        sys.modules["_workloads"] = wl
        spec.loader.exec_module(wl)
        if not torch.cuda.is_available():
            raise SystemExit("the reference extension needs a CUDA device")
        peak, _ = measured_peak()
        run_suite(torch, torch.device("cuda", 0), peak, args.suite_only, args.suite_iters, args.suite_out, False,
                  "reference", wl)
        return 0

    import mor_b200  # noqa: F401  fails loudly if the CUDA library or the shim is missing
    from mor_b200 import workloads
    from mor_b200.sharded import KIND_BLOCK, ShardedScaling, shard_rows

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU path (use --impl reference for the CPU arm)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    n_gpus = world

    if args.no_main:
        peak, _ = measured_peak()
        run_suite(torch, dev, peak, args.suite_only, args.suite_iters, args.suite_out, args.suite_graph, args.suite_impl)
        return 0

    rows = ROWS // args.scale
    r0, r1 = shard_rows(rows, world, rank, BLOCK)
    rows_local = r1 - r0
    # synthetic N(0,1) float32 slab, drawn on the device (seed 4000 + rank)
    g = torch.Generator(device=dev).manual_seed(4000 + rank)
    x = torch.empty(rows_local, COLS, dtype=torch.float32, device=dev)
    chunk = 4096
    for i in range(0, rows_local, chunk):
        x[i:i + chunk].normal_(generator=g)
    out = torch.empty_like(x)
    op = ShardedScaling(rows_local, COLS, BLOCK, BLOCK, torch.float32, dev, KIND_BLOCK, exchange=args.exchange)

    # events around the dominant kernel (scale + cast + error sums), on the launching stream
    cast_events = []
    amax_events = []
    inner_cast, inner_amax, inner_amax_local = op.backend.cast, op.backend.amax_nnz, op.backend.amax_nnz_local

    def timed_cast(*a):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record(); inner_cast(*a); e.record()
        cast_events.append((s, e))

    def timed_amax(*a):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record(); inner_amax(*a); e.record()
        amax_events.append((s, e))

    def timed_amax_local(*a):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record(); inner_amax_local(*a); e.record()
        amax_events.append((s, e))

    op.backend.cast, op.backend.amax_nnz, op.backend.amax_nnz_local = timed_cast, timed_amax, timed_amax_local

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        res = op(x, out, SS_MODE, THRESHOLD)
    barrier()
    cast_events.clear(); amax_events.clear()
    launches0 = op.backend.launches
    with ClockSampler(local_rank) as clocks:
        barrier()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        for _ in range(args.steps):
            res = op(x, out, SS_MODE, THRESHOLD)
        ev1.record()
        barrier()
    step_ms = ev0.elapsed_time(ev1) / args.steps
    launches = op.backend.launches - launches0
    cast_ms = statistics.mean(s.elapsed_time(e) for s, e in cast_events)
    amax_ms = statistics.mean(s.elapsed_time(e) for s, e in amax_events)
    meta = int(res.meta.item())

    t = torch.tensor([step_ms, cast_ms, amax_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    step_ms, cast_ms, amax_ms = t.tolist()

    total_elems = rows * COLS
    value = total_elems * BYTES_PER_ELEM_TWO_PASS / (step_ms * 1e-3) / 1e9
    peak, peak_kind = measured_peak()
    cast_bytes = rows_local * COLS * 8          # algorithmic bytes of one launch: float32 read + write
    achieved = cast_bytes / (cast_ms * 1e-3) / 1e9

    # ---- end to end from pinned host buffers ---------------------------------------
    e2e = None
    if not args.no_e2e:
        nbytes = rows_local * COLS * 4
        xh = torch.empty(rows_local, COLS, dtype=torch.float32, pin_memory=True)
        oh = torch.empty(rows_local, COLS, dtype=torch.float32, pin_memory=True)
        xh.copy_(x)
        scal_h = torch.empty(2, dtype=torch.float32, pin_memory=True)
        e2e_steps = max(2, min(args.steps, 10))
        out = None
        torch.cuda.empty_cache()
        from mor_b200.sharded import HostScaling
        host_op = HostScaling(rows_local, COLS, BLOCK, BLOCK, torch.float32, dev, KIND_BLOCK, exchange=args.exchange)

        def e2e_step():
            host_op(xh, oh, scal_h, SS_MODE, THRESHOLD)

        for _ in range(2):
            e2e_step()
        host_op.synchronize()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(e2e_steps):
            e2e_step()
        host_op.s_out.wait_stream(torch.cuda.current_stream())
        torch.cuda.current_stream().wait_stream(host_op.s_out)   # the last read-back ends the timed region
        e1.record()
        host_op.synchronize()
        barrier()
        e2e_ms = e0.elapsed_time(e1) / e2e_steps
        tt = torch.tensor([e2e_ms], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        e2e_ms = tt.item()
        e2e = {"value": total_elems * BYTES_PER_ELEM_TWO_PASS / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s",
               "h2d_bytes_per_step": nbytes * world, "d2h_bytes_per_step": (nbytes + 8) * world,
               "ms_per_step": e2e_ms, "steps": e2e_steps,
               "note": "mor_b200.sharded.HostScaling: pinned host float32 in and out, every step uploads its input and "
                       "reads its output back; two device buffer sets, so one step's upload overlaps the previous "
                       "step's read-back"}
        del xh, oh, host_op

    suite = None
    if args.suite and rank == 0 and world == 1:
        out = None
        torch.cuda.empty_cache()
        suite = run_suite(torch, dev, peak, args.suite_only, args.suite_iters, args.suite_out, args.suite_graph, args.suite_impl)

    if rank == 0:
        line = {
            "metric": "fake_quantize_throughput", "value": value, "unit": "GB/s", "n_gpus": n_gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": step_ms, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"config5: float32 {rows}x{COLS} (8 GiB / scale {args.scale}), row-sharded over "
                                   f"{n_gpus} GPU(s), 128x128 block scaling ss_mode 1 with global amax",
                       "bytes_per_element": BYTES_PER_ELEM_TWO_PASS, "l2": "inputs larger than L2, no flush",
                       "threshold": THRESHOLD, "meta": meta,
                       "exchange": ("single GPU" if n_gpus == 1 else ("peer stores over NVLink" if op.peer is not None else "NCCL"))},
            "elements_per_s": total_elems / (step_ms * 1e-3),
            "per_gpu": {"GB/s": value / n_gpus, "elements_per_s": total_elems / (step_ms * 1e-3) / n_gpus,
                        "pct_of_hbm_peak": 100.0 * value / n_gpus / peak, "peak_GB/s": peak, "peak_kind": peak_kind},
            "roofline": {"bound": "hbm", "kernel": "block_tile128_kernel<Fp32> (TMA-staged tile: scale + E4M3 cast + error sums)",
                         "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_kind": peak_kind, "ms_per_launch": cast_ms, "bytes_per_launch": cast_bytes,
                         "traffic": cast_bytes * TRAFFIC_PER_ALGORITHMIC_BYTE,
                         "traffic_source": "ncu dram__bytes_read+write on a 1 GiB slab, scaled by elements",
                         "amax_kernel": {"ms_per_launch": amax_ms,
                                         "achieved": rows_local * COLS * 4 / (amax_ms * 1e-3) / 1e9}},
            "clocks": clocks.summary(),
            "gpu_launches": launches * n_gpus,
        }
        if e2e:
            line["e2e"] = e2e
        if not args.no_cpu and world == 1:
            b = cpu_baseline()
            line["cpu_baseline"] = {k: b[k] for k in ("value", "unit", "cores", "kind", "sample")}
        if suite:
            line["suite_file"] = "gpurun_out/suite.json"
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
    return 0


def run_suite(torch, dev, peak, only="", iters=10, out_path=None, use_graph=False, impl="ours", workloads=None):
    """Times every kernel family on configurations 1-5 (one GPU).  Every operator runs
    `iters` times back to back between one pair of CUDA events on the launching stream;
    successive calls take their input from, and leave their outputs in, a ring of distinct
    buffers whose total size is at least four times the L2, so that no call finds its
    input or the lines of its output in cache.  The time per call is the total divided
    by `iters`: launch gaps between the kernels of a pipeline are part of it."""
    if workloads is None:
        from mor_b200 import workloads
    if impl == "reference":
        # the unmodified reference extension, built by oracle/build_ref.sh; it registers torch.ops.mor.*,
        # so this process must not load the repository's own extension
        ref_so = os.path.join(ROOT, "oracle", "_ref", "mor_ref_C.so")
        if not os.path.exists(ref_so):
            raise SystemExit("oracle/_ref/mor_ref_C.so is missing: run oracle/build_ref.sh where the reference sources are")
        torch.ops.load_library(ref_so)

        def call(op, x, args):
            return getattr(torch.ops.mor, op).default(x, *args)
    else:
        import mor

        def call(op, x, args):
            return getattr(mor.ops, op)(x, *args)
    results = []
    ring_bytes = 512 << 20

    def time_call(fn, x, n=iters, warm=3):
        k = max(2, -(-ring_bytes // (x.numel() * x.element_size())))
        xs = [x] + [x.clone() for _ in range(k - 1)]
        outs = [None] * k
        for i in range(max(warm, k + 1)):  # also fills the ring, so that no allocation is left for the timed loop
            outs[i % k] = fn(xs[i % k])
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for i in range(n):
            outs[i % k] = fn(xs[i % k])
        e.record()
        torch.cuda.synchronize()
        eager_ms = s.elapsed_time(e) / n
        # the same n calls as one CUDA graph: what the device needs when the host is out of the way
        graph_ms = None
        if use_graph:
            try:
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    for i in range(n):
                        outs[i % k] = fn(xs[i % k])
                g.replay()
                torch.cuda.synchronize()
                s.record(); g.replay(); e.record()
                torch.cuda.synchronize()
                graph_ms = s.elapsed_time(e) / n
                del g
            except Exception as ex:  # an operator that cannot be captured keeps its eager time only
                print(f"[suite] graph capture failed: {ex}", file=sys.stderr)
        return eager_ms, graph_ms, k

    def add(name, x, bytes_per_elem, op, args, ref_ok=False):
        if only and only not in name:
            return
        if impl == "reference" and not ref_ok:   # shapes or operators the reference does not have, or asserts on
            return
        fn = lambda t: call(op, t, args)  # noqa: E731
        ms, graph_ms, k = time_call(fn, x)
        n = x.numel()
        gbs = n * bytes_per_elem / (ms * 1e-3) / 1e9
        rec = {"name": name, "rows": x.shape[0], "cols": x.shape[1], "ms": ms, "GB/s": gbs,
               "elements_per_s": n / (ms * 1e-3), "bytes_per_element": bytes_per_elem,
               "frac_of_peak": gbs / peak, "buffers_in_ring": k}
        line = f"[suite] {name}: {ms:.4f} ms  {gbs:.0f} GB/s  {100 * gbs / peak:.1f}% of peak"
        if graph_ms:
            ggbs = n * bytes_per_elem / (graph_ms * 1e-3) / 1e9
            rec.update({"graph_ms": graph_ms, "graph_GB/s": ggbs, "graph_frac_of_peak": ggbs / peak})
            line += f"   | as a CUDA graph: {graph_ms:.4f} ms  {ggbs:.0f} GB/s  {100 * ggbs / peak:.1f}%"
        results.append(rec)
        print(line, file=sys.stderr)

    x = workloads.config1(device=dev)
    r, c = x.shape
    scale = (torch.tensor(448.0) / x.float().abs().max().cpu()).item()   # binary32 division, as the cast kernels do
    add("c1 per-tensor E4M3, scale given (fake_quantize mode 4)", x, 4, "fake_quantize", (r, c, 128, 128, scale, 4, 1), ref_ok=True)
    add("c1 per-tensor E4M3, self-contained (block_scaling ss 4)", x, 6, "fake_quantize_block_scaling", (r, c, 128, 128, 3e38, 4), ref_ok=True)
    del x
    x = workloads.config2(device=dev)
    r, c = x.shape
    add("c2 per-row E4M3 single pass (fake_quantize mode 2, 1x8192)", x, 4, "fake_quantize", (r, c, 1, c, 0.0, 2, 1))
    add("c2 per-row E5M2 single pass (fake_quantize mode 3, 1x8192)", x, 4, "fake_quantize", (r, c, 1, c, 0.0, 3, 1))
    # not for the reference arm: its channel path launches the 1024-thread reductions with the 64-thread
    # kernels' shared-memory size (fake_quantize.cu:2515-2522) and raised an illegal memory access at this size
    add("c2 per-row E4M3 pipeline (channel_scaling ss 3)", x, 6, "fake_quantize_channel_scaling", (r, c, 1, c, 3e38, 3))
    del x
    x = workloads.config3(device=dev)
    r, c = x.shape
    add("c3 MX 1x32 E8M0 E4M3 single pass (fake_quantize_mx)", x, 4, "fake_quantize_mx", (r, c, 32, 0, 2))
    add("c3 MX 1x32 E8M0 E2M3 single pass (fake_quantize_mx)", x, 4, "fake_quantize_mx", (r, c, 32, 3, 2))
    add("c3 MX 1x32 real quantization, E4M3 codes + E8M0 scales (quantize_mx)", x, 3.03125, "quantize_mx", (r, c, 32, 0))
    add("c3 MX 1x32 E4M3 pipeline (channel_scaling ss 2)", x, 6, "fake_quantize_channel_scaling", (r, c, 1, 32, 3e38, 2))
    del x
    x = workloads.config4(device=dev)
    r, c = x.shape
    if impl != "reference":
        amax_prev4 = x.float().abs().max().reshape(1)
        add("c4 block scaling 128x128, single pass with delayed amax (ss 1)", x, 4, "fake_quantize_block_scaling_delayed",
            (r, c, 128, 128, 3e38, 1, amax_prev4))
    add("c4 MoR 128x128 relative-error criterion (mode 1)", x, 4, "fake_quantize", (r, c, 128, 128, 1e-15, 1, 1), ref_ok=True)
    add("c4 MoR 128x128 dynamic-range criterion (mode 101)", x, 4, "fake_quantize", (r, c, 128, 128, 1e-15, 101, 1), ref_ok=True)
    add("c4 block scaling 128x128 pipeline (ss 1)", x, 6, "fake_quantize_block_scaling", (r, c, 128, 128, 3e38, 1), ref_ok=True)
    del x
    if impl != "reference":
        x = workloads.config5_slab(0, device=dev)
        r, c = x.shape
        add("c5 float32 1 GiB slab block scaling 128x128 pipeline (ss 1)", x, 12, "fake_quantize_block_scaling", (r, c, 128, 128, THRESHOLD, 1))
        amax_prev = x.abs().max().reshape(1).float()
        add("c5 float32 1 GiB slab block scaling, single pass with delayed amax (ss 1)", x, 8,
            "fake_quantize_block_scaling_delayed", (r, c, 128, 128, THRESHOLD, 1, amax_prev))
        add("c5 float32 1 GiB slab per-tensor pipeline (ss 4)", x, 12, "fake_quantize_block_scaling", (r, c, 128, 128, THRESHOLD, 4))
        del x
    os.makedirs(os.path.join(ROOT, "gpurun_out"), exist_ok=True)
    with open(out_path or os.path.join(ROOT, "gpurun_out", "suite.json"), "w") as f:
        json.dump({"peak_GB/s": peak, "impl": impl, "results": results}, f, indent=1)
    return results


if __name__ == "__main__":
    sys.exit(main())
