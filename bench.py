"""Benchmark of the fake-quantization hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W]            one JSON line on stdout
    python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N ...
    python bench.py --impl reference ...                           CPU arm (the oracle on the host cores)
    python bench.py --suite                                        every kernel family on configurations 1-5,
                                                                   full table in <out-dir>/suite.json

Workload: configuration 5 -- a float32 131072 x 16384 tensor (8 GiB, N(0,1), synthetic),
row-sharded over the N ranks, fake-quantized to E4M3 with 128 x 128 block scaling under
the global-mantissa rule (ss_mode 1): slab amax kernel, amax/nnz exchange, scale +
cast + error kernel, error gather, ordered error sum and BF16-fallback decision.
Total work is fixed as N grows ("strong" scaling).  A step is one pass over the tensor.
The tensor is drawn per 16384-row slab (seed 4000 + slab index), so it holds the same bits
whatever N is, and the line carries checksums of the output and the bit patterns of the
scalar results: equal across N means equal output.

Metric: algorithmic GB/s, whole job = 12 bytes per element (two reads and one write of
float32, the accounting of the reference authors' own harness) / step time; inputs are
resident in HBM when the timed region starts and are far larger than L2, so no flush
is needed.  `e2e` is the same metric from pinned HOST buffers through the same call
with both copies inside the timed region, next to a copy-only loop over the same buffers.

At N = 1 the line also carries `configs`: the other benchmark configurations (and the E8Mx and
column-group operators) timed eagerly and as a CUDA graph, each checked against the CPU oracle.
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
SLAB_ROWS = 16384              # rows drawn from one seed (1 GiB of float32)
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


def host_threads():
    """all the host cores this process may use, whatever OMP_NUM_THREADS says (torchrun sets it to 1)"""
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def gpu_numa_node(index: int):
    """NUMA node of the GPU's PCIe slot as the kernel reports it (None where that is not exposed)"""
    try:
        bus = subprocess.run(["nvidia-smi", "--query-gpu=pci.bus_id", "--format=csv,noheader", "-i", str(index)],
                             capture_output=True, text=True, timeout=20).stdout.strip().lower()
        dom, rest = bus.split(":", 1)
        return int(open(f"/sys/bus/pci/devices/{dom[-4:]}:{rest}/numa_node").read().strip())
    except Exception:
        return None


class ClockSampler:
    """SM clock and throttle reasons while the timed region runs: NVML queries (read-only) from a thread every few
    milliseconds, so that a region of some tens of milliseconds still gets samples; `nvidia-smi -lms` otherwise.
    Only samples taken between `mark_start()` and `mark_end()` count, if there are any."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")
    REASONS = (("hw_slowdown", 0x8), ("hw_thermal_slowdown", 0x40), ("sw_thermal_slowdown", 0x20), ("sw_power_cap", 0x4))

    def __init__(self, gpu_index: int):
        self.gpu, self.rows, self.proc, self.nvml, self.stop = gpu_index, [], None, None, False
        self.t0 = self.t1 = None

    def mark_start(self):
        self.t0 = time.time()

    def mark_end(self):
        self.t1 = time.time()

    def __enter__(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(self.gpu)
            self.max_sm = float(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
            self.nvml = pynvml
            self.t = threading.Thread(target=self._poll, daemon=True)
            self.t.start()
            return self
        except Exception:
            self.nvml = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.gpu)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None
        return self

    def _poll(self):
        n = self.nvml
        get_reasons = getattr(n, "nvmlDeviceGetCurrentClocksEventReasons", None) or n.nvmlDeviceGetCurrentClocksThrottleReasons
        while not self.stop:
            try:
                sm = float(n.nvmlDeviceGetClockInfo(self.handle, n.NVML_CLOCK_SM))
                mask = int(get_reasons(self.handle))
                self.rows.append((time.time(), sm, self.max_sm, [name for name, bit in self.REASONS if mask & bit]))
            except Exception:
                pass
            time.sleep(0.003)

    def _read(self):
        names = [name for name, _ in self.REASONS]
        for line in self.proc.stdout:
            r = [c.strip() for c in line.split(",")]
            try:
                self.rows.append((time.time(), float(r[1]), float(r[2]),
                                  [n for n, v in zip(names, r[5:9]) if v.lower().startswith("active")]))
            except Exception:
                continue

    def __exit__(self, *a):
        if self.nvml:
            self.stop = True
            self.t.join(timeout=2)
            try:
                self.nvml.nvmlShutdown()
            except Exception:
                pass
        elif self.proc:
            time.sleep(0.25)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()

    def summary(self):
        rows = self.rows
        if self.t0 is not None and self.t1 is not None:
            inside = [r for r in rows if self.t0 <= r[0] <= self.t1]
            rows = inside or rows
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        reasons = set()
        for r in rows:
            reasons.update(r[3])
        return {"sm_mhz": statistics.median(r[1] for r in rows), "sm_max_mhz": max(r[2] for r in rows),
                "reasons": sorted(reasons), "samples": len(rows), "source": "nvml" if self.nvml else "nvidia-smi"}


# --------------------------------------------------------------------------------------
# CPU legs: the only places where the oracle (a CPU port of the reference arithmetic) is used
# --------------------------------------------------------------------------------------
def cpu_baseline(sample=None, budget_s=12.0, passes=3, gpu_result=None):
    """Times the CPU oracle (OpenMP over blocks, all host threads) on a bounded row sample of the workload:
    one untimed pass, then the median of `passes` timed ones.  `sample` is a float32 [rows, COLS] array (the
    benchmark passes the first slab of the tensor it timed); without one a sample is drawn here.  With
    `gpu_result` = (global_amax, output rows, block errors) of the GPU run on that sample, the oracle's output
    for the same global amax is compared with it bit for bit."""
    import numpy as np
    import oracle
    oracle.set_num_threads(host_threads())
    threads = oracle.num_threads()
    origin = "the first rows of the timed tensor"
    if sample is None:
        origin = "N(0,1) drawn on the host"
        rng = np.random.default_rng(4000)
        probe = rng.standard_normal((BLOCK * 2, COLS), dtype=np.float32)
        t0 = time.perf_counter()
        oracle.block_scaling(probe, BLOCK, BLOCK, THRESHOLD, SS_MODE)
        rate = probe.size / max(time.perf_counter() - t0, 1e-4)
        rows = int(min(SLAB_ROWS, max(256, (rate * budget_s / (passes + 1)) // COLS // BLOCK * BLOCK)))
        sample = rng.standard_normal((rows, COLS), dtype=np.float32)
    rows = sample.shape[0]
    oracle.block_scaling(sample, BLOCK, BLOCK, THRESHOLD, SS_MODE)   # warm-up: page faults, thread pool
    times = []
    for _ in range(max(passes, 1)):
        t0 = time.perf_counter()
        oracle.block_scaling(sample, BLOCK, BLOCK, THRESHOLD, SS_MODE)
        times.append(time.perf_counter() - t0)
    dt = statistics.median(times)
    gbs = sample.size * BYTES_PER_ELEM_TWO_PASS / dt / 1e9
    res = {"value": gbs, "unit": "GB/s", "cores": threads, "kind": "port",
           "sample": f"{rows} of {ROWS} rows x {COLS} float32 ({origin}), block scaling ss_mode 1, "
                     f"{threads} OpenMP threads, median of {len(times)} warmed passes, {dt * 1e3:.0f} ms per pass",
           "elements_per_s": sample.size / dt, "ms_per_step": dt * 1e3}
    if gpu_result is not None:
        gamax, gpu_out, gpu_err = gpu_result
        # threshold out of reach: the tensor-level BF16 decision belongs to the whole tensor, not to the sample
        out, _, _, _, _, _, berr = oracle.block_scaling(sample, BLOCK, BLOCK, 3e38, SS_MODE, global_amax=gamax,
                                                        want_blocks=True)
        same_out = bool(np.array_equal(out.view(np.uint32), gpu_out.view(np.uint32)))
        same_err = bool(np.array_equal(berr.view(np.uint32), gpu_err.view(np.uint32)))
        res["parity"] = {"slab0_bit_exact": same_out, "slab0_block_errors_bit_exact": same_err, "rows_checked": rows}
    return res


def cpu_baseline_torch():
    """The reference's PyTorch CPU path (the computation its tests compare the kernels with,
    test/test_fake_quantize.py:96-104: scale = 448 / amax, cast to float8_e4m3fn and back, divide) on
    configuration 1 (bf16 4096 x 4096), at 4 bytes per element."""
    import torch
    g = torch.Generator().manual_seed(0)
    x = torch.randn(4096, 4096, generator=g).to(torch.bfloat16)

    def once():
        xf = x.float()
        scale = torch.tensor(448.0) / xf.abs().max()
        return ((xf * scale).to(torch.float8_e4m3fn).float() / scale).to(torch.bfloat16)

    once()
    times = []
    for _ in range(5):
        t0 = time.perf_counter()
        once()
        times.append(time.perf_counter() - t0)
    dt = statistics.median(times)
    return {"value": x.numel() * 4 / dt / 1e9, "unit": "GB/s", "threads": torch.get_num_threads(),
            "host_cores": os.cpu_count(), "kind": "reference tests' torch CPU path",
            "sample": f"configuration 1 (bf16 4096 x 4096, per-tensor E4M3), median of 5 passes, {dt * 1e3:.1f} ms per pass"}


def reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    b = cpu_baseline(budget_s=20.0, passes=max(args.steps, 1))
    line = {
        "impl": "reference", "metric": "fake_quantize_throughput", "value": b["value"], "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": b["ms_per_step"],
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "config5: float32 131072x16384, 128x128 block scaling ss_mode 1 (bounded row sample)"},
        "cpu_baseline": {k: b[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": b["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "elements_per_s": b["elements_per_s"], "gpu_launches": 0,
    }
    try:
        line["cpu_baseline_torch"] = cpu_baseline_torch()
    except Exception as e:  # a torch build without float8 on the CPU: the oracle number stands alone
        line["cpu_baseline_torch"] = {"unavailable": str(e)[:200]}
    print(json.dumps(line))
    return 0


# --------------------------------------------------------------------------------------
def draw_rows(torch, dev, r0, r1):
    """rows [r0, r1) of the benchmark tensor: slab s (SLAB_ROWS rows) is N(0,1) from seed 4000 + s"""
    x = torch.empty(r1 - r0, COLS, dtype=torch.float32, device=dev)
    s = r0 // SLAB_ROWS
    while s * SLAB_ROWS < r1:
        g = torch.Generator(device=dev).manual_seed(4000 + s)
        slab = torch.empty(SLAB_ROWS, COLS, dtype=torch.float32, device=dev)
        for i in range(0, SLAB_ROWS, 4096):
            slab[i:i + 4096].normal_(generator=g)
        a, b = max(r0, s * SLAB_ROWS), min(r1, (s + 1) * SLAB_ROWS)
        x[a - r0:b - r0] = slab[a - s * SLAB_ROWS:b - s * SLAB_ROWS]
        del slab
        s += 1
    return x


def checksums(torch, out, first_row):
    """two 64-bit sums of the output's 32-bit words (the second weighted by the global row number), additive over
    ranks, so that equal values across N mean equal output bits"""
    total = torch.zeros(2, dtype=torch.int64, device=out.device)
    for a in range(0, out.shape[0], 8192):      # in row chunks: the widened copy of 8 GiB would not be small
        w = out[a:a + 8192].view(torch.int32).to(torch.int64) & 0xFFFFFFFF
        rowsum = w.sum(dim=1)
        weights = torch.arange(first_row + a + 1, first_row + a + 1 + rowsum.numel(), device=out.device, dtype=torch.int64)
        total += torch.stack([rowsum.sum(), (rowsum * weights).sum()])
    return total


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--suite", action="store_true", help="time every suite entry (the default line carries a compact set)")
    ap.add_argument("--scale", type=int, default=1, help="divide the row count (development only; reported)")
    ap.add_argument("--no-main", action="store_true", help="skip the configuration-5 workload (profiling the suite)")
    ap.add_argument("--suite-only", default="", help="substring filter on suite entry names")
    ap.add_argument("--suite-iters", type=int, default=10)
    ap.add_argument("--suite-impl", choices=["ours", "reference"], default="ours",
                    help="reference: time the unmodified reference CUDA extension (oracle/_ref) on the configurations it supports")
    ap.add_argument("--suite-graph", action="store_true", help="also time the suite calls replayed as one CUDA graph")
    ap.add_argument("--out-dir", default=None, help="folder for suite.json (default: suite_out under the current directory)")
    ap.add_argument("--suite-out", default=None, help="file for the suite table (overrides --out-dir)")
    ap.add_argument("--exchange", choices=["auto", "nccl", "p2p"], default="auto",
                    help="how ranks exchange amax / non-zero count / error sums (N > 1): NCCL collectives or peer stores")
    ap.add_argument("--no-overlap", action="store_true", help="do not pipeline consecutive steps (every step's kernels in one stream)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-configs", action="store_true", help="leave the other configurations out of the line")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        return reference_arm(args)
    suite_path = args.suite_out or os.path.join(args.out_dir or os.path.join(os.getcwd(), "suite_out"), "suite.json")

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
        run_suite(torch, torch.device("cuda", 0), peak, args.suite_only, args.suite_iters, suite_path, False,
                  "reference", wl)
        return 0

    import mor_b200  # noqa: F401  fails loudly if the CUDA library or the shim is missing
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
        run_suite(torch, dev, peak, args.suite_only, args.suite_iters, suite_path, args.suite_graph, args.suite_impl)
        return 0

    rows = ROWS // args.scale
    if (rows // BLOCK) % world:
        raise SystemExit(f"{rows // BLOCK} block rows do not divide over {world} ranks: every rank must hold a slab of the same height")
    r0, r1 = shard_rows(rows, world, rank, BLOCK)
    rows_local = r1 - r0
    x = draw_rows(torch, dev, r0, r1)
    out = torch.empty_like(x)
    # consecutive steps are pipelined: the chain of small kernels after the cast (error exchange, ordered sum,
    # decision, conditional copy) runs on a second stream under the amax pass of the next step
    op = ShardedScaling(rows_local, COLS, BLOCK, BLOCK, torch.float32, dev, KIND_BLOCK, exchange=args.exchange,
                        overlap=not args.no_overlap)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        res = op(x, out, SS_MODE, THRESHOLD)
    barrier()
    launches0 = sum(b.launches for b in op.backends)
    with ClockSampler(local_rank) as clocks:
        barrier()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        clocks.mark_start()
        ev0.record()
        for _ in range(args.steps):
            res = op(x, out, SS_MODE, THRESHOLD)
        ev1.record()
        barrier()
        clocks.mark_end()
    step_ms = ev0.elapsed_time(ev1) / args.steps
    launches = sum(b.launches for b in op.backends) - launches0

    # ---- where a step's time goes: CUDA events around every phase, in a loop of its own (outside the timed region)
    phase_events = {}
    names = {"amax_nnz": "amax", "amax_nnz_local": "amax", "amax_nnz_exchange": "amax", "exchange_scalars": "exchange1", "cast": "cast",
             "exchange_errors": "exchange2", "finalize": "sum", "finalize_ptr": "sum", "fallback": "fallback"}
    originals = []
    for bk in op.backends:
        for meth, label in names.items():
            inner = getattr(bk, meth)
            originals.append((bk, meth, inner))

            def timed(*a, _inner=inner, _label=label):
                s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                s.record(); r = _inner(*a); e.record()   # on the stream the phase is enqueued on
                if r is not False:                       # False: nothing was launched, the caller takes another way
                    phase_events.setdefault(_label, []).append((s, e))
                return r
            setattr(bk, meth, timed)
    barrier()
    n_phase_steps = 8
    for _ in range(n_phase_steps):                   # back to back, as in the timed loop: the host stays ahead of the device
        res = op(x, out, SS_MODE, THRESHOLD)
    barrier()
    for bk, meth, inner in originals:
        setattr(bk, meth, inner)
    # the first two steps start on an idle device (their events also see the host's launch latency): left out
    phases_ms = {k: statistics.mean(s.elapsed_time(e) for s, e in v[2 * len(v) // n_phase_steps:]) for k, v in phase_events.items()}
    # with the exchange of the amax built into the amax kernel there is no "exchange1" of its own: it is part of "amax"
    order = ["amax", "exchange1", "cast", "exchange2", "sum", "fallback"]
    t = torch.tensor([step_ms] + [phases_ms.get(k, 0.0) for k in order], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    vals = t.tolist()
    step_ms = vals[0]
    phases_ms = dict(zip(order, vals[1:]))
    cast_ms, amax_ms = phases_ms["cast"], phases_ms["amax"]

    # ---- what was computed: bit patterns of the scalars, checksums of the output, cross-checks ----
    meta = int(res.meta.item())
    amax_bits = int(res.global_amax.view(torch.int32).item()) & 0xFFFFFFFF
    err_bits = int(res.global_error.view(torch.int32).item()) & 0xFFFFFFFF
    nnz = int(res.global_nnz.item())
    cs = checksums(torch, out, r0)
    # amax and count recomputed by torch, reduced over the ranks by NCCL: independent of the kernels and of the exchange
    chk = torch.zeros(2, dtype=torch.float64, device=dev)
    for a in range(0, rows_local, 8192):
        xc = x[a:a + 8192]
        chk[0] = torch.maximum(chk[0], xc.abs().max().to(torch.float64))
        chk[1] += (xc != 0).sum().to(torch.float64)
    if world > 1:
        dist.all_reduce(cs, op=dist.ReduceOp.SUM)
        mx = chk[0:1].clone(); sm = chk[1:2].clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        dist.all_reduce(sm, op=dist.ReduceOp.SUM)
        chk = torch.cat([mx, sm])
        same = torch.tensor([meta, amax_bits, err_bits, nnz], dtype=torch.int64, device=dev)
        lo, hi = same.clone(), same.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        ranks_agree = bool((lo == hi).all().item())
    else:
        ranks_agree = True
    verified = {"amax_equals_torch_max": float(res.global_amax.item()) == chk[0].item(),
                "nnz_equals_torch_count": nnz == int(chk[1].item()),
                "scalars_identical_on_every_rank": ranks_agree}
    result = {"meta": meta, "global_amax_bits": f"0x{amax_bits:08x}", "global_error_bits": f"0x{err_bits:08x}", "global_nnz": nnz,
              "output_checksum": [f"0x{int(v) & 0xFFFFFFFFFFFFFFFF:016x}" for v in cs.tolist()]}

    total_elems = rows * COLS
    value = total_elems * BYTES_PER_ELEM_TWO_PASS / (step_ms * 1e-3) / 1e9
    peak, peak_kind = measured_peak()
    cast_bytes = rows_local * COLS * 8          # algorithmic bytes of one launch: float32 read + write
    achieved = cast_bytes / (cast_ms * 1e-3) / 1e9

    # the first rows of the timed tensor and what the GPU made of them, for the CPU leg's comparison
    cpu_sample = None
    if rank == 0 and world == 1 and not args.no_cpu:
        n_chk = min(SLAB_ROWS, rows_local)
        cpu_sample = (x[:n_chk].cpu().numpy(), (float(res.global_amax.item()), out[:n_chk].cpu().numpy(),
                                                op.local_err[:(n_chk // BLOCK) * (COLS // BLOCK)].cpu().numpy()))

    # ---- end to end from pinned host buffers ---------------------------------------
    e2e = None
    if not args.no_e2e:
        nbytes = rows_local * COLS * 4
        xh = torch.empty(rows_local, COLS, dtype=torch.float32, pin_memory=True)
        oh = torch.empty(rows_local, COLS, dtype=torch.float32, pin_memory=True)
        xh.copy_(x)
        scal_h = torch.empty(2, dtype=torch.float32, pin_memory=True)
        e2e_steps = max(4, min(args.steps, 16))
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
        starts = [torch.cuda.Event(enable_timing=True) for _ in range(e2e_steps)]
        e0.record()
        for i in range(e2e_steps):
            starts[i].record(host_op.s_in)      # on the upload stream: when this step's upload could begin
            e2e_step()
        host_op.s_out.wait_stream(torch.cuda.current_stream())
        torch.cuda.current_stream().wait_stream(host_op.s_out)   # the last read-back ends the timed region
        e1.record()
        host_op.synchronize()
        barrier()
        e2e_ms = e0.elapsed_time(e1) / e2e_steps
        # the timed region starts with an empty pipeline and ends when it has drained: one upload and one read-back
        # of its K steps overlap nothing.  The period between the uploads of consecutive steps, once both
        # directions are busy, is what a long run sees per step.
        first = min(2, e2e_steps - 2)
        steady_ms = starts[first].elapsed_time(starts[-1]) / (e2e_steps - 1 - first)
        # the same buffers, the same two copy streams, no kernels: what the host links give on their own
        c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        cur = torch.cuda.current_stream()
        host_op.s_in.wait_stream(cur); host_op.s_out.wait_stream(cur)
        c0.record()
        host_op.s_in.wait_event(c0); host_op.s_out.wait_event(c0)
        for i in range(e2e_steps):
            with torch.cuda.stream(host_op.s_in):
                host_op.x[i & 1].copy_(xh, non_blocking=True)
            with torch.cuda.stream(host_op.s_out):
                oh.copy_(host_op.out[i & 1], non_blocking=True)
        cur.wait_stream(host_op.s_in); cur.wait_stream(host_op.s_out)
        c1.record()
        barrier()
        copy_ms = c0.elapsed_time(c1) / e2e_steps
        tt = torch.tensor([e2e_ms, copy_ms, steady_ms], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        e2e_ms, copy_ms, steady_ms = tt.tolist()
        job_bytes = total_elems * BYTES_PER_ELEM_TWO_PASS
        numa = gpu_numa_node(local_rank)
        e2e = {"value": job_bytes / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s",
               "h2d_bytes_per_step": nbytes * world, "d2h_bytes_per_step": (nbytes + 8) * world,
               "ms_per_step": e2e_ms, "steps": e2e_steps,
               "copy_only_GBs": job_bytes / (copy_ms * 1e-3) / 1e9, "copy_only_ms_per_step": copy_ms,
               "frac_of_copy": copy_ms / e2e_ms,
               "steady_state": {"ms_per_step": steady_ms, "GB/s": job_bytes / (steady_ms * 1e-3) / 1e9,
                                "frac_of_copy": copy_ms / steady_ms,
                                "note": "period between the uploads of consecutive steps after the first two; "
                                        "value above is the whole timed region, pipeline fill and drain included"},
               "host_link_GBs_per_direction_per_gpu": nbytes / (copy_ms * 1e-3) / 1e9,
               "host": {"cpu_affinity_cores": host_threads(), "gpu_numa_node": numa},
               "note": "mor_b200.sharded.HostScaling: pinned host float32 in and out, every step uploads its input and "
                       "reads its output back; two device buffer sets, so one step's upload overlaps the previous "
                       "step's read-back.  copy_only: the same uploads and read-backs with no kernels between them, "
                       "in the same units (12 B per element / time)"}
        del xh, oh, host_op

    configs = None
    if rank == 0 and world == 1 and (args.suite or not args.no_configs):
        out = None
        x = None
        torch.cuda.empty_cache()
        configs = run_suite(torch, dev, peak, args.suite_only, args.suite_iters, suite_path, True, args.suite_impl,
                            compact=not args.suite, check=not args.no_cpu)

    if rank == 0:
        line = {
            "metric": "fake_quantize_throughput", "value": value, "unit": "GB/s", "n_gpus": n_gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": step_ms, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"config5: float32 {rows}x{COLS} (8 GiB / scale {args.scale}), row-sharded over "
                                   f"{n_gpus} GPU(s), 128x128 block scaling ss_mode 1 with global amax",
                       "bytes_per_element": BYTES_PER_ELEM_TWO_PASS, "l2": "inputs larger than L2, no flush",
                       "threshold": THRESHOLD, "meta": meta, "seed": "4000 + index of the 16384-row slab",
                       "steps_pipelined": op.overlap,
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
            "phases_us": {k: round(v * 1e3, 2) for k, v in phases_ms.items()},
            "phases_note": "CUDA events around each phase in back-to-back steps; with pipelined steps exchange2, sum and "
                           "fallback run on the second stream under the next step's amax pass, so their figures include "
                           "waiting for free SMs and are not part of the step's critical path",
            "result": result, "verified": verified,
            "clocks": clocks.summary(),
            "gpu_launches": launches * n_gpus,
        }
        if e2e:
            line["e2e"] = e2e
        if cpu_sample is not None:
            b = cpu_baseline(sample=cpu_sample[0], gpu_result=cpu_sample[1])
            line["cpu_baseline"] = {k: b[k] for k in ("value", "unit", "cores", "kind", "sample")}
            line["parity"] = b["parity"]
            try:
                line["cpu_baseline_torch"] = cpu_baseline_torch()
            except Exception as e:
                line["cpu_baseline_torch"] = {"unavailable": str(e)[:200]}
        if configs is not None:
            line["configs"] = [{k: (round(v, 5) if isinstance(v, float) else v) for k, v in c.items()
                                if k in ("name", "ms", "GB/s", "frac_of_peak", "graph_ms", "graph_frac_of_peak", "parity", "launches")}
                               for c in configs]
        print(json.dumps(line))
    if world > 1:
        torch.cuda.synchronize()
        op.close()
        dist.destroy_process_group()
    return 0


# --------------------------------------------------------------------------------------
def oracle_check(op, x, args, outs):
    """Compares one suite call with the CPU oracle, bit for bit (bench.py's CPU leg: a checker, never timed)."""
    import numpy as np
    import torch
    import oracle

    def bits(t):
        t = t.detach().cpu().contiguous()
        if t.dtype == torch.bfloat16:
            return t.view(torch.int16).numpy().view(np.uint16)
        return t.numpy()

    def same(a, b):
        a, b = np.ascontiguousarray(a), np.ascontiguousarray(b)
        return a.shape == b.shape and bool(np.array_equal(a.view(np.uint8), b.view(np.uint8)))

    def f32(v):
        return int(np.array([v], np.float32).view(np.uint32)[0])

    xb = bits(x)
    outs = outs if isinstance(outs, (list, tuple)) else [outs]
    if op == "fake_quantize":
        _, _, bx, by, clamp, mode, sf = args
        eo, em = oracle.fake_quantize(xb, bx, by, clamp, mode, sf)
        return same(bits(outs[0]), eo) and same(outs[1].cpu().numpy(), em)
    if op in ("fake_quantize_block_scaling", "fake_quantize_channel_scaling"):
        _, _, bx, by, thr, ss = args
        fn = oracle.block_scaling if op == "fake_quantize_block_scaling" else oracle.channel_scaling
        e = fn(xb, bx, by, thr, ss)
        return (same(bits(outs[0]), e[0]) and int(outs[1].item()) == e[1] and f32(outs[2].item()) == f32(e[2]) and
                int(outs[3].item()) == e[3] and f32(outs[4].item()) == f32(e[4]))
    if op == "fake_quantize_block_scaling_delayed":
        _, _, bx, by, thr, ss, amax_in = args
        e = oracle.block_scaling(xb, bx, by, thr, ss, global_amax=float(amax_in.item()))
        return same(bits(outs[0]), e[0]) and int(outs[1].item()) == e[1] and int(outs[3].item()) == e[3] and f32(outs[4].item()) == f32(e[4])
    if op == "fake_quantize_block_scaling_delayed_t":
        _, _, bx, by, thr, ss, amax_in = args
        e = oracle.block_scaling(xb, bx, by, thr, ss, global_amax=float(amax_in.item()))
        return same(bits(outs[0]), e[0]) and same(bits(outs[1]), np.ascontiguousarray(e[0].T)) and int(outs[2].item()) == e[1]
    if op == "quantize_scaled":
        _, _, bx, by, ss = args
        ep, es, _ = oracle.quantize_scaled(xb, bx, by, ss)
        return same(outs[0].cpu().numpy(), ep) and same(outs[1].cpu().numpy(), es)
    if op == "fake_quantize_mx":
        _, _, by, fmt, sf = args
        eo, es = oracle.fake_quantize_group(xb, 1, by, fmt, sf, want_scales=True)
        return same(bits(outs[0]), eo) and same(outs[1].cpu().numpy().reshape(-1), es)
    if op == "quantize_mx":
        _, _, by, fmt = args
        ep, es = oracle.quantize_mx(xb, by, fmt)
        return same(outs[0].cpu().numpy(), ep) and same(outs[1].cpu().numpy(), es)
    if op == "fake_quantize_e8mx":
        _, _, _, _, qt, strat = args
        eo, _ = oracle.e8mx(xb, qt, strat)
        return same(bits(outs[0]), eo)
    return None


def run_suite(torch, dev, peak, only="", iters=10, out_path=None, use_graph=False, impl="ours", workloads=None,
              compact=False, check=False):
    """Times every kernel family on configurations 1-5 (one GPU).  Every operator runs
    `iters` times back to back between one pair of CUDA events on the launching stream;
    successive calls take their input from, and leave their outputs in, a ring of distinct
    buffers whose total size is at least four times the L2, so that no call finds its
    input or the lines of its output in cache.  The time per call is the total divided
    by `iters`: launch gaps between the kernels of a pipeline are part of it.
    `compact` keeps one or two entries per configuration (what the default benchmark line carries);
    `check` compares each entry's output with the CPU oracle (outside every timed region)."""
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

    def add(name, x, bytes_per_elem, op, args, ref_ok=False, headline=True):
        if only and only not in name:
            return
        if compact and not headline:
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
        if check and impl != "reference":
            try:
                rec["parity"] = oracle_check(op, x, args, fn(x))
            except Exception as ex:
                rec["parity"] = f"check failed: {str(ex)[:120]}"
            line += f"   | oracle: {rec['parity']}"
        results.append(rec)
        print(line, file=sys.stderr)

    x = workloads.config1(device=dev)
    r, c = x.shape
    scale = (torch.tensor(448.0) / x.float().abs().max().cpu()).item()   # binary32 division, as the cast kernels do
    add("c1 per-tensor E4M3, scale given (fake_quantize mode 4)", x, 4, "fake_quantize", (r, c, 128, 128, scale, 4, 1), ref_ok=True)
    add("c1 per-tensor E4M3, self-contained (block_scaling ss 4)", x, 6, "fake_quantize_block_scaling", (r, c, 128, 128, 3e38, 4), ref_ok=True)
    add("c1 block scaling 128x128 (ss 1)", x, 6, "fake_quantize_block_scaling", (r, c, 128, 128, 3e38, 1), ref_ok=True, headline=False)
    add("c1 E8M3 with tensor scale (fake_quantize_e8mx)", x, 6, "fake_quantize_e8mx", (r, c, 128, 128, 3, 1), ref_ok=True)
    del x
    x = workloads.config2(device=dev)
    r, c = x.shape
    add("c2 per-row E4M3 single pass (fake_quantize mode 2, 1x8192)", x, 4, "fake_quantize", (r, c, 1, c, 0.0, 2, 1))
    add("c2 per-row E5M2 single pass (fake_quantize mode 3, 1x8192)", x, 4, "fake_quantize", (r, c, 1, c, 0.0, 3, 1), headline=False)
    # not for the reference arm: its channel path launches the 1024-thread reductions with the 64-thread
    # kernels' shared-memory size (fake_quantize.cu:2515-2522) and raised an illegal memory access at this size
    # strategies 2 and 3 scale a group by its own amax: one pass over the tensor (read + write)
    add("c2 per-row E4M3 pipeline (channel_scaling ss 3)", x, 4, "fake_quantize_channel_scaling", (r, c, 1, c, 3e38, 3))
    add("c2 per-column E4M3 pipeline (channel_scaling 8192x1, ss 1)", x, 6, "fake_quantize_channel_scaling", (r, c, r, 1, 3e38, 1))
    del x
    x = workloads.config3(device=dev)
    r, c = x.shape
    add("c3 MX 1x32 E8M0 E4M3 single pass (fake_quantize_mx)", x, 4, "fake_quantize_mx", (r, c, 32, 0, 2))
    add("c3 MX 1x32 E8M0 E2M3 single pass (fake_quantize_mx)", x, 4, "fake_quantize_mx", (r, c, 32, 3, 2), headline=False)
    add("c3 MX 1x32 real quantization, E4M3 codes + E8M0 scales (quantize_mx)", x, 3.03125, "quantize_mx", (r, c, 32, 0), headline=False)
    add("c3 MX 1x32 E4M3 pipeline (channel_scaling ss 2)", x, 4, "fake_quantize_channel_scaling", (r, c, 1, 32, 3e38, 2))
    del x
    x = workloads.config4(device=dev)
    r, c = x.shape
    if impl != "reference":
        amax_prev4 = x.float().abs().max().reshape(1)
        add("c4 block scaling 128x128, single pass with delayed amax (ss 1)", x, 4, "fake_quantize_block_scaling_delayed",
            (r, c, 128, 128, 3e38, 1, amax_prev4), headline=False)
        add("c4 block scaling 128x128, single pass, result also transposed (ss 1)", x, 6, "fake_quantize_block_scaling_delayed_t",
            (r, c, 128, 128, 3e38, 1, amax_prev4), headline=False)
        add("c4 real quantization, E4M3 bytes + float32 block scales (quantize_scaled ss 1)", x, 5, "quantize_scaled",
            (r, c, 128, 128, 1), headline=False)
    add("c4 MoR 128x128 relative-error criterion (mode 1)", x, 4, "fake_quantize", (r, c, 128, 128, 1e-15, 1, 1), ref_ok=True)
    add("c4 MoR 128x128 dynamic-range criterion (mode 101)", x, 4, "fake_quantize", (r, c, 128, 128, 1e-15, 101, 1), ref_ok=True, headline=False)
    add("c4 block scaling 128x128 pipeline (ss 1)", x, 6, "fake_quantize_block_scaling", (r, c, 128, 128, 3e38, 1), ref_ok=True)
    del x
    if impl != "reference" and not compact:
        x = workloads.config5_slab(0, device=dev)
        r, c = x.shape
        add("c5 float32 1 GiB slab block scaling 128x128 pipeline (ss 1)", x, 12, "fake_quantize_block_scaling", (r, c, 128, 128, THRESHOLD, 1))
        amax_prev = x.abs().max().reshape(1).float()
        add("c5 float32 1 GiB slab block scaling, single pass with delayed amax (ss 1)", x, 8,
            "fake_quantize_block_scaling_delayed", (r, c, 128, 128, THRESHOLD, 1, amax_prev))
        add("c5 float32 1 GiB slab per-tensor pipeline (ss 4)", x, 12, "fake_quantize_block_scaling", (r, c, 128, 128, THRESHOLD, 4))
        del x
    if out_path:
        os.makedirs(os.path.dirname(os.path.abspath(out_path)), exist_ok=True)
        with open(out_path, "w") as f:
            json.dump({"peak_GB/s": peak, "impl": impl, "results": results}, f, indent=1)
    return results


if __name__ == "__main__":
    sys.exit(main())
