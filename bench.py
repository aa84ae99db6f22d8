#!/usr/bin/env python
"""Benchmark of the dense-GEMM hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

One JSON line on stdout (rank 0).  A "step" is one GEMM over one set of synthetic operands.

Headline workload: bf16 x bf16 -> fp32 accumulate -> bf16, M = N = K = 8192, A row-major, B
column-major, alpha = 1, beta = 0, seeded N(0,1) / N(0,1) * K^-1/2 operands generated on the device
by gz_fill.  Three operand sets (384 MiB each, larger than the 126 MB L2) are rotated so that no
step finds its inputs in L2.  With N > 1 GPUs every rank runs the same slab on its own GPU (global
problem M = K = 8192, N = 8192 * N_gpus, B sharded by column blocks, A replicated, no collective on
the data path: weak scaling).  The timed region of K steps is measured `--repeats` times, each
bracketed by a barrier and a device synchronisation and each after a short idle pause and three
untimed steps, so that every repeat is the same measurement (K steps from a cool chip); `value` is
the median repeat (max over ranks), and the spread is reported beside the SM clock sampled during
each repeat.  What the chip sustains once the power limit sets the clock is the `sustained` leg.

Keys beyond the base contract:
  roofline            tensor-bound: achieved = 2MNK / mean kernel time of the median repeat (CUDA
                      events on the launching stream), peak = the measured cuBLAS bf16 burst;
                      traffic = DRAM bytes per launch from the committed ncu summary of exactly this
                      kernel configuration and workload (null when none matches)
  roofline_sustained  the same kernel in a seconds-long loop against the measured sustained peak
  sustained           seconds-long loops of own kernel and cuBLASLt: TFLOP/s, SM clock, watts
  partitioned         the column-partitioned configuration: ONE bf16 16384^3 problem, rank g
                      computing column block g of N over the N GPUs (strong scaling), each rank's
                      block checked against the CPU oracle on seeded rows and by a row-sum checksum
  e2e                 the headline metric through the host-operand entry points with pinned HOST
                      operands, host<->device copies inside the timed region (1 GPU:
                      gz_gemm_run_host; N GPUs: each rank uploads 1/N of the replicated A and the
                      slices are all-gathered over NVLink)
  configs             every benchmark configuration of the specification on one GPU, own kernel
                      beside cuBLASLt (device time per launch from CUDA-graph replays), each with its
                      roofline
  fused_epilogue      bf16 2048 x 14336 x 4096 with bias + GELU in the epilogue beside the plain GEMM
  timeline            where the time of a short launch goes (the kernel's own global-timer stamps)
  cublaslt            cuBLASLt on the headline operands in the same process, interleaved
  cpu_baseline        the CPU restatement of the reference's naive GEMM (oracle/), OpenMP over all
                      host cores, timed on a bounded row sample of the headline workload
  ksharded            (N > 1) K-sharded GEMM with the reduce-scatter fused into the epilogue, beside
                      the GEMM + NCCL reduce-scatter route
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

M = N = K = 8192
PART = 16384  # the column-partitioned configuration is PART^3
NOMINAL_BF16_TFLOPS = 2250.0
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
L2_BYTES = 126 << 20
METRIC = "bf16 GEMM TFLOP/s at M=N=K=8192"


def load_peaks():
    """Measured peaks of this pool (a JSON file beside this script, written by whoever measured
    them), else the stated fallback figures."""
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            d = json.loads(p.read_text())
            return d, "measured"
        except Exception:
            pass
    return dict(FALLBACK_PEAKS), "fallback"


def committed_traffic(kernel_config, m, n, k, in_name, out_name):
    """DRAM bytes per launch for (kernel configuration, problem) from the table of ncu captures under
    profiles/; None when the table has no row for exactly this kernel configuration and problem."""
    table = ROOT / "profiles" / "dram_traffic_per_launch.txt"
    if not table.exists():
        return None
    for line in table.read_text().splitlines():
        f = line.split()
        if len(f) >= 7 and not line.startswith("#"):
            try:
                if (int(f[0]), int(f[1]), int(f[2]), int(f[3]), f[4], f[5]) == (kernel_config, m, n, k, in_name, out_name):
                    return float(f[6])
            except ValueError:
                continue
    return None


class ClockSampler:
    """Samples SM clock, power and throttle reasons through NVML while timed regions run."""

    def __init__(self, index):
        self.index = index
        self.samples = []  # (time, sm_mhz, watts)
        self.reasons = set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        self.ok = False
        try:
            import pynvml
            self.nv = pynvml
            pynvml.nvmlInit()
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            self.ok = False

    def _loop(self):
        nv = self.nv
        names = {
            getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4): "sw_power_cap",
            getattr(nv, "nvmlClocksThrottleReasonHwPowerBrakeSlowdown", 0x80): "hw_power_brake",
        }
        while not self._stop.is_set():
            try:
                mhz = nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)
                try:
                    watts = nv.nvmlDeviceGetPowerUsage(self.h) / 1000.0
                except Exception:
                    watts = None
                self.samples.append((time.perf_counter(), mhz, watts))
                r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.002)

    def start(self):
        if self.ok:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()

    def median_mhz(self, t0=None, t1=None):
        s = sorted(m for (t, m, _) in self.samples if (t0 is None or t >= t0) and (t1 is None or t <= t1))
        return s[len(s) // 2] if s else None

    def median_watts(self, t0=None, t1=None):
        s = sorted(w for (t, _, w) in self.samples if w is not None and (t0 is None or t >= t0) and (t1 is None or t <= t1))
        return s[len(s) // 2] if s else None

    def stop(self):
        if self._thread:
            self._stop.set()
            self._thread.join()
        return {"sm_mhz": self.median_mhz(), "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


def physical_gpu_index(local_rank):
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_rank])
        except Exception:
            return local_rank
    return local_rank


def workload_name(gpus):
    base = ("bf16xbf16->fp32acc->bf16 GEMM M=N=K=8192, A row-major, B column-major, alpha=1 beta=0, "
            "3 rotating operand sets of 384 MiB (inputs larger than L2)")
    if gpus > 1:
        base += f"; x{gpus} GPUs: N sharded by column blocks (global N={N * gpus}), A replicated, no collective"
    return base


def config_dict(gpus):
    return {"workload": workload_name(gpus), "l2": "inputs larger than L2, 3 operand sets rotated"}


# ------------------------------------------------------------------ CPU baseline / reference arm
_CPU_DATA = {}


def cpu_reference_tflops(rows, threads=None):
    """Time the CPU oracle on `rows` rows of the headline workload; returns (TFLOP/s, seconds, cores)."""
    import numpy as np
    from oracle import cpu_oracle as orc
    # torch.distributed.run exports OMP_NUM_THREADS=1 to its ranks; the baseline is
    # defined on all cores this process may run on, so set the count explicitly.
    orc.lib().oracle_set_threads(threads or len(os.sched_getaffinity(0)))
    if "b" not in _CPU_DATA:
        rng = np.random.default_rng(1)
        # bf16 bit patterns of N(0,1) and N(0,1)/sqrt(K): top 16 bits of the fp32 values.
        _CPU_DATA["a"] = (rng.standard_normal((M, K), dtype=np.float32).view(np.uint32) >> 16).astype(np.uint16)
        _CPU_DATA["b"] = ((rng.standard_normal((N, K), dtype=np.float32) * K ** -0.5).view(np.uint32) >> 16).astype(np.uint16)
        orc.gemm_f64(orc.DT_BF16, orc.DT_BF16, _CPU_DATA["a"][:8], _CPU_DATA["b"], None, 8, N, K, b_col_major=True)
    a, b = _CPU_DATA["a"][:rows], _CPU_DATA["b"]
    t0 = time.perf_counter()
    orc.gemm_f64(orc.DT_BF16, orc.DT_BF16, a, b, None, rows, N, K, b_col_major=True)
    dt = time.perf_counter() - t0
    return 2.0 * rows * N * K / dt / 1e12, dt, orc.num_threads()


def run_reference(args, rank):
    """--impl reference: the reference's GEMM arithmetic on the host cores.

    AD2605/gemm-zoo has no CPU implementation of the path (its naive GEMMs are
    device kernels), so this arm times the CPU restatement in oracle/ (kind "port")."""
    if rank != 0:
        return
    rows = 256
    for _ in range(max(args.warmup, 0)):
        cpu_reference_tflops(32)
    ts, secs = [], 0.0
    for _ in range(args.steps):
        tf, dt, cores = cpu_reference_tflops(rows)
        ts.append(tf)
        secs += dt
    value = sum(ts) / len(ts)
    sample = f"{rows} of {M} rows of A per step (all {N} columns, K={K}); fp64 accumulation; scaled by 2*rows*N*K"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": secs / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": config_dict(args.gpus),
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------ helpers
class Ctx:
    """What every leg needs: torch, the binding, the device, the launching stream, the ranks."""

    def __init__(self, torch, dist, gz, dev, stream, rank, world, local_rank):
        self.torch, self.dist, self.gz, self.dev, self.stream = torch, dist, gz, dev, stream
        self.rank, self.world, self.local_rank = rank, world, local_rank

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize(self.dev)

    def max_over_ranks(self, values):
        t = self.torch.tensor(list(values), dtype=self.torch.float64, device=self.dev)
        if self.world > 1:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return [float(v) for v in t.tolist()]

    def all_ok(self, flag):
        t = self.torch.tensor([0 if flag else 1], dtype=self.torch.int32, device=self.dev)
        if self.world > 1:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.SUM)
        return int(t.item()) == 0


def timed_region(cx, fn, steps):
    """K steps between two events on the launching stream, a barrier and a synchronise either side.
    Returns (ms on this rank, host time at start, host time at end)."""
    torch = cx.torch
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    cx.barrier()
    t0 = time.perf_counter()
    e0.record(cx.stream)
    for i in range(steps):
        fn(i)
    e1.record(cx.stream)
    cx.barrier()
    t1 = time.perf_counter()
    return e0.elapsed_time(e1), t0, t1


# ------------------------------------------------------------------ the column-partitioned configuration
def partitioned_leg(cx, steps, warmup):
    """ONE bf16 PART^3 problem (A row-major, B column-major, N(0,1)/128, seed 5): rank g computes
    the column block gz_partition_columns gives it.  Aggregate = 2 * PART^3 / max-over-ranks time.
    Parity per rank: 16 seeded rows of its block against the CPU oracle (fp64 accumulation) and a
    row-sum checksum over the whole block."""
    import numpy as np
    torch, gz = cx.torch, cx.gz
    from gemm_zoo_b200.partition import PartitionedGemm
    from oracle import cpu_oracle as orc
    n = PART
    bf16 = torch.bfloat16
    a = torch.empty(n, n, dtype=bf16, device=cx.dev)
    b_full = torch.empty(n, n, dtype=bf16, device=cx.dev)  # column-major K x N: row j is column j of B
    gz.fill(a, 5, 1, 1, 1.0 / 128)
    gz.fill(b_full, 5, 2, 1, 1.0 / 128)  # every rank generates the same global B and keeps its block
    pg = PartitionedGemm(n, n, n, gz.DT_BF16, gz.DT_BF16, cx.rank, cx.world, cx.local_rank)
    lo, hi = pg.col_begin, pg.col_end
    b = b_full[lo:hi]
    d = torch.empty(n, hi - lo, dtype=bf16, device=cx.dev)
    info = pg.info()

    def step(_):
        pg(a, b, None, d, 1.0, 0.0, cx.stream)

    for i in range(warmup):
        step(i)
    ms, _, _ = timed_region(cx, step, steps)
    ms_max = cx.max_over_ranks([ms])[0]
    st, detail = pg.gemm.plan.device_status(cx.stream)
    # ---- parity of this rank's block
    rows = np.sort(np.random.default_rng(5 + cx.rank).choice(n, size=16, replace=False))
    ri = torch.from_numpy(rows).to(cx.dev)
    ah = orc.bits_of(a[ri])
    bh = orc.bits_of(b)
    orc.lib().oracle_set_threads(max(1, len(os.sched_getaffinity(0)) // max(1, cx.world)))
    ref = orc.gemm_f64(orc.DT_BF16, orc.DT_BF16, ah, bh, None, 16, hi - lo, n, b_col_major=True)
    scale = orc.abs_gemm(orc.DT_BF16, ah, bh, 16, hi - lo, n, b_col_major=True)
    got = d[ri].double().cpu().numpy()
    err = np.abs(got - ref)
    rows_ok = bool((err <= 2.0 ** -8 * np.abs(ref) + 2.0 ** -20 * scale + 1e-7).all()) and bool(np.isfinite(got).all())
    # sum_j D[i, j] == A[i, :] . (sum_j B[:, j]) over this rank's columns, every row
    bsum = b.double().sum(dim=0)
    want = torch.empty(n, dtype=torch.float64, device=cx.dev)
    wscale = torch.empty_like(want)
    babs = b.double().abs().sum(dim=0)
    for r0 in range(0, n, 2048):
        blk = a[r0:r0 + 2048].double()
        want[r0:r0 + 2048] = blk @ bsum
        wscale[r0:r0 + 2048] = blk.abs() @ babs
    gsum = d.double().sum(dim=1)
    dabs = d.double().abs().sum(dim=1)
    sum_ok = bool(((gsum - want).abs() <= 2.0 ** -9 * dabs + 2.0 ** -18 * wscale).all())
    ok = cx.all_ok(rows_ok and sum_ok and st == 0)
    flops = 2.0 * n * n * n
    out = {
        "workload": f"bf16 {n}^3, A row-major replicated, B column-major sharded by N over {cx.world} GPU(s) "
                    "(gz_partition_columns), D shards local, no collective; strong scaling",
        "value": flops / (ms_max / steps * 1e-3) / 1e12, "unit": "TFLOP/s", "scaling": "strong",
        "ms_per_step": ms_max / steps, "steps": steps, "warmup": warmup,
        "rank0_columns": [lo, hi], "rank0_kernel": {"config": info.config, "tile": [info.tile_m, info.tile_n, info.tile_k],
                                                    "grid": info.grid, "tiles": info.tiles},
        "parity": "ok" if ok else "FAILED",
        "parity_detail": {"oracle_rows_per_rank": 16, "rank0_max_err_over_scale": float((err / np.maximum(scale, 1e-30)).max()),
                          "row_sum_checksum": "all rows of every rank's block", "device_status": st},
        "gpu_launches": steps,
    }
    del a, b_full, b, d, want, wscale
    torch.cuda.empty_cache()
    return out


# ------------------------------------------------------------------ end to end with host operands
def e2e_leg(cx, gemm, A0, B0, steps):
    """The headline GEMM with pinned HOST operands, copies inside the timed region.  One GPU:
    gz_gemm_run_host.  N GPUs: rank g uploads rows g of N of the replicated A, the slices are
    all-gathered over NVLink, and only this rank's B block and D block cross its PCIe link."""
    torch, gz = cx.torch, cx.gz
    from gemm_zoo_b200 import partition
    bf16 = torch.bfloat16
    phys = physical_gpu_index(cx.local_rank)
    ha = partition.pin_near_gpu((M, K), bf16, phys)
    hb = partition.pin_near_gpu((N, K), bf16, phys)
    hd = partition.pin_near_gpu((M, N), bf16, phys)
    ha.copy_(A0)
    hb.copy_(B0)
    if cx.world == 1:
        run = lambda _: gemm.plan.run_host(ha, hb, None, hd, 1.0, 0.0, cx.stream)
        h2d = 2 * M * K * 2
        how = "gz_gemm_run_host: A, then B in column blocks up, D blocks down, GEMM per block (3 streams)"
    else:
        pg = partition.PartitionedHostGemm(M, N * cx.world, K, gz.DT_BF16, gz.DT_BF16, cx.rank, cx.world, cx.local_rank)
        # the global B is N*world columns; this rank's block is its own hb
        run = lambda _: pg(ha, hb, None, hd, 1.0, 0.0, cx.stream)
        h2d = pg.h2d_bytes
        how = (f"each rank uploads 1/{cx.world} of A's rows and its B block; A slices all-gathered over NVLink "
               "(NCCL) into local memory; D block down")
    for i in range(2):
        run(i)
    ms, _, _ = timed_region(cx, run, steps)
    ms_max = cx.max_over_ranks([ms])[0]
    d2h = M * N * 2
    # What the bus alone needs for one step's bytes: the same host buffers copied up and down at the
    # same time on two streams, no GEMM, all ranks at once.  The leg above cannot be faster than this.
    up = torch.empty(h2d // 2, dtype=bf16, device=cx.dev)
    down = torch.empty(M, N, dtype=bf16, device=cx.dev)
    s_up, s_down = torch.cuda.Stream(cx.dev), torch.cuda.Stream(cx.dev)
    flat_a, flat_b = ha.view(-1), hb.view(-1)
    na = h2d // 2 - flat_b.numel()

    def bus_only(_):
        s_up.wait_stream(cx.stream)
        s_down.wait_stream(cx.stream)
        with torch.cuda.stream(s_up):
            up[:na].copy_(flat_a[:na], non_blocking=True)
            up[na:].copy_(flat_b, non_blocking=True)
        with torch.cuda.stream(s_down):
            hd.copy_(down, non_blocking=True)
        cx.stream.wait_stream(s_up)
        cx.stream.wait_stream(s_down)

    bus_only(0)
    bus_ms, _, _ = timed_region(cx, bus_only, steps)
    bus_ms_max = cx.max_over_ranks([bus_ms])[0]
    run(0)  # leave the product in hd again for the caller's comparison
    flops = 2.0 * M * N * K
    # the result the host now holds is the product: compare a few entries with the device-resident run
    checksum = float(hd[:4, :4].float().abs().sum())
    per_rank_ms = ms / steps
    return {"value": cx.world * flops / (ms_max / steps * 1e-3) / 1e12, "unit": "TFLOP/s",
            "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": ms_max / steps, "steps": steps,
            "rank0_h2d_gbs": h2d / per_rank_ms / 1e6, "rank0_d2h_gbs": d2h / per_rank_ms / 1e6,
            "aggregate_pcie_gbs": cx.world * (h2d + d2h) / (ms_max / steps) / 1e6,
            "bus_only": {"ms_per_step": bus_ms_max / steps, "aggregate_gbs": cx.world * (h2d + d2h) / (bus_ms_max / steps) / 1e6,
                         "what": "the step's host-to-device and device-to-host bytes copied concurrently, no GEMM, all ranks at once"},
            "fraction_of_bus_only": (bus_ms_max / steps) / (ms_max / steps),
            "path": how, "result_checksum": checksum, "host_memory": "pinned, first touched on the GPU's NUMA node"}, hd


# ------------------------------------------------------------------ single-GPU extras
def _time_interleaved(torch, stream, fns, sets, reps=20, warm=3):
    """Median ms of each callable, reps interleaved so both see the same thermal state."""
    for f in fns:
        for i in range(warm):
            f(i % sets)
    torch.cuda.synchronize()
    times = [[] for _ in fns]
    for r in range(reps):
        for j, f in enumerate(fns):
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record(stream)
            f(r % sets)
            e.record(stream)
            times[j].append((s, e))
    torch.cuda.synchronize()
    out = []
    for ts in times:
        v = sorted(s.elapsed_time(e) for s, e in ts)
        out.append(v[len(v) // 2])
    return out


def compare_cublaslt(cx, A, B, D, gemm, flops):
    from gemm_zoo_b200.cublaslt import CublasLtGemm
    torch, gz, stream = cx.torch, cx.gz, cx.stream
    lt = CublasLtGemm(M, N, K, gz.DT_BF16, gz.DT_BF16, layout_b=gz.COL_MAJOR)
    best_ms, best_idx = None, 0
    for idx in range(min(lt.num_algos, 6)):
        lt.select(idx)
        try:
            ms, = _time_interleaved(torch, stream, [lambda i: lt(A[i], B[i], None, D, 1.0, 0.0, stream)], len(A), reps=5, warm=1)
        except Exception:
            continue
        if best_ms is None or ms < best_ms:
            best_ms, best_idx = ms, idx
    lt.select(best_idx)
    own_ms, lt_ms = _time_interleaved(
        torch, stream,
        [lambda i: gemm(A[i], B[i], None, D, 1.0, 0.0, stream), lambda i: lt(A[i], B[i], None, D, 1.0, 0.0, stream)],
        len(A))
    return lt, {"value": flops / lt_ms / 1e9, "unit": "TFLOP/s", "own_interleaved": flops / own_ms / 1e9,
                "ratio_own_over_cublaslt": lt_ms / own_ms, "algo_index": best_idx, "candidates": lt.num_algos}


def sustained_compare(cx, A, B, D, gemm, lt, flops, seconds, sampler):
    """Seconds-long back-to-back loops (the power-capped regime): TFLOP/s, median SM clock and
    board power over the second half of each loop, cuBLASLt then the own kernel."""
    torch, stream = cx.torch, cx.stream

    def loop(fn):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        n, t0 = 0, time.perf_counter()
        e0.record(stream)
        while time.perf_counter() - t0 < seconds:
            for _ in range(100):
                fn(n % len(A))
                n += 1
            torch.cuda.synchronize()
        e1.record(stream)
        torch.cuda.synchronize()
        t1 = time.perf_counter()
        ms = e0.elapsed_time(e1) / n
        mid = t0 + (t1 - t0) / 2
        return {"tflops": flops / ms / 1e9, "ms": ms, "launches": n, "sm_mhz": sampler.median_mhz(mid, t1),
                "watts": sampler.median_watts(mid, t1)}

    out = {"seconds_each": seconds}
    if lt is not None:
        out["cublaslt"] = loop(lambda i: lt(A[i], B[i], None, D, 1.0, 0.0, stream))
        time.sleep(0.5)
    out["own"] = loop(lambda i: gemm(A[i], B[i], None, D, 1.0, 0.0, stream))
    if lt is not None:
        out["ratio_own_over_cublaslt"] = out["own"]["tflops"] / out["cublaslt"]["tflops"]
    return out


# name, in, out, m, n, k, B column-major, alpha, beta, fill of A (dist, scale), fill of B (dist, scale)
def config_table(gz):
    return [
        ("c1_fp16_1024", gz.DT_F16, gz.DT_F16, 1024, 1024, 1024, True, 1, 0, (0, 1.0), (0, 1.0)),
        ("c5_bf16_m1", gz.DT_BF16, gz.DT_BF16, 1, 14336, 4096, True, 1, 0, (1, 1.0), (1, 0.02)),
        ("c5_bf16_m16", gz.DT_BF16, gz.DT_BF16, 16, 14336, 4096, True, 1, 0, (1, 1.0), (1, 0.02)),
        ("c5_bf16_m128", gz.DT_BF16, gz.DT_BF16, 128, 14336, 4096, True, 1, 0, (1, 1.0), (1, 0.02)),
        ("c2_bf16_4096_beta", gz.DT_BF16, gz.DT_BF16, 4096, 4096, 4096, True, 1, 0.5, (1, 4096 ** -0.5), (1, 4096 ** -0.5)),
        ("c5_bf16_m2048", gz.DT_BF16, gz.DT_BF16, 2048, 14336, 4096, True, 1, 0, (1, 1.0), (1, 0.02)),
        ("headline_bf16_8192", gz.DT_BF16, gz.DT_BF16, 8192, 8192, 8192, True, 1, 0, (1, 1.0), (1, 8192 ** -0.5)),
        ("fp16_8192", gz.DT_F16, gz.DT_F16, 8192, 8192, 8192, True, 1, 0, (1, 1.0), (1, 8192 ** -0.5)),
        ("c3_tf32_8192", gz.DT_F32, gz.DT_F32, 8192, 8192, 8192, False, 1, 0, (0, 1.0), (0, 1.0)),
        ("c4_s8_8192", gz.DT_S8, gz.DT_S32, 8192, 8192, 8192, True, 1, 0, (2, 1.0), (2, 1.0)),
        ("c5_bf16_m16384", gz.DT_BF16, gz.DT_BF16, 16384, 14336, 4096, True, 1, 0, (1, 1.0), (1, 0.02)),
        ("c5_bf16_16384_cube", gz.DT_BF16, gz.DT_BF16, 16384, 16384, 16384, True, 1, 0, (1, 1.0), (1, 1.0 / 128)),
        ("next_e4m3_8192_bf16out", gz.DT_E4M3, gz.DT_BF16, 8192, 8192, 8192, True, 1, 0, (1, 1.0), (1, 8192 ** -0.5)),
    ]


def graph_time_us(torch, calls, stream, reps):
    """Device time per launch: the launches of one pass are captured in a CUDA graph and replayed
    between two events, so the host's launch rate (a ctypes call costs more than the small
    configurations run) is not in the figure."""
    with torch.cuda.stream(stream):
        for f in calls:
            f()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            for f in calls:
                f()
        g.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            g.replay()
        e1.record()
        torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / (reps * len(calls))


def configs_leg(cx, peaks, peak_kind, reps=20):
    """Every configuration of the specification on one GPU, own kernel beside cuBLASLt (heuristic's
    first algorithm), alternating, better of two rounds each; operands rotate over enough sets that
    no launch finds them in L2."""
    from gemm_zoo_b200.cublaslt import CublasLtGemm
    torch, gz = cx.torch, cx.gz
    T = {gz.DT_F16: torch.float16, gz.DT_BF16: torch.bfloat16, gz.DT_F32: torch.float32, gz.DT_S8: torch.int8,
         gz.DT_S32: torch.int32, gz.DT_E4M3: torch.float8_e4m3fn}
    SIZE = {gz.DT_F16: 2, gz.DT_BF16: 2, gz.DT_F32: 4, gz.DT_S8: 1, gz.DT_S32: 4, gz.DT_E4M3: 1}
    bf16_peak = float(peaks.get("bf16_tflops", FALLBACK_PEAKS["bf16_tflops"]))
    hbm_peak = float(peaks.get("hbm_gbs", FALLBACK_PEAKS["hbm_gbs"]))
    stream = torch.cuda.Stream(cx.dev)
    table = {}
    for (name, it, ot, m, n, k, b_col, alpha, beta, fa, fb) in config_table(gz):
        try:
            op_bytes = (m * k + n * k) * SIZE[it]
            sets = 2 if op_bytes > 2 * L2_BYTES else max(1, min(8, (2 * L2_BYTES) // op_bytes + 1))
            A = [torch.empty(m, k, dtype=T[it], device=cx.dev) for _ in range(sets)]
            B = [torch.empty((n, k) if b_col else (k, n), dtype=T[it], device=cx.dev) for _ in range(sets)]
            for i in range(sets):
                gz.fill(A[i], 7, 2 * i, fa[0], fa[1])
                gz.fill(B[i], 7, 2 * i + 1, fb[0], fb[1])
            C = None
            if beta:
                C = torch.empty(m, n, dtype=T[ot], device=cx.dev)
                gz.fill(C, 7, 99, 1, 1.0)
            D = torch.empty(m, n, dtype=T[ot], device=cx.dev)
            layout_b = gz.COL_MAJOR if b_col else gz.ROW_MAJOR
            own = gz.Sm100Gemm(m, n, k, it, ot, layout_b=layout_b, device=cx.local_rank)
            lt = CublasLtGemm(m, n, k, it, ot, layout_b=layout_b)
            per_pass = max(sets, 4 if m * n * k < 2 ** 33 else sets)
            own_calls = [(lambda i: (lambda: own(A[i % sets], B[i % sets], C, D, alpha, beta, stream=stream)))(i)
                         for i in range(per_pass)]
            lt_calls = [(lambda i: (lambda: lt(A[i % sets], B[i % sets], C, D, alpha, beta, stream=stream)))(i)
                        for i in range(per_pass)]
            r = reps if m * n * k < 2 ** 40 else max(3, reps // 4)
            if m <= 128:
                time.sleep(1.5)  # the weight-streaming shapes are sensitive to the state the last one left
            rounds = [(graph_time_us(torch, own_calls, stream, r), graph_time_us(torch, lt_calls, stream, r))
                      for _ in range(2)]
            t_own = min(x[0] for x in rounds)
            t_lt = min(x[1] for x in rounds)
            st = own.plan.device_status(stream)[0]
            flops = 2.0 * m * n * k
            abytes = (m * k + n * k) * SIZE[it] + m * n * SIZE[ot] * (2 if beta else 1)
            info = own.info()
            e = {"m": m, "n": n, "k": k, "kernel_config": info.config, "grid": info.grid, "split_k": info.split_k,
                 "own_us": round(t_own, 2), "cublaslt_us": round(t_lt, 2), "own_over_cublaslt": round(t_lt / t_own, 3),
                 "own": round(flops / t_own / 1e6, 1), "cublaslt": round(flops / t_lt / 1e6, 1),
                 "unit": "TOPS" if it == gz.DT_S8 else "TFLOP/s", "device_status": st, "operand_sets": sets}
            if m <= 128:
                gbs = abytes / t_own / 1e3
                e["roofline"] = {"bound": "hbm", "achieved": round(gbs, 1), "peak": hbm_peak, "unit": "GB/s",
                                 "frac": round(gbs / hbm_peak, 3), "peak_source": f"{peak_kind} HBM copy"}
            else:
                scale = {gz.DT_F32: 0.5, gz.DT_S8: 2.0, gz.DT_E4M3: 2.0}.get(it, 1.0)
                tf = flops / t_own / 1e6
                label = f"{peak_kind} cuBLAS bf16 burst" + ("" if scale == 1.0 else f" x {scale} (nominal ratio to bf16)")
                e["roofline"] = {"bound": "tensor", "achieved": round(tf, 1), "peak": round(bf16_peak * scale, 1),
                                 "unit": e["unit"], "frac": round(tf / (bf16_peak * scale), 3), "peak_source": label}
            table[name] = e
            own.plan.destroy()
            lt.destroy()
            del A, B, C, D
            torch.cuda.empty_cache()
            time.sleep(0.5)
        except Exception as ex:  # one configuration failing must not lose the line
            table[name] = {"error": repr(ex)}
    return table


def fused_epilogue_leg(cx, reps=20):
    """bf16 2048 x 14336 x 4096 with bias + GELU in the epilogue beside the plain GEMM."""
    torch, gz = cx.torch, cx.gz
    m, n, k = 2048, 14336, 4096
    stream = torch.cuda.Stream(cx.dev)
    sets = 2
    A = [torch.empty(m, k, dtype=torch.bfloat16, device=cx.dev) for _ in range(sets)]
    B = [torch.empty(n, k, dtype=torch.bfloat16, device=cx.dev) for _ in range(sets)]
    for i in range(sets):
        gz.fill(A[i], 8, 2 * i, 1, 1.0)
        gz.fill(B[i], 8, 2 * i + 1, 1, 0.02)
    bias = torch.randn(n, device=cx.dev, dtype=torch.float32)
    D = torch.empty(m, n, dtype=torch.bfloat16, device=cx.dev)
    g = gz.Sm100Gemm(m, n, k, gz.DT_BF16, gz.DT_BF16, layout_b=gz.COL_MAJOR, device=cx.local_rank)
    plain = [(lambda i: (lambda: g(A[i], B[i], None, D, 1.0, 0.0, stream=stream)))(i) for i in range(sets)]
    fused = [(lambda i: (lambda: g.plan.run_ex(A[i], B[i], None, D, 1.0, 0.0, bias=bias, activation=gz.ACT_GELU,
                                                stream=stream)))(i) for i in range(sets)]
    t_plain = min(graph_time_us(torch, plain, stream, reps) for _ in range(2))
    t_fused = min(graph_time_us(torch, fused, stream, reps) for _ in range(2))
    return {"workload": "bf16 2048x14336x4096, B column-major", "plain_us": round(t_plain, 2),
            "bias_gelu_us": round(t_fused, 2), "fused_over_plain_time": round(t_fused / t_plain, 3)}


def timeline_leg(cx):
    """Where the time of a short launch goes.  Six launches of one problem back to back in one CUDA
    graph, each plan with the kernel's built-in timeline switched on (gz_gemm_plan_set_profile:
    global-timer stamps per CTA); reported per phase in microseconds, medians over launches 2..6:
      release     last CTA of the previous launch left -> this launch may touch global memory
                  (the launch itself and its set-up overlap the previous kernel: programmatic
                  dependent launch)
      first_data  -> the first operand stage has landed at the MMA warp (slowest CTA)
      main_loop   -> the last MMA is issued
      acc_ready   -> the last accumulator is complete and the epilogue warps have woken
      epilogue    -> the last output stores are issued
      tail        -> the last CTA has left
    The stamps cost a few clock reads per K block, so the sum runs a few percent above an
    uninstrumented launch."""
    torch, gz = cx.torch, cx.gz
    stream = torch.cuda.Stream(cx.dev)
    W = gz.PROFILE_WORDS_PER_CTA
    out = {}
    for name, (m, n, k, cfg) in {"bf16_1024_cubed": (1024, 1024, 1024, gz.CFG_1CTA_N64),
                                 "bf16_m16_n14336_k4096": (16, 14336, 4096, gz.CFG_SWAP_M16),
                                 "bf16_2048_cubed": (2048, 2048, 2048, gz.CFG_2CTA_N256)}.items():
        L = 6
        A = [torch.empty(m, k, dtype=torch.bfloat16, device=cx.dev) for _ in range(L)]
        B = [torch.empty(n, k, dtype=torch.bfloat16, device=cx.dev) for _ in range(L)]
        D = torch.empty(m, n, dtype=torch.bfloat16, device=cx.dev)
        for i in range(L):
            gz.fill(A[i], 9, 2 * i, 1, 1.0)
            gz.fill(B[i], 9, 2 * i + 1, 1, k ** -0.5)
        plans = [gz.Sm100Gemm(m, n, k, gz.DT_BF16, gz.DT_BF16, layout_b=gz.COL_MAJOR, config=cfg, device=cx.local_rank)
                 for _ in range(L)]
        grid = plans[0].info().grid
        bufs = [torch.zeros(W * grid, dtype=torch.int64, device=cx.dev) for _ in range(L)]
        for pl, b in zip(plans, bufs):
            pl.plan.set_profile(b)
        with torch.cuda.stream(stream):
            for _ in range(3):
                for i in range(L):
                    plans[i](A[i], B[i], None, D, 1.0, 0.0, stream=stream)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                for i in range(L):
                    plans[i](A[i], B[i], None, D, 1.0, 0.0, stream=stream)
            g.replay()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            g.replay()
            e1.record()
            torch.cuda.synchronize()
        ws = [b.cpu().view(grid, W)[:, 16:].double() for b in bufs]

        def col(w, i, fn):
            v = w[:, i]
            v = v[v > 0]  # CTAs that do not play the role (the second CTA of a pair) leave zeros
            return float(fn(v)) if len(v) else float("nan")

        phases = {"release": [], "first_data": [], "main_loop": [], "acc_ready": [], "epilogue": [], "tail": [],
                  "launch_to_launch": []}
        for i in range(1, L):
            prev_exit = col(ws[i - 1], 7, max)
            ready = col(ws[i], 1, max)
            first = col(ws[i], 2, max)
            mma_done = col(ws[i], 3, max)
            acc = col(ws[i], 4, max)
            stores = col(ws[i], 5, max)
            exit_ = col(ws[i], 7, max)
            phases["release"].append(ready - prev_exit)
            phases["first_data"].append(first - ready)
            phases["main_loop"].append(mma_done - first)
            phases["acc_ready"].append(acc - mma_done)
            phases["epilogue"].append(stores - acc)
            phases["tail"].append(exit_ - stores)
            phases["launch_to_launch"].append(exit_ - prev_exit)
        med = lambda v: round(sorted(v)[len(v) // 2] / 1e3, 2)
        out[name] = {"kernel_config": cfg, "grid": grid, "us": {k2: med(v) for k2, v in phases.items()},
                     "graph_us_per_launch": round(e0.elapsed_time(e1) * 1e3 / L, 2)}
        for pl in plans:
            pl.plan.destroy()
        del A, B, D, bufs
    return out


def ksharded_leg(cx, reps=20):
    """K-sharded GEMM (rank g holds A[:, K_g], B[K_g, :]) with the reduce-scatter fused into the
    epilogue (peer stores over NVLink), beside the GEMM + NCCL reduce-scatter route; both routes
    are compared with each other (they add the ranks' partial sums in different orders)."""
    torch, gz, dist = cx.torch, cx.gz, cx.dist
    from gemm_zoo_b200.ksharded import KShardedGemm
    m, n, k_local = 4096, 8192, 4096
    cols = n // cx.world
    a = torch.empty(m, k_local, dtype=torch.bfloat16, device=cx.dev)
    b = torch.empty(n, k_local, dtype=torch.bfloat16, device=cx.dev)  # column-major K x N slice
    gz.fill(a, 31 + cx.rank, 0, 1, 1.0)
    gz.fill(b, 31 + cx.rank, 1, 1, 0.02)
    d_fused = torch.empty(m, cols, dtype=torch.bfloat16, device=cx.dev)
    fused = KShardedGemm(m, n, k_local, gz.DT_BF16, gz.DT_BF16, layout_b=gz.COL_MAJOR)
    for _ in range(3):
        fused(a, b, None, d_fused, 1, 0, cx.stream)
    ms, _, _ = timed_region(cx, lambda i: fused(a, b, None, d_fused, 1, 0, cx.stream), reps)
    fused_ms = cx.max_over_ranks([ms])[0] / reps
    st = fused.plan.status(cx.stream)[0]
    # comparison route: fp32 partial product, transposing copy into column blocks, ncclReduceScatter, cast
    part = torch.empty(m, n, dtype=torch.float32, device=cx.dev)
    blocks = torch.empty(cx.world, m, cols, dtype=torch.float32, device=cx.dev)
    mine = torch.empty(m, cols, dtype=torch.float32, device=cx.dev)
    d_lib = torch.empty_like(d_fused)
    g = gz.Sm100Gemm(m, n, k_local, gz.DT_BF16, gz.DT_F32, layout_b=gz.COL_MAJOR, device=cx.local_rank)

    def library_route(_):
        g(a, b, None, part, 1.0, 0.0, cx.stream)
        blocks.copy_(part.view(m, cx.world, cols).permute(1, 0, 2))
        dist.reduce_scatter_tensor(mine, blocks)
        d_lib.copy_(mine)

    for _ in range(3):
        library_route(0)
    ms2, _, _ = timed_region(cx, library_route, reps)
    nccl_ms = cx.max_over_ranks([ms2])[0] / reps
    err = float((d_fused.float() - d_lib.float()).abs().max() / d_lib.float().abs().max())
    err = cx.max_over_ranks([err])[0]
    fused.close()
    flops = 2.0 * m * n * k_local
    link_bytes = m * n * 4 * (cx.world - 1) / cx.world
    floor_ms = max(flops / 1.6e15, link_bytes / 770e9) * 1e3
    return {"workload": f"bf16 {m}x{n}x{k_local} per rank, K sharded over {cx.world} GPUs", "fused_us": round(fused_ms * 1e3, 1),
            "gemm_plus_nccl_us": round(nccl_ms * 1e3, 1), "speedup": round(nccl_ms / fused_ms, 2),
            "roofline_us": round(floor_ms * 1e3, 1), "frac": round(floor_ms / fused_ms, 3), "device_status": st,
            "max_abs_diff_over_max_abs_between_routes": round(err, 5)}


# ------------------------------------------------------------------ main
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--repeats", type=int, default=10, help="how many times the timed region of --steps steps is measured")
    ap.add_argument("--cooldown", type=float, default=0.3, help="idle seconds between repeats")
    ap.add_argument("--no-die-order", action="store_true",
                    help="headline plan without the die-aware tile order (for before/after counter captures)")
    ap.add_argument("--impl", default="own", choices=["own", "reference"])
    ap.add_argument("--no-extras", action="store_true",
                    help="headline leg, partitioned leg and end-to-end leg only (same as --extras none)")
    ap.add_argument("--extras", default="all",
                    help="comma list of the optional legs: cublaslt,sustained,configs,fused,timeline,cpu,ksharded; all; none")
    ap.add_argument("--sustain", type=float, default=2.0,
                    help="seconds each of the seconds-long own / cuBLASLt loops (0 = skip)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "own" else args.warmup
    all_extras = {"cublaslt", "sustained", "configs", "fused", "timeline", "cpu", "ksharded"}
    extras = set() if (args.no_extras or args.extras == "none") else (
        all_extras if args.extras == "all" else set(args.extras.split(",")) & all_extras)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference(args, rank)
        return

    import torch
    import torch.distributed as dist
    import gemm_zoo_b200 as gz

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (no CPU fallback exists for the product path)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    gz.lib()  # fail loudly if the extension is missing
    stream = torch.cuda.current_stream(dev)
    cx = Ctx(torch, dist, gz, dev, stream, rank, world, local_rank)

    SETS = 3
    bf16 = torch.bfloat16
    A = [torch.empty(M, K, dtype=bf16, device=dev) for _ in range(SETS)]
    B = [torch.empty(N, K, dtype=bf16, device=dev) for _ in range(SETS)]  # column-major K x N
    D = torch.empty(M, N, dtype=bf16, device=dev)
    for i in range(SETS):
        # A is replicated across ranks (same seed); each rank owns its own column block of B.
        gz.fill(A[i], 1000 + i, 1, 1, 1.0)
        gz.fill(B[i], 2000 + i, 2 + rank, 1, K ** -0.5)
    gemm = gz.Sm100Gemm(M, N, K, gz.DT_BF16, gz.DT_BF16, layout_b=gz.COL_MAJOR, device=local_rank,
                        flags=gz.FLAG_NO_DIE_ORDER if args.no_die_order else 0)
    info = gemm.info()
    flops = 2.0 * M * N * K

    def step(i):
        gemm(A[i % SETS], B[i % SETS], None, D, 1.0, 0.0, stream)

    # ---- headline: `repeats` timed regions of `steps` steps
    for i in range(args.warmup):
        step(i)
    cx.barrier()
    sampler = ClockSampler(physical_gpu_index(local_rank))
    sampler.start()
    regions = []
    for r in range(max(1, args.repeats)):
        if r:
            # Every repeat measures the same thing as the first: K steps on a chip that was idle just
            # before (the seconds-long loop further down measures the power-capped regime).
            time.sleep(args.cooldown)
            for i in range(3):
                step(i)
        regions.append(timed_region(cx, step, args.steps))
    t_head_end = time.perf_counter()
    status, detail = gemm.plan.device_status(stream)
    if status != 0:
        raise SystemExit(f"device status {status} {detail}")
    ms_max = cx.max_over_ranks([r[0] for r in regions])
    order = sorted(range(len(ms_max)), key=lambda i: ms_max[i])
    med = order[len(order) // 2]
    ms_per_step = ms_max[med] / args.steps
    value = world * flops / (ms_per_step * 1e-3) / 1e12
    tf_of = lambda ms: world * flops / (ms / args.steps * 1e-3) / 1e12
    rep_mhz = [sampler.median_mhz(r[1], r[2]) for r in regions]
    repeats = {"n": len(regions), "tflops_median": value, "tflops_min": tf_of(max(ms_max)), "tflops_max": tf_of(min(ms_max)),
               "tflops": [round(tf_of(x), 1) for x in ms_max], "rank0_sm_mhz": rep_mhz,
               # time x clock: constant when the spread between repeats (and chips) is clock alone
               "rank0_ms_per_step_x_ghz": [round(regions[i][0] / args.steps * (rep_mhz[i] or 0) / 1e3, 4) for i in range(len(regions))]}
    head_clocks = {"sm_mhz": sampler.median_mhz(regions[0][1], t_head_end), "sm_max_mhz": sampler.max_mhz}

    # ---- the column-partitioned configuration (strong scaling) and the end-to-end leg
    part = partitioned_leg(cx, steps=max(3, min(args.steps, 10)), warmup=3)
    e2e_steps = max(3, min(args.steps, 10))
    e2e, hd = e2e_leg(cx, gemm, A[0], B[0], e2e_steps)
    # the host result of the end-to-end leg against the device-resident run on the same operands
    step(0)
    torch.cuda.synchronize(dev)
    e2e["matches_device_run"] = cx.all_ok(bool(torch.equal(hd.view(torch.int16), D.cpu().view(torch.int16))))

    peaks, peak_kind = load_peaks()
    peak_tf = float(peaks.get("bf16_tflops", FALLBACK_PEAKS["bf16_tflops"]))
    achieved = flops / (regions[med][0] / args.steps * 1e-3) / 1e12  # this rank's kernel, the median repeat
    line = {
        "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": config_dict(world),
        "kernel": {"config": info.config, "tile": [info.tile_m, info.tile_n, info.tile_k], "stages": info.stages,
                   "ctas_per_tile": info.ctas_per_tile, "grid": info.grid, "epilogue_tma": info.epilogue_tma,
                   "die_order": info.die_order},
        "repeats": repeats,
        "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak_tf, "unit": "TFLOP/s",
                     "frac": achieved / peak_tf,
                     "traffic": committed_traffic(info.config, M, N, K, "bf16", "bf16"),
                     "peak_source": f"{peak_kind} cuBLAS bf16 burst", "frac_of_nominal_2250": achieved / NOMINAL_BF16_TFLOPS,
                     "algorithmic_flops_per_launch": flops, "algorithmic_bytes_per_launch": 3 * M * N * 2},
        "partitioned": part,
        "e2e": e2e,
        "gpu_launches": args.steps,
    }

    if rank == 0 and world == 1 and extras & {"cublaslt", "sustained"}:
        lt = None
        try:
            lt, line["cublaslt"] = compare_cublaslt(cx, A, B, D, gemm, flops)
        except Exception as e:  # the comparator is optional equipment
            line["cublaslt"] = {"error": repr(e)}
        if args.sustain > 0 and "sustained" in extras:
            try:
                sus = sustained_compare(cx, A, B, D, gemm, lt, flops, args.sustain, sampler)
                line["sustained"] = sus
                sus_peak = float(peaks.get("bf16_tflops_sustained", FALLBACK_PEAKS["bf16_tflops_sustained"]))
                line["roofline_sustained"] = {"bound": "tensor", "achieved": sus["own"]["tflops"], "peak": sus_peak,
                                              "unit": "TFLOP/s", "frac": sus["own"]["tflops"] / sus_peak,
                                              "peak_source": f"{peak_kind} cuBLAS bf16, seconds-long loop under the power cap",
                                              "sm_mhz": sus["own"]["sm_mhz"], "watts": sus["own"]["watts"]}
            except Exception as e:
                line["sustained"] = {"error": repr(e)}
        if lt is not None:
            lt.destroy()
    clocks = sampler.stop()
    clocks.update(headline_sm_mhz=head_clocks["sm_mhz"])
    line["clocks"] = clocks
    del A, B, D
    torch.cuda.empty_cache()
    line["cpu_baseline"] = None
    if rank == 0 and world == 1:
        time.sleep(1.0)
        if "configs" in extras:
            try:
                line["configs"] = configs_leg(cx, peaks, peak_kind)
            except Exception as e:
                line["configs"] = {"error": repr(e)}
        if "fused" in extras:
            try:
                line["fused_epilogue"] = fused_epilogue_leg(cx)
            except Exception as e:
                line["fused_epilogue"] = {"error": repr(e)}
        if "timeline" in extras:
            try:
                line["timeline"] = timeline_leg(cx)
            except Exception as e:
                line["timeline"] = {"error": repr(e)}
        if "cpu" in extras:
            # a bounded sample of 10-20 s of CPU work: a 256-row probe sets the row count
            tf0, _, _ = cpu_reference_tflops(256)
            rows = int(max(256, min(M, 15.0 * tf0 * 1e12 / (2.0 * N * K)) // 256 * 256))
            tf, dt, cores = cpu_reference_tflops(rows)
            line["cpu_baseline"] = {"value": tf, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                                    "sample": f"{rows} of {M} rows of A (all columns, full K), {dt:.1f} s, fp64 accumulation"}
    if world > 1 and "ksharded" in extras:
        try:
            line["ksharded"] = ksharded_leg(cx)
        except Exception as e:
            line["ksharded"] = {"error": repr(e)}
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
