#!/usr/bin/env python
"""Benchmark of the dense-GEMM hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

One JSON line on stdout (rank 0).  A "step" is one GEMM over one set of
synthetic operands.

Workload (N = 1): bf16 x bf16 -> fp32 accumulate -> bf16, M = N = K = 8192, A
row-major, B column-major, alpha = 1, beta = 0, seeded N(0,1) / N(0,1)*K^-1/2
operands generated on the device by gz_fill.  Three operand sets (384 MiB each,
larger than the 126 MB L2) are rotated so that no step finds its inputs in L2.
With N > 1 GPUs every rank runs the same slab on its own GPU: the global problem
is M = K = 8192, N = 8192 * N_gpus with B sharded by column blocks and A
replicated, no collective on the data path (weak scaling).

Keys beyond the base contract:
  roofline      tensor-bound: achieved = 2MNK / mean kernel time (CUDA events on the
                launching stream), peak = measured cuBLAS bf16 burst (MEASURED_PEAKS.json)
  cpu_baseline  the CPU restatement of the reference's naive GEMM (oracle/), OpenMP over
                all host cores, timed on a bounded row sample of the same workload
  e2e           same metric through gz_gemm_run_host with pinned HOST operands: H2D of A
                and B and D2H of D inside the timed region
  cublaslt      cuBLASLt on the same operands in the same process, interleaved
  sustained     (--sustain S) seconds-long loops of own kernel and cuBLASLt: TFLOP/s, SM clock, watts
  other_dtypes  fp16 / tf32 / s8 / fp8 at 8192^3 and the bf16 4096^3 beta=0.5 config (own | cuBLASLt)
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
NOMINAL_BF16_TFLOPS = 2250.0
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the bench kernel
# (profiles/sm100_gemm_bf16_8192_512x256.md); algorithmic bytes are 3 * 128 MiB.
NCU_TRAFFIC_BYTES_PER_LAUNCH = 1.037e9


def load_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            d = json.loads(p.read_text())
            return d, "measured"
        except Exception:
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""

    def __init__(self, index):
        self.index = index
        self.samples = []
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
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
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

    def stop(self):
        if self._thread:
            self._stop.set()
            self._thread.join()
        s = sorted(self.samples)
        return {"sm_mhz": (s[len(s) // 2] if s else None), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(s)}


def physical_gpu_index(local_rank):
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_rank])
        except Exception:
            return local_rank
    return local_rank


_CPU_DATA = {}


def cpu_reference_tflops(rows, threads=None):
    """Time the CPU oracle on `rows` rows of the bench workload; returns (TFLOP/s, seconds, cores)."""
    import numpy as np
    from oracle import cpu_oracle as orc
    # torch.distributed.run exports OMP_NUM_THREADS=1 to its ranks; the baseline is
    # defined on all cores this process may run on, so set the count explicitly.
    orc.lib().oracle_set_threads(threads or len(os.sched_getaffinity(0)))
    if "b" not in _CPU_DATA:
        rng = np.random.default_rng(1)
        # bf16 bit patterns of N(0,1) and N(0,1)/sqrt(K): top 16 bits of the fp32 values.
        _CPU_DATA["a"] = (rng.standard_normal((2048, K), dtype=np.float32).view(np.uint32) >> 16).astype(np.uint16)
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
        "impl": "reference", "metric": "bf16 GEMM TFLOP/s at M=N=K=8192", "value": value, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": secs / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": workload_name(args.gpus), "sample": sample},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_name(gpus):
    base = ("bf16xbf16->fp32acc->bf16 GEMM M=N=K=8192, A row-major, B column-major, alpha=1 beta=0, "
            "3 rotating operand sets of 384 MiB (inputs larger than L2)")
    if gpus > 1:
        base += f"; x{gpus} GPUs: N sharded by column blocks (global N={N * gpus}), A replicated, no collective"
    return base


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="own", choices=["own", "reference"])
    ap.add_argument("--no-extras", action="store_true", help="skip cuBLASLt / other dtypes / CPU baseline")
    ap.add_argument("--sustain", type=float, default=0.0,
                    help="also run own kernel and cuBLASLt back to back for this many seconds each and "
                         "report throughput, SM clock and board power under the power cap")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "own" else args.warmup

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

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    gz.lib()  # fail loudly if the extension is missing
    SETS = 3
    bf16 = torch.bfloat16
    A = [torch.empty(M, K, dtype=bf16, device=dev) for _ in range(SETS)]
    B = [torch.empty(N, K, dtype=bf16, device=dev) for _ in range(SETS)]  # column-major K x N
    D = torch.empty(M, N, dtype=bf16, device=dev)
    for i in range(SETS):
        # A is replicated across ranks (same seed); each rank owns its own column block of B.
        gz.fill(A[i], 1000 + i, 1, 1, 1.0)
        gz.fill(B[i], 2000 + i, 2 + rank, 1, K ** -0.5)
    gemm = gz.Sm100Gemm(M, N, K, gz.DT_BF16, gz.DT_BF16, layout_b=gz.COL_MAJOR, device=local_rank)
    info = gemm.info()
    stream = torch.cuda.current_stream(dev)
    flops = 2.0 * M * N * K

    def step(i):
        gemm(A[i % SETS], B[i % SETS], None, D, 1.0, 0.0, stream)

    for i in range(args.warmup):
        step(i)
    barrier()
    sampler = ClockSampler(physical_gpu_index(local_rank))
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record(stream)
    for i in range(args.steps):
        step(i)
    e1.record(stream)
    barrier()
    clocks = sampler.stop()
    ms_total = e0.elapsed_time(e1)
    status, detail = gemm.plan.device_status(stream)
    if status != 0:
        raise SystemExit(f"device status {status} {detail}")
    t = torch.tensor([ms_total], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_total_max = float(t.item())
    ms_per_step = ms_total_max / args.steps
    value = world * flops / (ms_per_step * 1e-3) / 1e12

    # ---- end to end through the C ABI with host operands (pinned), copies inside the timed region
    ha = torch.empty(M, K, dtype=bf16).pin_memory()
    hb = torch.empty(N, K, dtype=bf16).pin_memory()
    hd = torch.empty(M, N, dtype=bf16).pin_memory()
    ha.copy_(A[0])
    hb.copy_(B[0])
    e2e_steps = max(3, min(args.steps, 10))
    for _ in range(2):
        gemm.plan.run_host(ha, hb, None, hd, 1.0, 0.0, stream)
    barrier()
    e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2.record(stream)
    for _ in range(e2e_steps):
        gemm.plan.run_host(ha, hb, None, hd, 1.0, 0.0, stream)
    e3.record(stream)
    barrier()
    t2 = torch.tensor([e2.elapsed_time(e3)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t2, op=dist.ReduceOp.MAX)
    e2e_ms = float(t2.item()) / e2e_steps
    e2e_value = world * flops / (e2e_ms * 1e-3) / 1e12
    checksum = float(hd[:4, :4].float().abs().sum())  # the D2H result is read on the host

    peaks, peak_kind = load_peaks()
    peak_tf = float(peaks.get("bf16_tflops", FALLBACK_PEAKS["bf16_tflops"]))
    achieved = flops / (ms_total / args.steps * 1e-3) / 1e12  # this rank's kernel
    line = {
        "metric": "bf16 GEMM TFLOP/s at M=N=K=8192", "value": value, "unit": "TFLOP/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": workload_name(world), "l2": "inputs larger than L2, 3 operand sets rotated",
                   "kernel": {"config": info.config, "tile": [info.tile_m, info.tile_n, info.tile_k],
                              "stages": info.stages, "ctas_per_tile": info.ctas_per_tile, "grid": info.grid,
                              "epilogue_tma": info.epilogue_tma}},
        "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak_tf, "unit": "TFLOP/s",
                     "frac": achieved / peak_tf, "traffic": NCU_TRAFFIC_BYTES_PER_LAUNCH,
                     "peak_source": f"{peak_kind} cuBLAS bf16 burst", "frac_of_nominal_2250": achieved / NOMINAL_BF16_TFLOPS,
                     "algorithmic_flops_per_launch": flops,
                     "algorithmic_bytes_per_launch": 3 * M * N * 2},
        "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": 2 * M * K * 2,
                "d2h_bytes_per_step": M * N * 2, "ms_per_step": e2e_ms, "steps": e2e_steps,
                "result_checksum": checksum},
        "gpu_launches": args.steps,
        "clocks": clocks,
    }

    if rank == 0 and world == 1 and args.sustain > 0:
        line["sustained"] = sustained_compare(gz, torch, dev, stream, A, B, D, gemm, flops, args.sustain,
                                              physical_gpu_index(local_rank))
    if rank == 0 and world == 1 and not args.no_extras:
        try:
            line["cublaslt"] = compare_cublaslt(gz, torch, dev, stream, A, B, D, gemm, flops)
        except Exception as e:  # the comparator is optional equipment
            line["cublaslt"] = {"error": repr(e)}
        try:
            line["other_dtypes"] = other_dtypes(gz, torch, dev, stream)
        except Exception as e:
            line["other_dtypes"] = {"error": repr(e)}
        rows = 2048 if (os.cpu_count() or 1) >= 32 else 512
        tf, dt, cores = cpu_reference_tflops(rows)
        line["cpu_baseline"] = {"value": tf, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                                "sample": f"{rows} of {M} rows of A (all columns, full K), {dt:.1f} s, fp64 accumulation"}
    elif rank == 0:
        line["cpu_baseline"] = None
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        print(json.dumps(line), flush=True)


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


def sustained_compare(gz, torch, dev, stream, A, B, D, gemm, flops, seconds, nvml_index):
    """Seconds-long back-to-back loops (the power-capped regime): TFLOP/s, median SM clock and board
    power over the second half of each loop, own kernel then cuBLASLt, twice."""
    import pynvml
    from gemm_zoo_b200.cublaslt import CublasLtGemm
    pynvml.nvmlInit()
    h = pynvml.nvmlDeviceGetHandleByIndex(nvml_index)
    lt = CublasLtGemm(M, N, K, gz.DT_BF16, gz.DT_BF16, layout_b=gz.COL_MAJOR)

    def loop(fn):
        samples, stop = [], threading.Event()

        def sample():
            while not stop.is_set():
                samples.append((pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM),
                                pynvml.nvmlDeviceGetPowerUsage(h) / 1000.0))
                time.sleep(0.02)
        th = threading.Thread(target=sample, daemon=True)
        th.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        n, t0 = 0, time.time()
        e0.record(stream)
        while time.time() - t0 < seconds:
            for _ in range(100):
                fn(n % len(A))
                n += 1
            torch.cuda.synchronize()
        e1.record(stream)
        torch.cuda.synchronize()
        stop.set()
        th.join()
        ms = e0.elapsed_time(e1) / n
        half = samples[len(samples) // 2:] or [(0, 0.0)]
        clk = sorted(x[0] for x in half)[len(half) // 2]
        pw = sorted(x[1] for x in half)[len(half) // 2]
        return {"tflops": flops / ms / 1e9, "ms": ms, "sm_mhz": clk, "watts": pw}

    out = {"seconds_each": seconds, "own": [], "cublaslt": []}
    for _ in range(2):
        out["own"].append(loop(lambda i: gemm(A[i], B[i], None, D, 1.0, 0.0, stream)))
        time.sleep(1.0)
        out["cublaslt"].append(loop(lambda i: lt(A[i], B[i], None, D, 1.0, 0.0, stream)))
        time.sleep(1.0)
    lt.destroy()
    return out


def compare_cublaslt(gz, torch, dev, stream, A, B, D, gemm, flops):
    from gemm_zoo_b200.cublaslt import CublasLtGemm
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
    lt.destroy()
    return {"value": flops / lt_ms / 1e9, "unit": "TFLOP/s", "own_interleaved": flops / own_ms / 1e9,
            "ratio_own_over_cublaslt": lt_ms / own_ms, "algo_index": best_idx, "candidates": lt.num_algos}


def other_dtypes(gz, torch, dev, stream):
    """The remaining BASELINE configurations, own kernel and cuBLASLt interleaved."""
    from gemm_zoo_b200.cublaslt import CublasLtGemm
    res = {}
    cases = [
        ("fp16_8192", gz.DT_F16, gz.DT_F16, torch.float16, torch.float16, 8192, gz.COL_MAJOR, 1.0, 0.0),
        ("tf32_8192_rowrow", gz.DT_F32, gz.DT_F32, torch.float32, torch.float32, 8192, gz.ROW_MAJOR, 1.0, 0.0),
        ("s8_8192", gz.DT_S8, gz.DT_S32, torch.int8, torch.int32, 8192, gz.COL_MAJOR, 1, 0),
        ("bf16_4096_beta0.5", gz.DT_BF16, gz.DT_BF16, torch.bfloat16, torch.bfloat16, 4096, gz.COL_MAJOR, 1.0, 0.5),
        ("e4m3_8192_bf16out", gz.DT_E4M3, gz.DT_BF16, torch.float8_e4m3fn, torch.bfloat16, 8192, gz.COL_MAJOR, 1.0, 0.0),
    ]
    for name, it, ot, tin, tout, sz, lb, alpha, beta in cases:
        sets = 2 if sz == 8192 else 4
        a = [torch.empty(sz, sz, dtype=tin, device=dev) for _ in range(sets)]
        b = [torch.empty(sz, sz, dtype=tin, device=dev) for _ in range(sets)]
        c = torch.empty(sz, sz, dtype=tout, device=dev)
        d = torch.empty(sz, sz, dtype=tout, device=dev)
        for i in range(sets):
            if it == gz.DT_S8:
                gz.fill(a[i], 3, 10 + i, 2)
                gz.fill(b[i], 3, 20 + i, 2)
            else:
                gz.fill(a[i], 3, 10 + i, 1, 1.0)
                gz.fill(b[i], 3, 20 + i, 1, sz ** -0.5)
        gz.fill(c, 3, 30, 2 if it == gz.DT_S8 else 1, 1.0)
        own = gz.Sm100Gemm(sz, sz, sz, it, ot, layout_b=lb, device=dev.index or 0)
        cc = c if beta != 0 else None
        fns = [lambda i: own(a[i], b[i], cc, d, alpha, beta, stream)]
        lt = None
        try:
            lt = CublasLtGemm(sz, sz, sz, it, ot, layout_b=lb)
            fns.append(lambda i: lt(a[i], b[i], cc, d, alpha, beta, stream))
        except Exception:
            lt = None
        ms = _time_interleaved(torch, stream, fns, sets, reps=10)
        fl = 2.0 * sz ** 3
        entry = {"own": fl / ms[0] / 1e9, "unit": "TOPS" if it == gz.DT_S8 else "TFLOP/s",
                 "config": own.info().config}
        if lt is not None:
            entry["cublaslt"] = fl / ms[1] / 1e9
            lt.destroy()
        res[name] = entry
        own.plan.destroy()
        del a, b, c, d
        torch.cuda.empty_cache()
    return res


if __name__ == "__main__":
    main()
