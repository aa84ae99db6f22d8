"""Every BASELINE configuration on one GPU: own kernel beside cuBLASLt, with its roofline.

    python -m gemm_zoo_b200.bench_configs [--reps 20] [--only NAME]

One JSON line per configuration.  Timing (own and cuBLASLt alternate, two rounds, the better round of each is
reported): the launches of one pass over `sets` rotating operand
sets (enough of them that no launch finds its operands in L2) are captured in a CUDA graph and the
graph is replayed `--reps` times between two CUDA events, so the figure is device time per launch
without the host's launch rate in it (a Python ctypes call costs 5-8 us, more than the small
configurations run).  The same graph-and-replay is done for cuBLASLt (heuristic's first algorithm).

Roofline per configuration: tensor-bound shapes are held against the measured cuBLAS bf16 burst
of MEASURED_PEAKS.json (scaled by the nominal ratio for tf32 / int8, labelled as such); the
skinny weight-streaming shapes (M <= 128) against the measured HBM copy bandwidth, with
algorithmic bytes = A + B + D.
"""
from __future__ import annotations

import argparse
import json
import time
from pathlib import Path

import torch

import gemm_zoo_b200 as gz
from gemm_zoo_b200.cublaslt import CublasLtGemm

ROOT = Path(__file__).resolve().parent.parent
L2_BYTES = 126 << 20

T = {gz.DT_F16: torch.float16, gz.DT_BF16: torch.bfloat16, gz.DT_F32: torch.float32, gz.DT_S8: torch.int8,
     gz.DT_S32: torch.int32}
SIZE = {gz.DT_F16: 2, gz.DT_BF16: 2, gz.DT_F32: 4, gz.DT_S8: 1, gz.DT_S32: 4}

# name, in, out, m, n, k, B column-major, alpha, beta, fill of A (dist, scale), fill of B (dist, scale)
CONFIGS = [
    ("headline_bf16_8192", gz.DT_BF16, gz.DT_BF16, 8192, 8192, 8192, True, 1, 0, (1, 1.0), (1, 8192 ** -0.5)),
    ("c1_fp16_1024", gz.DT_F16, gz.DT_F16, 1024, 1024, 1024, True, 1, 0, (0, 1.0), (0, 1.0)),
    ("c2_bf16_4096_beta", gz.DT_BF16, gz.DT_BF16, 4096, 4096, 4096, True, 1, 0.5, (1, 4096 ** -0.5), (1, 4096 ** -0.5)),
    ("c3_tf32_8192", gz.DT_F32, gz.DT_F32, 8192, 8192, 8192, False, 1, 0, (0, 1.0), (0, 1.0)),
    ("c4_s8_8192", gz.DT_S8, gz.DT_S32, 8192, 8192, 8192, True, 1, 0, (2, 1.0), (2, 1.0)),
    ("c5_bf16_m1", gz.DT_BF16, gz.DT_BF16, 1, 14336, 4096, True, 1, 0, (1, 1.0), (1, 0.02)),
    ("c5_bf16_m16", gz.DT_BF16, gz.DT_BF16, 16, 14336, 4096, True, 1, 0, (1, 1.0), (1, 0.02)),
    ("c5_bf16_m128", gz.DT_BF16, gz.DT_BF16, 128, 14336, 4096, True, 1, 0, (1, 1.0), (1, 0.02)),
    ("c5_bf16_m2048", gz.DT_BF16, gz.DT_BF16, 2048, 14336, 4096, True, 1, 0, (1, 1.0), (1, 0.02)),
    ("c5_bf16_m16384", gz.DT_BF16, gz.DT_BF16, 16384, 14336, 4096, True, 1, 0, (1, 1.0), (1, 0.02)),
    ("c5_bf16_16384_cube", gz.DT_BF16, gz.DT_BF16, 16384, 16384, 16384, True, 1, 0, (1, 1.0), (1, 1.0 / 128)),
]


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["bf16_tflops"]), float(d["hbm_gbs"]), "measured"
    return 1590.0, 6650.0, "fallback"


def graph_time_us(calls, stream, reps):
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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--only", default=None)
    ap.add_argument("--pause", type=float, default=3.0, help="seconds of idle time between configurations")
    args = ap.parse_args()
    bf16_peak, hbm_peak, src = peaks()
    stream = torch.cuda.Stream()
    for (name, it, ot, m, n, k, b_col, alpha, beta, fa, fb) in CONFIGS:
        if args.only and args.only != name:
            continue
        op_bytes = (m * k + n * k) * SIZE[it]
        sets = max(1, min(8, (2 * L2_BYTES) // op_bytes + 1))
        if op_bytes > 2 * L2_BYTES:
            sets = 2
        A = [torch.empty(m, k, dtype=T[it], device="cuda") for _ in range(sets)]
        B = [torch.empty((n, k) if b_col else (k, n), dtype=T[it], device="cuda") for _ in range(sets)]
        for i in range(sets):
            gz.fill(A[i], 7, 2 * i, fa[0], fa[1])
            gz.fill(B[i], 7, 2 * i + 1, fb[0], fb[1])
        C = None
        if beta:
            C = torch.empty(m, n, dtype=T[ot], device="cuda")
            gz.fill(C, 7, 99, 1, 1.0)
        D = torch.empty(m, n, dtype=T[ot], device="cuda")
        layout_b = gz.COL_MAJOR if b_col else gz.ROW_MAJOR
        own = gz.Sm100Gemm(m, n, k, it, ot, layout_b=layout_b)
        lt = CublasLtGemm(m, n, k, it, ot, layout_b=layout_b)
        per_pass = max(sets, 4 if m * n * k < 2 ** 33 else sets)
        own_calls = [(lambda i: (lambda: own(A[i % sets], B[i % sets], C, D, alpha, beta, stream=stream)))(i)
                     for i in range(per_pass)]
        lt_calls = [(lambda i: (lambda: lt(A[i % sets], B[i % sets], C, D, alpha, beta, stream=stream)))(i)
                    for i in range(per_pass)]
        reps = args.reps if m * n * k < 2 ** 40 else max(3, args.reps // 4)
        # alternate the two so that neither always runs on the warmer chip; keep the better round
        rounds = [(graph_time_us(own_calls, stream, reps), graph_time_us(lt_calls, stream, reps)) for _ in range(2)]
        t_own = min(r[0] for r in rounds)
        t_lt = min(r[1] for r in rounds)
        st = own.plan.device_status(stream)[0]
        flops = 2.0 * m * n * k
        abytes = (m * k + n * k) * SIZE[it] + m * n * SIZE[ot] * (2 if beta else 1)
        info = own.info()
        line = {"config": name, "m": m, "n": n, "k": k, "kernel_config": info.config, "grid": info.grid,
                "split_k": info.split_k, "own_us": round(t_own, 2), "cublaslt_us": round(t_lt, 2),
                "own_over_cublaslt_speed": round(t_lt / t_own, 3), "device_status": st,
                "own_tflops": round(flops / t_own / 1e6, 1), "cublaslt_tflops": round(flops / t_lt / 1e6, 1),
                "operand_sets": sets}
        if m <= 128:
            gbs = abytes / t_own / 1e3
            line["roofline"] = {"bound": "hbm", "achieved": round(gbs, 1), "peak": hbm_peak, "unit": "GB/s",
                                "frac": round(gbs / hbm_peak, 3), "peak_source": f"{src} HBM copy"}
        else:
            scale = {gz.DT_F32: 0.5, gz.DT_S8: 2.0}.get(it, 1.0)
            tf = flops / t_own / 1e6
            label = f"{src} cuBLAS bf16 burst" + ("" if scale == 1.0 else f" x {scale} (nominal ratio to bf16)")
            line["roofline"] = {"bound": "tensor", "achieved": round(tf, 1), "peak": round(bf16_peak * scale, 1),
                                "unit": "TFLOP/s" if it != gz.DT_S8 else "TOPS",
                                "frac": round(tf / (bf16_peak * scale), 3), "peak_source": label}
        print(json.dumps(line), flush=True)
        del A, B, C, D, own, lt
        torch.cuda.empty_cache()
        time.sleep(args.pause)  # let the chip cool: the seconds-scale configurations leave it at its power limit


if __name__ == "__main__":
    main()
