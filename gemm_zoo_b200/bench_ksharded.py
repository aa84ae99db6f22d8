"""Timing of the K-sharded GEMM (fused push reduce-scatter) beside the library route.

Run with one process per GPU on one node:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node G --master-addr 127.0.0.1 \
        --master-port 29500 -m gemm_zoo_b200.bench_ksharded

Per shape rank 0 prints one JSON line:
  fused_us      KShardedGemm: the GEMM's epilogue stores fp32 partial sums straight into the owners'
                memory, then the flag kernel and the reduce kernel (alpha, cast) run
  nccl_route_us the same result the library way: local GEMM into an fp32 partial matrix, a
                transposing copy into contiguous column blocks, NCCL reduce-scatter, cast
  local_gemm_us the local GEMM of the library route alone (what both routes have to pay)
Times are CUDA-event means over `--reps` back-to-back calls, maximum over ranks.
Every rank multiplies its own K slice (synthetic N(0,1) x N(0,0.02) operands); the two routes are
compared against each other (they add the ranks' partial sums in different orders, so agreement
is to bf16 rounding, not bitwise).
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

import gemm_zoo_b200 as gz
from gemm_zoo_b200 import ksharded

SHAPES = [(1, 14336, 4096), (16, 14336, 4096), (128, 14336, 4096), (1024, 8192, 4096), (4096, 8192, 4096)]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    args = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl")
    dev = torch.device("cuda", local)

    def timed(fn):
        for _ in range(args.warmup):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / args.reps * 1e3], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return round(t.item(), 2)

    for (m, n, k_local) in SHAPES:
        if n % (32 * world):
            continue
        cols = n // world
        a = torch.empty(m, k_local, dtype=torch.bfloat16, device=dev)
        b = torch.empty(n, k_local, dtype=torch.bfloat16, device=dev)  # column-major K x N slice
        gz.fill(a, 1 + rank, 0, 1, 1.0)
        gz.fill(b, 1 + rank, 1, 1, 0.02)
        d_fused = torch.empty(m, cols, dtype=torch.bfloat16, device=dev)
        fused = ksharded.KShardedGemm(m, n, k_local, gz.DT_BF16, gz.DT_BF16, layout_b=gz.COL_MAJOR)
        t_fused = timed(lambda: fused(a, b, None, d_fused, 1, 0))
        status = fused.plan.status()[0]

        part = torch.empty(m, n, dtype=torch.float32, device=dev)
        blocks = torch.empty(world, m, cols, dtype=torch.float32, device=dev)
        mine = torch.empty(m, cols, dtype=torch.float32, device=dev)
        d_lib = torch.empty_like(d_fused)
        local_gemm = gz.Sm100Gemm(m, n, k_local, gz.DT_BF16, gz.DT_F32, layout_b=gz.COL_MAJOR, device=local)

        def library_route():
            local_gemm(a, b, None, part, 1, 0)
            blocks.copy_(part.view(m, world, cols).permute(1, 0, 2))
            dist.reduce_scatter_tensor(mine, blocks)
            d_lib.copy_(mine)

        t_lib = timed(library_route)
        t_gemm = timed(lambda: local_gemm(a, b, None, part, 1, 0))
        err = (d_fused.float() - d_lib.float()).abs().max()
        ref = d_lib.float().abs().max()
        dist.all_reduce(err, op=dist.ReduceOp.MAX)
        dist.all_reduce(ref, op=dist.ReduceOp.MAX)
        if rank == 0:
            print(json.dumps({"m": m, "n": n, "k_local": k_local, "world": world, "dtype": "bf16",
                              "fused_us": t_fused, "nccl_route_us": t_lib, "local_gemm_us": t_gemm,
                              "speedup_over_nccl_route": round(t_lib / t_fused, 2), "device_status": status,
                              "max_abs_diff_over_max_abs": round((err / ref).item(), 5)}), flush=True)
        fused.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
