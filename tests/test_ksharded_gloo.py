"""The K-sharded GEMM's host logic on two CPU ranks (gloo): every rank takes the K slice
`ksharded.k_slice` gives it, forms its partial product with the CPU oracle, the partials are
summed across ranks, and rank r keeps column block r.  The result equals the unsharded oracle
(bit for bit for s8, whose int32 sums do not depend on the order).  This is what
`KShardedGemm` computes, minus the GPU and with gloo's all-reduce standing in for the push."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent
M, N, K = 16, 128, 320


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, str(ROOT))
    from gemm_zoo_b200 import ksharded
    from oracle import cpu_oracle as orc
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    a = np.random.default_rng(0).integers(-128, 128, (M, K), dtype=np.int8)
    b = np.random.default_rng(1).integers(-128, 128, (N, K), dtype=np.int8)  # column-major K x N
    k0, k1 = ksharded.k_slice(K, world, rank, 64)
    part = orc.gemm_s8(np.ascontiguousarray(a[:, k0:k1]), np.ascontiguousarray(b[:, k0:k1]), None, M, N, k1 - k0,
                       b_col_major=True)
    total = torch.from_numpy(part.astype(np.int32))
    dist.all_reduce(total)
    cols = N // world
    mine = total[:, rank * cols:(rank + 1) * cols].numpy()
    full = orc.gemm_s8(a, b, None, M, N, K, b_col_major=True)
    ok = np.array_equal(mine, full[:, rank * cols:(rank + 1) * cols])
    spans = [torch.zeros(2, dtype=torch.int64) for _ in range(world)]
    dist.all_gather(spans, torch.tensor([k0, k1]))
    flags = torch.tensor([int(ok)])
    dist.all_reduce(flags)
    if rank == 0:
        b_ = [tuple(int(v) for v in s) for s in spans]
        covered = b_[0][0] == 0 and b_[-1][1] == K and all(b_[i][1] == b_[i + 1][0] for i in range(world - 1))
        (Path(out_dir) / "result.txt").write_text(f"{int(flags.item())} {int(covered)}")
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_k_partition(tmp_path):
    port = _free_port()
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    ok, covered = (tmp_path / "result.txt").read_text().split()
    assert ok == "2" and covered == "1"
