"""The N-column partition on two CPU ranks (gloo): each rank takes the column block
gz_partition_columns gives it (B sharded, A replicated, no data-path collective),
computes its shard with the CPU oracle, and the gathered shards equal the
unpartitioned result bit for bit.  This is the host logic `bench.py --gpus N` and
the multi-GPU tests run, minus the GPU."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent
M, N, K = 24, 200, 64


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, str(ROOT))
    import gemm_zoo_b200 as gz
    from oracle import cpu_oracle as orc
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    rng = np.random.default_rng(0)                      # A replicated: same seed on every rank
    a = rng.integers(-128, 128, (M, K), dtype=np.int8)
    b_full = np.random.default_rng(1).integers(-128, 128, (N, K), dtype=np.int8)  # column-major K x N
    lo, hi = gz.partition_columns(N, world, rank, 8)
    shard = orc.gemm_s8(a, b_full[lo:hi], None, M, hi - lo, K, b_col_major=True)
    # verification only: gather the shards on rank 0 (the data path itself has no collective)
    sizes = [torch.zeros(2, dtype=torch.int64) for _ in range(world)]
    dist.all_gather(sizes, torch.tensor([lo, hi]))
    padded = torch.zeros(M, N, dtype=torch.int32)
    padded[:, lo:hi] = torch.from_numpy(shard)
    dist.all_reduce(padded)                             # disjoint column blocks: the sum is the concatenation
    if rank == 0:
        full = orc.gemm_s8(a, b_full, None, M, N, K, b_col_major=True)
        ok = np.array_equal(padded.numpy(), full)
        bounds = [tuple(int(v) for v in s) for s in sizes]
        contiguous = all(bounds[i][1] == bounds[i + 1][0] for i in range(world - 1))
        (Path(out_dir) / "result.txt").write_text(f"{int(ok)} {int(contiguous)} {bounds[0][0]} {bounds[-1][1]}")
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_column_partition(tmp_path):
    port = _free_port()
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    ok, contiguous, first, last = (tmp_path / "result.txt").read_text().split()
    assert ok == "1" and contiguous == "1" and int(first) == 0 and int(last) == N
