"""Host logic of the column-partitioned GEMM with host operands, on two CPU ranks (gloo): every
rank holds only its own row slice of the replicated operand A, `gather_rows` completes it on
every rank (the step that runs over NVLink on GPUs), for row counts that divide evenly and that
do not; the row slices tile [0, M) exactly; and the per-rank upload accounting adds up to one
copy of A plus B."""
import os
import socket
import sys
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, str(ROOT))
    from gemm_zoo_b200 import partition
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    ok = True
    for m in (64, 37, 3, 1):  # even split, ragged split, fewer rows than... and a single row
        k = 16
        truth = torch.arange(m * k, dtype=torch.float32).view(m, k)
        lo, hi = partition.row_slice(m, world, rank)
        mine = torch.full((m, k), -1.0)
        mine[lo:hi] = truth[lo:hi]          # only this rank's slice is valid on entry
        partition.gather_rows(mine, m, world, rank)
        ok = ok and torch.equal(mine, truth)
    if rank == 0:
        (Path(out_dir) / "ok.txt").write_text(str(int(ok)))
    dist.barrier()
    dist.destroy_process_group()


def test_gather_rows_completes_the_replicated_operand(tmp_path):
    port = _free_port()
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert (tmp_path / "ok.txt").read_text() == "1"


@pytest.mark.parametrize("m,world", [(8192, 8), (8192, 2), (37, 4), (3, 8), (1, 2)])
def test_row_slices_tile_the_rows_exactly(m, world):
    from gemm_zoo_b200 import partition
    bounds = [partition.row_slice(m, world, r) for r in range(world)]
    assert bounds[0][0] == 0 and bounds[-1][1] == m
    assert all(bounds[i][1] == bounds[i + 1][0] for i in range(world - 1))
    sizes = [hi - lo for lo, hi in bounds]
    assert max(sizes) - min(sizes) <= 1
