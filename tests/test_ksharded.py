"""K-sharded GEMM with the reduce-scatter fused into the epilogue (include/gemmzoo/ksharded.h).

On one GPU the ranks are emulated in one process: every virtual rank has its own workspace and
plan, all pushes are issued before any reduce (kernels that wait on one another must not be
separate launches on one GPU, so no reduce is launched before the flags it waits for are set).
With two or more GPUs the real thing runs as one process per GPU with CUDA IPC workspaces.
Inputs are small integers, so partial sums are exact and the result must equal the unsharded
GEMM bit for bit whatever the order of addition.
"""
import os
import socket
import sys
from pathlib import Path

import pytest
import torch

import gemm_zoo_b200 as gz
from gemm_zoo_b200 import api, ksharded

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent

TORCH = {gz.DT_BF16: torch.bfloat16, gz.DT_F16: torch.float16, gz.DT_F32: torch.float32, gz.DT_S8: torch.int8,
         gz.DT_S32: torch.int32}


def _ints(shape, dtype, seed, lo=-3, hi=4, device="cuda:0"):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return torch.randint(lo, hi, shape, generator=g).to(TORCH[dtype]).to(device)


def _expected(a, b_nk, c_full, alpha, beta, out_t):
    """alpha * A @ B + beta * C with exact integer arithmetic (fp64 holds these sums exactly)."""
    r = alpha * (a.double().cpu() @ b_nk.double().cpu().t())
    if c_full is not None:
        r = r + beta * c_full.double().cpu()
    return r.to(TORCH[out_t])


@pytest.mark.parametrize("in_t,out_t,m,n,k,world,alpha,beta", [
    (gz.DT_BF16, gz.DT_BF16, 16, 1024, 2048, 2, 1, 0),      # skinny: swapped tiles, split-K inside each rank
    (gz.DT_BF16, gz.DT_BF16, 16, 2048, 4096, 4, 2, -1),
    (gz.DT_BF16, gz.DT_F32, 100, 512, 1024, 2, 1, 1),       # ragged M on 128-row tiles
    (gz.DT_F16, gz.DT_F16, 384, 1024, 768, 2, 1, 0),        # 128x128 / 256x256 tiles, direct stores
    (gz.DT_F32, gz.DT_F32, 256, 512, 512, 4, 1, 0),         # tf32
    (gz.DT_S8, gz.DT_S32, 300, 768, 2048, 3, 3, -2),        # int32 partial sums, world not a power of two
    (gz.DT_BF16, gz.DT_BF16, 1, 14336, 4096, 8, 1, 0),      # the inference-shaped skinny problem over 8 ranks
])
def test_emulated_ranks_match_unsharded(in_t, out_t, m, n, k, world, alpha, beta):
    lo, hi = (-128, 128) if in_t == gz.DT_S8 else (-3, 4)
    a = _ints((m, k), in_t, 1, lo, hi)
    b = _ints((n, k), in_t, 2, lo, hi)            # column-major K x N
    c = _ints((m, n), out_t, 3, -5, 6) if beta else None
    cols = n // world
    align = 128 if in_t == gz.DT_S8 else 64
    spaces, plans, outs, keep = [], [], [], []
    for r in range(world):
        k0, k1 = ksharded.k_slice(k, world, r, align)
        d = ksharded.make_desc(in_t, out_t, m, n, k1 - k0, world, r, layout_b=gz.COL_MAJOR, lda=k, ldb=k)
        if r == 0:
            nbytes = ksharded.workspace_bytes(d)
            spaces = [ksharded.SharedWorkspace(nbytes) for _ in range(world)]
        plans.append((ksharded.KsPlan(d, [s.ptr for s in spaces]), k0))
    for rep in range(3):                          # the two slot sets alternate: run more than twice
        for plan, k0 in plans:
            plan.push(a.data_ptr() + k0 * a.element_size(), b.data_ptr() + k0 * b.element_size())
        outs = []
        for r, (plan, _) in enumerate(plans):
            d_r = torch.full((m, cols), 77, dtype=TORCH[out_t], device="cuda:0")
            c_r = c[:, r * cols:(r + 1) * cols].contiguous() if c is not None else None
            keep.append(c_r)
            plan.reduce(c_r, d_r, alpha, beta)
            outs.append(d_r)
        torch.cuda.synchronize()
        for plan, _ in plans:
            assert plan.status()[0] == api.GZ_OK
        got = torch.cat([o.cpu() for o in outs], dim=1)
        want = _expected(a, b, c, alpha, beta, out_t)
        assert torch.equal(got, want), (rep, (got.double() - want.double()).abs().max())
    for plan, _ in plans:
        plan.destroy()
    for s in spaces:
        s.free()


def test_missing_peer_times_out_and_context_survives():
    """A rank whose peer never pushes: the reduce kernel's bounded wait gives up, the status says
    which rank was awaited, nothing hangs, and the same plans work once the peer shows up."""
    m, n, k, world = 16, 512, 1024, 2
    a = _ints((m, k), gz.DT_BF16, 1)
    b = _ints((n, k), gz.DT_BF16, 2)
    descs = [ksharded.make_desc(gz.DT_BF16, gz.DT_BF16, m, n, k // 2, world, r, layout_b=gz.COL_MAJOR, lda=k, ldb=k,
                                wait_limit_ns=2_000_000) for r in range(world)]
    spaces = [ksharded.SharedWorkspace(ksharded.workspace_bytes(descs[0])) for _ in range(world)]
    plans = [ksharded.KsPlan(d, [s.ptr for s in spaces]) for d in descs]
    d0 = torch.zeros(m, n // 2, dtype=torch.bfloat16, device="cuda:0")
    plans[0].push(a, b)
    plans[0].reduce(None, d0, 1, 0)               # rank 1 has not pushed: flag [1] stays at 0
    st, detail = plans[0].status()
    assert st == api.GZ_ERR_DEVICE_TIMEOUT and detail[0] == ksharded.WAIT_PEER_FLAG and detail[2] == 1
    assert plans[0].status()[0] == api.GZ_OK      # cleared by the read
    # the peer arrives (same epoch), and the reduce of that epoch now completes
    off = (k // 2) * a.element_size()
    plans[1].push(a.data_ptr() + off, b.data_ptr() + off)
    d1 = torch.zeros_like(d0)
    plans[0].reduce(None, d0, 1, 0)
    plans[1].reduce(None, d1, 1, 0)
    torch.cuda.synchronize()
    assert plans[0].status()[0] == api.GZ_OK and plans[1].status()[0] == api.GZ_OK
    want = _expected(a, b, None, 1, 0, gz.DT_BF16)
    assert torch.equal(torch.cat([d0.cpu(), d1.cpu()], dim=1), want)
    for p in plans:
        p.destroy()
    for s in spaces:
        s.free()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, str(ROOT))
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)   # host plumbing only: handles and barriers
    dev = f"cuda:{rank}"
    ok = True
    for (in_t, out_t, m, n, k) in ((gz.DT_BF16, gz.DT_BF16, 16, 14336, 4096), (gz.DT_S8, gz.DT_S32, 512, 2048, 4096)):
        lo, hi = (-128, 128) if in_t == gz.DT_S8 else (-3, 4)
        a = _ints((m, k), in_t, 1, lo, hi, dev)
        b = _ints((n, k), in_t, 2, lo, hi, dev)
        k0, k1 = ksharded.k_slice(k, world, rank, 128)
        g = ksharded.KShardedGemm(m, n, k1 - k0, in_t, out_t, layout_b=gz.COL_MAJOR, lda=k, ldb=k)
        cols = n // world
        d = torch.zeros(m, cols, dtype=TORCH[out_t], device=dev)
        for _ in range(3):
            g(a.data_ptr() + k0 * a.element_size(), b.data_ptr() + k0 * b.element_size(), None, d, 1, 0)
        torch.cuda.synchronize()
        ok = ok and g.plan.status()[0] == api.GZ_OK
        want = _expected(a, b, None, 1, 0, out_t)[:, rank * cols:(rank + 1) * cols]
        ok = ok and torch.equal(d.cpu(), want)
        g.close()
    # A peer that misses a step: rank 1 stays out of one push (it is between steps, nothing of its
    # own in flight).  The other ranks' reduce kernels give up after their bounded wait and report
    # which rank they were waiting for; the contexts stay usable, and once rank 1 has caught up the
    # same epoch reduces correctly on every rank.
    m, n, k = 16, 2048, 2048
    a = _ints((m, k), gz.DT_BF16, 5, device=dev)
    b = _ints((n, k), gz.DT_BF16, 6, device=dev)
    k0, k1 = ksharded.k_slice(k, world, rank, 128)
    g = ksharded.KShardedGemm(m, n, k1 - k0, gz.DT_BF16, gz.DT_BF16, layout_b=gz.COL_MAJOR, lda=k, ldb=k,
                              wait_limit_ns=20_000_000)
    cols = n // world
    d = torch.zeros(m, cols, dtype=torch.bfloat16, device=dev)
    pa, pb = a.data_ptr() + k0 * 2, b.data_ptr() + k0 * 2
    if rank != 1:
        g.plan.push(pa, pb)
        g.plan.reduce(None, d, 1, 0)
        st, detail = g.plan.status()
        ok = ok and st == api.GZ_ERR_DEVICE_TIMEOUT and detail[0] == ksharded.WAIT_PEER_FLAG and detail[2] == 1
    dist.barrier()
    if rank == 1:
        g.plan.push(pa, pb)
        torch.cuda.synchronize()
    dist.barrier()
    g.plan.reduce(None, d, 1, 0)
    torch.cuda.synchronize()
    ok = ok and g.plan.status()[0] == api.GZ_OK
    want = _expected(a, b, None, 1, 0, gz.DT_BF16)[:, rank * cols:(rank + 1) * cols]
    ok = ok and torch.equal(d.cpu(), want)
    g.close()
    flag = torch.tensor([int(ok)])
    dist.all_reduce(flag)
    if rank == 0:
        (Path(out_dir) / "result.txt").write_text(str(int(flag.item())))
    dist.barrier()
    dist.destroy_process_group()


def test_real_ranks_over_ipc(tmp_path):
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    import torch.multiprocessing as mp
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert (tmp_path / "result.txt").read_text() == str(world)
