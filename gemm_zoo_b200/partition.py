"""Column-partitioned GEMM over the GPUs of one node, one process per GPU.

Output columns are independent (D[:, J] = alpha * A * B[:, J] + beta * C[:, J]), so GPU g owns the
column block `partition_columns(N, G, g)`: B, C and D are sharded, A is replicated, and the GEMM
itself needs no collective.  The reference harness is single-GPU (it hard-codes device 0,
nvidia/utils/benchmark.cuh:20); this is the multi-GPU form of the same call.

`PartitionedGemm`      operands already in device memory: one plan for this rank's column block.
`PartitionedHostGemm`  operands in HOST memory.  A replicated operand must not cross the host's
                       PCIe fabric once per GPU: rank g uploads only rows `row_slice(M, G, g)` of A
                       over its own link and the slices are all-gathered GPU to GPU (NCCL over
                       NVLink) into every GPU's LOCAL copy of A; then this rank's column blocks
                       of B stream up; the kernels read local memory only.  Per rank and
                       call the bus carries |A|/G + |B shard| up and |D shard| down.

`pin_near_gpu` allocates pinned host memory on the NUMA node the GPU hangs off, so that its DMA
does not cross the socket interconnect.
"""
from __future__ import annotations

import os

from . import api


def row_slice(m: int, world: int, rank: int):
    """Rows of the replicated operand that `rank` uploads: equal blocks, the remainder spread
    over the first ranks (the same rule as gz_partition_columns with align 1)."""
    return api.partition_columns(m, world, rank, 1)


def gather_rows(full, m: int, world: int, rank: int, group=None):
    """All-gather over dim 0 of `full` (m rows): on entry rank r holds valid rows row_slice(m, world, r)
    only, on return every rank holds all of them.  In place; `full` may be a CUDA tensor (NCCL) or a
    CPU tensor (gloo).  Equal slices use one all-gather; ragged ones a broadcast per rank."""
    import torch.distributed as dist
    if world == 1:
        return full
    lo, hi = row_slice(m, world, rank)
    if m % world == 0:
        dist.all_gather_into_tensor(full[:m], full[lo:hi], group=group)
    else:
        for r in range(world):
            a, b = row_slice(m, world, r)
            if b > a:
                dist.broadcast(full[a:b], src=dist.get_global_rank(group, r) if group is not None else r, group=group)
    return full


def gpu_cpu_affinity(physical_index: int):
    """CPU ids NVML reports as local to the GPU (empty set when NVML cannot say)."""
    try:
        import pynvml
        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(physical_index)
        words = pynvml.nvmlDeviceGetCpuAffinity(h, (os.cpu_count() + 63) // 64)
        cpus = {64 * w + b for w, word in enumerate(words) for b in range(64) if (word >> b) & 1}
        return cpus & os.sched_getaffinity(0)
    except Exception:
        return set()


def pin_near_gpu(shape, dtype, physical_index: int):
    """Pinned host tensor whose pages are first touched by a thread running on the GPU's own NUMA
    node (Linux places a page where it is first touched).  Falls back to a plain pinned tensor."""
    import torch
    before = os.sched_getaffinity(0)
    near = gpu_cpu_affinity(physical_index)
    try:
        if near:
            os.sched_setaffinity(0, near)
        t = torch.empty(shape, dtype=dtype).pin_memory()
        t.view(torch.uint8).zero_() if t.dtype in (torch.float8_e4m3fn, torch.float8_e5m2) else t.zero_()
    finally:
        os.sched_setaffinity(0, before)
    return t


class PartitionedGemm:
    """This rank's column block of D = alpha * A * B + beta * C, operands in device memory."""

    def __init__(self, m, n_global, k, in_dtype, out_dtype, rank, world, device, layout_a=api.ROW_MAJOR,
                 layout_b=api.COL_MAJOR, align=None, ldd=0, ldc=0, ldb=0):
        self.m, self.n_global, self.k, self.rank, self.world = m, n_global, k, rank, world
        # Column-block boundaries are multiples of `align` so that every shard keeps TMA's 16-byte rule.
        self.col_begin, self.col_end = api.partition_columns(n_global, world, rank, align or 16)
        self.n_local = self.col_end - self.col_begin
        self.gemm = None
        if self.n_local > 0:
            self.gemm = api.Sm100Gemm(m, self.n_local, k, in_dtype, out_dtype, layout_a=layout_a, layout_b=layout_b,
                                      device=device, ldd=ldd, ldc=ldc, ldb=ldb)

    def __call__(self, a, b_shard, c_shard, d_shard, alpha, beta, stream=None):
        if self.gemm is not None:
            self.gemm(a, b_shard, c_shard, d_shard, alpha, beta, stream)

    def info(self):
        return self.gemm.info() if self.gemm is not None else None


class PartitionedHostGemm(PartitionedGemm):
    """The same column block with HOST operands (see the module docstring).  B is column-major
    (a column block is contiguous), A row-major."""

    def __init__(self, m, n_global, k, in_dtype, out_dtype, rank, world, device, group=None):
        import torch
        super().__init__(m, n_global, k, in_dtype, out_dtype, rank, world, device)
        self.group = group
        self.dev = torch.device("cuda", device)
        tin = {v: kk for kk, v in api_torch_dtypes().items()}[self.gemm.desc.in_type]
        self.a_dev = torch.empty(m, k, dtype=tin, device=self.dev)  # this GPU's local copy of A
        self.side = torch.cuda.Stream(self.dev)                     # upload + all-gather of A
        self.row_begin, self.row_end = row_slice(m, world, rank)
        self.h2d_bytes = ((self.row_end - self.row_begin) * k + self.n_local * k) * self.a_dev.element_size()

    def __call__(self, a_host, b_host_shard, c_host_shard, d_host_shard, alpha, beta, stream=None):
        """a_host: the whole of A in pinned host memory (only this rank's row slice is read);
        b/c/d_host_shard: this rank's column blocks.  Returns when D's block is in d_host_shard."""
        import torch
        stream = stream or torch.cuda.current_stream(self.dev)
        self.side.wait_stream(stream)
        with torch.cuda.stream(self.side):
            lo, hi = self.row_begin, self.row_end
            if hi > lo:
                self.a_dev[lo:hi].copy_(a_host[lo:hi], non_blocking=True)
            gather_rows(self.a_dev, self.m, self.world, self.rank, self.group)
        # Everything below is ordered after A on `stream`: the slice had the upload direction of the
        # link to itself, the gather ran over NVLink, and now the blocks of B follow.
        stream.wait_stream(self.side)
        self.gemm.plan.run_host(self.a_dev, b_host_shard, c_host_shard, d_host_shard, alpha, beta, stream,
                                a_on_device=True)


def api_torch_dtypes():
    import torch
    return {torch.float16: api.DT_F16, torch.bfloat16: api.DT_BF16, torch.float32: api.DT_F32,
            torch.int8: api.DT_S8, torch.int32: api.DT_S32, torch.float8_e4m3fn: api.DT_E4M3,
            torch.float8_e5m2: api.DT_E5M2}
