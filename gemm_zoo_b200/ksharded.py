"""Host side of the K-sharded GEMM (include/gemmzoo/ksharded.h).

One process per GPU.  ``torch.distributed`` is plumbing only: it carries the 64-byte CUDA IPC
handles of the ranks' workspaces at construction, and (for the comparison path) the NCCL
reduce-scatter.  The data path of :class:`KShardedGemm` is the library's own: the GEMM epilogue
pushes partial sums to the owners' memory over NVLink, a flag kernel and a reduce kernel finish.

The reference (AD2605/gemm-zoo) is single-GPU and has no counterpart.
"""
from __future__ import annotations

import ctypes as C

from . import api
from .api import GZ_OK, GzError, _ptr, _scalar, _stream_handle, lib

MAX_WORLD = 8
IPC_HANDLE_BYTES = 64
WAIT_PEER_FLAG = 16  # detail[0] of a timed-out reduce

EXPORTED_SYMBOLS = [
    "gz_ks_workspace_bytes", "gz_ipc_alloc", "gz_ipc_open", "gz_ipc_close", "gz_ipc_free",
    "gz_ks_plan_create", "gz_ks_plan_destroy", "gz_ks_run", "gz_ks_push", "gz_ks_reduce", "gz_ks_status",
]


class KsDesc(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32), ("in_type", C.c_int32), ("out_type", C.c_int32),
        ("layout_a", C.c_int32), ("layout_b", C.c_int32),
        ("m", C.c_int64), ("n", C.c_int64), ("k_local", C.c_int64), ("lda", C.c_int64), ("ldb", C.c_int64),
        ("world", C.c_int32), ("rank", C.c_int32), ("device", C.c_int32), ("reserved", C.c_int32),
        ("wait_limit_ns", C.c_uint64),
    ]


_bound = False


def _bind():
    global _bound
    L = lib()
    if _bound:
        return L
    vp, i64 = C.c_void_p, C.c_int64
    L.gz_ks_workspace_bytes.argtypes = [C.POINTER(KsDesc), C.POINTER(C.c_size_t)]
    L.gz_ipc_alloc.argtypes = [C.c_size_t, C.POINTER(vp), C.c_char_p]
    L.gz_ipc_open.argtypes = [C.c_char_p, C.POINTER(vp)]
    L.gz_ipc_close.argtypes = [vp]
    L.gz_ipc_free.argtypes = [vp]
    L.gz_ks_plan_create.argtypes = [C.POINTER(vp), C.POINTER(KsDesc), C.POINTER(vp)]
    L.gz_ks_plan_destroy.argtypes = [vp]
    L.gz_ks_run.argtypes = [vp, vp, vp, vp, vp, i64, i64, vp, vp, vp]
    L.gz_ks_push.argtypes = [vp, vp, vp, vp]
    L.gz_ks_reduce.argtypes = [vp, vp, vp, i64, i64, vp, vp, vp]
    L.gz_ks_status.argtypes = [vp, vp, C.POINTER(C.c_uint32 * 4)]
    for name in EXPORTED_SYMBOLS:
        getattr(L, name).restype = C.c_int
    _bound = True
    return L


def k_slice(k: int, world: int, rank: int, align: int = 64):
    """[k0, k1) of rank `rank` when K is cut into `world` slices whose boundaries are multiples of
    `align` elements (TMA needs 16-byte aligned rows: 8 elements of bf16, 16 of s8; 64 keeps whole
    128-byte K blocks together).  Same arithmetic as the column partition."""
    return api.partition_columns(k, world, rank, align)


def make_desc(in_type, out_type, m, n, k_local, world, rank, layout_a=api.ROW_MAJOR, layout_b=api.ROW_MAJOR,
              lda=0, ldb=0, device=0, wait_limit_ns=0) -> KsDesc:
    d = KsDesc()
    d.struct_size = C.sizeof(KsDesc)
    d.in_type, d.out_type, d.layout_a, d.layout_b = in_type, out_type, layout_a, layout_b
    d.m, d.n, d.k_local, d.lda, d.ldb = m, n, k_local, lda, ldb
    d.world, d.rank, d.device, d.wait_limit_ns = world, rank, device, wait_limit_ns
    return d


def workspace_bytes(desc: KsDesc) -> int:
    n = C.c_size_t(0)
    st = _bind().gz_ks_workspace_bytes(C.byref(desc), C.byref(n))
    if st != GZ_OK:
        raise GzError(st, "gz_ks_workspace_bytes")
    return n.value


class SharedWorkspace:
    """A zero-filled device allocation plus its IPC handle."""

    def __init__(self, nbytes: int):
        p = C.c_void_p()
        h = C.create_string_buffer(IPC_HANDLE_BYTES)
        st = _bind().gz_ipc_alloc(nbytes, C.byref(p), h)
        if st != GZ_OK:
            raise GzError(st, "gz_ipc_alloc")
        self.ptr, self.handle, self.nbytes = p.value, h.raw, nbytes

    def free(self):
        if self.ptr:
            _bind().gz_ipc_free(self.ptr)
            self.ptr = None


def open_handle(handle: bytes) -> int:
    p = C.c_void_p()
    st = _bind().gz_ipc_open(handle, C.byref(p))
    if st != GZ_OK:
        raise GzError(st, "gz_ipc_open")
    return p.value


class KsPlan:
    """Owns a gz_ks_plan over given workspace addresses (one per rank, own included)."""

    def __init__(self, desc: KsDesc, workspaces):
        self.desc = desc
        arr = (C.c_void_p * len(workspaces))(*workspaces)
        h = C.c_void_p()
        st = _bind().gz_ks_plan_create(C.byref(h), C.byref(desc), arr)
        if st != GZ_OK:
            raise GzError(st, "gz_ks_plan_create")
        self._h = h

    def push(self, a, b, stream=None):
        st = _bind().gz_ks_push(self._h, _ptr(a), _ptr(b), _stream_handle(stream))
        if st != GZ_OK:
            raise GzError(st, "gz_ks_push")

    def reduce(self, c, d, alpha, beta, ldc=0, ldd=0, stream=None):
        al, be = _scalar(self.desc.in_type, alpha), _scalar(self.desc.in_type, beta)
        st = _bind().gz_ks_reduce(self._h, _ptr(c), _ptr(d), ldc, ldd, C.byref(al), C.byref(be),
                                  _stream_handle(stream))
        if st != GZ_OK:
            raise GzError(st, "gz_ks_reduce")

    def run(self, a, b, c, d, alpha, beta, ldc=0, ldd=0, stream=None):
        al, be = _scalar(self.desc.in_type, alpha), _scalar(self.desc.in_type, beta)
        st = _bind().gz_ks_run(self._h, _ptr(a), _ptr(b), _ptr(c), _ptr(d), ldc, ldd, C.byref(al), C.byref(be),
                               _stream_handle(stream))
        if st != GZ_OK:
            raise GzError(st, "gz_ks_run")

    def status(self, stream=None):
        detail = (C.c_uint32 * 4)()
        st = _bind().gz_ks_status(self._h, _stream_handle(stream), C.byref(detail))
        return st, list(detail)

    def destroy(self):
        if self._h:
            _bind().gz_ks_plan_destroy(self._h)
            self._h = None


class KShardedGemm:
    """K-sharded GEMM over the ranks of a ``torch.distributed`` process group (one GPU each, one node).

    ``D_r = alpha * sum_g A_g @ B_g[:, J_r] + beta * C_r`` with ``A_g``: m x k_local, ``B_g``:
    k_local x n (or its column-major storage) and ``C_r``/``D_r``: m x n/world on every rank.
    """

    def __init__(self, m, n, k_local, in_dtype, out_dtype, group=None, layout_a=api.ROW_MAJOR,
                 layout_b=api.ROW_MAJOR, lda=0, ldb=0, wait_limit_ns=0):
        import torch
        import torch.distributed as dist
        self.group = group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        it = in_dtype if isinstance(in_dtype, int) else api._torch_dtype_code(in_dtype)
        ot = out_dtype if isinstance(out_dtype, int) else api._torch_dtype_code(out_dtype)
        dev = torch.cuda.current_device()
        self.desc = make_desc(it, ot, m, n, k_local, self.world, self.rank, layout_a, layout_b, lda, ldb, dev,
                              wait_limit_ns)
        self.own = SharedWorkspace(workspace_bytes(self.desc))
        handles = [None] * self.world
        dist.all_gather_object(handles, self.own.handle, group=group)
        self.peers = [self.own.ptr if g == self.rank else open_handle(handles[g]) for g in range(self.world)]
        self.plan = KsPlan(self.desc, self.peers)
        dist.barrier(group=group)  # every rank has mapped every workspace before anyone pushes

    def __call__(self, a, b, c, d, alpha, beta, stream=None):
        self.plan.run(a, b, c, d, alpha, beta, stream=stream)

    def close(self):
        import torch
        import torch.distributed as dist
        torch.cuda.synchronize()
        dist.barrier(group=self.group)  # nobody unmaps while a peer may still push
        self.plan.destroy()
        for g, p in enumerate(self.peers):
            if g != self.rank:
                _bind().gz_ipc_close(p)
        dist.barrier(group=self.group)
        self.own.free()
