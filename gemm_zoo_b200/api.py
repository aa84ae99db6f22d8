"""ctypes binding of include/gemmzoo/gemm.h, plus ``Sm100Gemm``, a Python mirror
of the reference functor concept (constructed from the problem, then called
with operands, scalars and a stream; nvidia/kernel_functors/bf16_mma_gemm.cuh:17-18,51-52).
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

PKG = Path(__file__).resolve().parent

# enums (mirror gemm.h)
DT_F16, DT_BF16, DT_F32, DT_S8, DT_S32, DT_E4M3, DT_E5M2 = 0, 1, 2, 3, 4, 5, 6
ROW_MAJOR, COL_MAJOR = 0, 1
CFG_AUTO, CFG_1CTA_N256, CFG_1CTA_N128, CFG_1CTA_N64, CFG_2CTA_N256, CFG_2CTA_N128, CFG_SIMT = 0, 1, 2, 3, 4, 5, 15
CFG_SWAP_M16, CFG_SWAP_M32, CFG_SWAP_M64, CFG_SWAP_M128 = 6, 7, 8, 9
CFG_2CTA_M512_N256 = 10
FLAG_EPILOGUE_DIRECT, FLAG_EPILOGUE_TMA, FLAG_TEST_WITHHOLD_ACC_READY = 0x1, 0x2, 0x80000000
FLAG_NO_SPLIT_K, FLAG_SPLIT_K = 0x4, 0x8
FLAG_BROADCAST_A, FLAG_BROADCAST_B = 0x10, 0x20
FLAG_NO_DIE_ORDER = 0x40
HOST_A_ON_DEVICE = 0x1
PROFILE_WORDS_PER_CTA = 24

GZ_OK = 0
GZ_ERR_INVALID_ARG, GZ_ERR_UNSUPPORTED, GZ_ERR_MISALIGNED, GZ_ERR_CUDA = 1, 2, 3, 4
GZ_ERR_DEVICE_TIMEOUT, GZ_ERR_NO_DEVICE, GZ_ERR_TOO_LARGE, GZ_ERR_OUT_OF_MEMORY = 5, 6, 7, 8
GZ_ERR_DEBUG_CHECK = 9

# Every symbol include/gemmzoo/gemm.h declares.
EXPORTED_SYMBOLS = [
    "gz_gemm_desc_validate", "gz_gemm_plan_create", "gz_gemm_plan_destroy", "gz_gemm_plan_info",
    "gz_gemm_plan_set_profile",
    "gz_gemm_run", "gz_gemm_run_ex", "gz_gemm_run_host", "gz_gemm_run_host_ex", "gz_gemm_skinny_static", "gz_static_last_device_status",
    "gz_last_device_status", "gz_status_string",
    "gz_last_cuda_error", "gz_fill", "gz_tile_coords", "gz_partition_columns", "gz_version",
    "gz_device_placement", "gz_classify_dies",
]


ACT_NONE, ACT_RELU, ACT_GELU, ACT_GELU_TANH, ACT_SILU = 0, 1, 2, 3, 4


class Epilogue(C.Structure):
    """gz_epilogue: D = act(alpha * row_scale[i] * col_scale[j] * acc + beta * C + bias[j])."""
    _fields_ = [("struct_size", C.c_uint32), ("activation", C.c_int32), ("bias", C.c_void_p),
                ("row_scale", C.c_void_p), ("col_scale", C.c_void_p)]

    @classmethod
    def make(cls, bias=None, row_scale=None, col_scale=None, activation=ACT_NONE):
        e = cls()
        e.struct_size = C.sizeof(cls)
        e.activation = activation
        e.bias, e.row_scale, e.col_scale = _ptr(bias), _ptr(row_scale), _ptr(col_scale)
        return e


class GemmDesc(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32), ("in_type", C.c_int32), ("out_type", C.c_int32),
        ("layout_a", C.c_int32), ("layout_b", C.c_int32), ("device", C.c_int32),
        ("config", C.c_int32), ("flags", C.c_uint32),
        ("m", C.c_int64), ("n", C.c_int64), ("k", C.c_int64),
        ("lda", C.c_int64), ("ldb", C.c_int64), ("ldc", C.c_int64), ("ldd", C.c_int64),
        ("wait_limit_ns", C.c_uint64),
        ("batch", C.c_int64), ("stride_a", C.c_int64), ("stride_b", C.c_int64), ("stride_c", C.c_int64),
        ("stride_d", C.c_int64),
    ]

    @classmethod
    def make(cls, in_type, out_type, m, n, k, layout_a=ROW_MAJOR, layout_b=ROW_MAJOR, lda=0, ldb=0,
             ldc=0, ldd=0, device=0, config=CFG_AUTO, flags=0, wait_limit_ns=0, batch=1, stride_a=0,
             stride_b=0, stride_c=0, stride_d=0):
        d = cls()
        d.struct_size = C.sizeof(cls)
        d.in_type, d.out_type = in_type, out_type
        d.layout_a, d.layout_b = layout_a, layout_b
        d.device, d.config, d.flags = device, config, flags
        d.m, d.n, d.k = m, n, k
        d.lda, d.ldb, d.ldc, d.ldd = lda, ldb, ldc, ldd
        d.wait_limit_ns = wait_limit_ns
        d.batch, d.stride_a, d.stride_b, d.stride_c, d.stride_d = batch, stride_a, stride_b, stride_c, stride_d
        return d


class PlanInfo(C.Structure):
    _fields_ = [
        ("config", C.c_int32), ("tile_m", C.c_int32), ("tile_n", C.c_int32), ("tile_k", C.c_int32),
        ("stages", C.c_int32), ("ctas_per_tile", C.c_int32), ("grid", C.c_int32),
        ("smem_bytes", C.c_int32), ("epilogue_tma", C.c_int32), ("sm_count", C.c_int32),
        ("split_k", C.c_int32), ("reserved", C.c_int32),
        ("tiles", C.c_int64), ("workspace_bytes", C.c_int64),
        ("lda", C.c_int64), ("ldb", C.c_int64), ("ldc", C.c_int64), ("ldd", C.c_int64),
        ("die_order", C.c_int32), ("reserved2", C.c_int32),
    ]

    def as_dict(self):
        return {f: getattr(self, f) for f, _ in self._fields_}


class GzError(RuntimeError):
    def __init__(self, status, where=""):
        self.status = status
        msg = status_string(status)
        if status == GZ_ERR_CUDA:
            msg += ": " + lib().gz_last_cuda_error().decode()
        super().__init__(f"{where}: {msg}" if where else msg)


_lib = None


def lib_path() -> Path:
    return PKG / "libgemmzoo.so"


def debug_lib_path() -> Path:
    """The same library compiled with -DGZ_BOUNDS_CHECK (bounds-checked epilogue stores); tests
    load it by pointing `lib_path` at it in a process of their own."""
    return PKG / "libgemmzoo_dbg.so"


def lib():
    """Load libgemmzoo.so.  Raises if it has not been built: there is no fallback path."""
    global _lib
    if _lib is not None:
        return _lib
    p = lib_path()
    if not p.exists():
        raise RuntimeError(f"{p} is missing; build it with `python -m gemm_zoo_b200.build lib` "
                           "(or __graft_entry__.build())")
    L = C.CDLL(str(p))
    vp, i32, i64, u32, u64 = C.c_void_p, C.c_int32, C.c_int64, C.c_uint32, C.c_uint64
    L.gz_gemm_desc_validate.argtypes = [C.POINTER(GemmDesc), C.c_int, C.POINTER(PlanInfo)]
    L.gz_gemm_desc_validate.restype = C.c_int
    L.gz_gemm_plan_create.argtypes = [C.POINTER(vp), C.POINTER(GemmDesc)]
    L.gz_gemm_plan_create.restype = C.c_int
    L.gz_gemm_plan_destroy.argtypes = [vp]
    L.gz_gemm_plan_destroy.restype = C.c_int
    L.gz_gemm_plan_info.argtypes = [vp, C.POINTER(PlanInfo)]
    L.gz_gemm_plan_info.restype = C.c_int
    L.gz_gemm_run.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp]
    L.gz_gemm_run.restype = C.c_int
    L.gz_gemm_run_ex.argtypes = [vp, vp, vp, vp, vp, vp, vp, C.POINTER(Epilogue), vp]
    L.gz_gemm_run_ex.restype = C.c_int
    L.gz_gemm_plan_set_profile.argtypes = [vp, vp]
    L.gz_gemm_plan_set_profile.restype = C.c_int
    L.gz_gemm_run_host.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp]
    L.gz_gemm_run_host.restype = C.c_int
    L.gz_gemm_run_host_ex.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, u32]
    L.gz_gemm_run_host_ex.restype = C.c_int
    L.gz_gemm_skinny_static.argtypes = [C.POINTER(GemmDesc), vp, vp, vp, vp, vp, vp, vp]
    L.gz_gemm_skinny_static.restype = C.c_int
    L.gz_static_last_device_status.argtypes = [i32, vp, C.POINTER(u32 * 4)]
    L.gz_static_last_device_status.restype = C.c_int
    L.gz_last_device_status.argtypes = [vp, vp, C.POINTER(u32 * 4)]
    L.gz_last_device_status.restype = C.c_int
    L.gz_status_string.argtypes = [C.c_int]
    L.gz_status_string.restype = C.c_char_p
    L.gz_last_cuda_error.argtypes = []
    L.gz_last_cuda_error.restype = C.c_char_p
    L.gz_fill.argtypes = [vp, i32, i64, u64, u32, i32, C.c_float, vp]
    L.gz_fill.restype = C.c_int
    L.gz_tile_coords.argtypes = [u32, u32, u32, u32, C.POINTER(u32), C.POINTER(u32)]
    L.gz_tile_coords.restype = None
    L.gz_partition_columns.argtypes = [i64, i32, i32, i64, C.POINTER(i64), C.POINTER(i64)]
    L.gz_partition_columns.restype = C.c_int
    L.gz_device_placement.argtypes = [i32, vp, C.POINTER(i32 * 2)]
    L.gz_device_placement.restype = C.c_int
    L.gz_classify_dies.argtypes = [vp, i32, i32, vp, C.POINTER(i32 * 2)]
    L.gz_classify_dies.restype = C.c_int
    L.gz_version.argtypes = []
    L.gz_version.restype = i32
    _lib = L
    return L


def status_string(status: int) -> str:
    return lib().gz_status_string(int(status)).decode()


def validate(desc: GemmDesc, sm_count: int = 0):
    """Host-only validation.  Returns (status, PlanInfo)."""
    info = PlanInfo()
    st = lib().gz_gemm_desc_validate(C.byref(desc), sm_count, C.byref(info))
    return st, info


def tile_coords(tiles_m, tiles_n, group_m, t):
    tm, tn = C.c_uint32(), C.c_uint32()
    lib().gz_tile_coords(tiles_m, tiles_n, group_m, t, C.byref(tm), C.byref(tn))
    return tm.value, tn.value


def partition_columns(n, parts, p, align=8):
    b, e = C.c_int64(), C.c_int64()
    st = lib().gz_partition_columns(n, parts, p, align, C.byref(b), C.byref(e))
    if st != GZ_OK:
        raise GzError(st, "gz_partition_columns")
    return b.value, e.value


def classify_dies(clocks):
    """gz_classify_dies on a (sms x lines) uint32 numpy array.  Returns (status, die_of_sm list, [n0, n1])."""
    import numpy as np
    c = np.ascontiguousarray(clocks, dtype=np.uint32)
    sms, lines = c.shape
    dies = (C.c_uint8 * 160)()
    counts = (C.c_int32 * 2)()
    st = lib().gz_classify_dies(c.ctypes.data, sms, lines, C.addressof(dies), C.byref(counts))
    return st, list(dies)[:sms], list(counts)


def device_placement(device=0):
    """gz_device_placement: (status, die_of_sm list, [n0, n1])."""
    dies = (C.c_uint8 * 160)()
    counts = (C.c_int32 * 2)()
    st = lib().gz_device_placement(device, C.addressof(dies), C.byref(counts))
    return st, list(dies), list(counts)


def _scalar(in_type, v, out_type=None):
    """alpha / beta in the type the C ABI reads: int32 for s32 outputs, float otherwise."""
    is_int = (out_type == DT_S32) if out_type is not None else (in_type == DT_S8)
    return C.c_int32(int(v)) if is_int else C.c_float(float(v))


def _ptr(x):
    """Device/host address of a torch tensor, numpy array, int, or None."""
    if x is None:
        return None
    if isinstance(x, int):
        return x
    if hasattr(x, "data_ptr"):
        return x.data_ptr()
    if hasattr(x, "ctypes"):
        return x.ctypes.data
    raise TypeError(type(x))


def _stream_handle(stream):
    if stream is None:
        return None
    if isinstance(stream, int):
        return stream or None
    return stream.cuda_stream or None  # torch.cuda.Stream


class Plan:
    """Owns a gz_plan."""

    def __init__(self, desc: GemmDesc):
        self.desc = desc
        self._h = C.c_void_p()
        st = lib().gz_gemm_plan_create(C.byref(self._h), C.byref(desc))
        if st != GZ_OK:
            self._h = C.c_void_p()
            raise GzError(st, "gz_gemm_plan_create")

    def info(self) -> PlanInfo:
        info = PlanInfo()
        st = lib().gz_gemm_plan_info(self._h, C.byref(info))
        if st != GZ_OK:
            raise GzError(st, "gz_gemm_plan_info")
        return info

    def run(self, a, b, c, d, alpha, beta, stream=None):
        al, be = (_scalar(self.desc.in_type, alpha, self.desc.out_type),
                  _scalar(self.desc.in_type, beta, self.desc.out_type))
        st = lib().gz_gemm_run(self._h, _ptr(a), _ptr(b), _ptr(c), _ptr(d), C.byref(al), C.byref(be),
                               _stream_handle(stream))
        if st != GZ_OK:
            raise GzError(st, "gz_gemm_run")

    def run_ex(self, a, b, c, d, alpha, beta, bias=None, row_scale=None, col_scale=None, activation=ACT_NONE,
               stream=None):
        """gz_gemm_run_ex: bias / row_scale / col_scale are fp32 device vectors (or None)."""
        al, be = (_scalar(self.desc.in_type, alpha, self.desc.out_type),
                  _scalar(self.desc.in_type, beta, self.desc.out_type))
        ep = Epilogue.make(bias, row_scale, col_scale, activation)
        st = lib().gz_gemm_run_ex(self._h, _ptr(a), _ptr(b), _ptr(c), _ptr(d), C.byref(al), C.byref(be),
                                  C.byref(ep), _stream_handle(stream))
        if st != GZ_OK:
            raise GzError(st, "gz_gemm_run_ex")

    def run_host(self, a, b, c, d, alpha, beta, stream=None, a_on_device=False):
        """Host operands (gz_gemm_run_host).  a_on_device: `a` is already in this GPU's memory
        (gz_gemm_run_host_ex with GZ_HOST_A_ON_DEVICE); b, c, d stay host pointers."""
        al, be = (_scalar(self.desc.in_type, alpha, self.desc.out_type),
                  _scalar(self.desc.in_type, beta, self.desc.out_type))
        st = lib().gz_gemm_run_host_ex(self._h, _ptr(a), _ptr(b), _ptr(c), _ptr(d), C.byref(al),
                                       C.byref(be), _stream_handle(stream), HOST_A_ON_DEVICE if a_on_device else 0)
        if st != GZ_OK:
            raise GzError(st, "gz_gemm_run_host")

    def set_profile(self, buf):
        """buf: contiguous torch int64 CUDA tensor of at least PROFILE_WORDS_PER_CTA * info().grid
        words (the kernel writes that many per CTA), or None to switch the counters off."""
        if buf is not None:
            import torch
            need = PROFILE_WORDS_PER_CTA * self.info().grid
            if not (isinstance(buf, torch.Tensor) and buf.is_cuda and buf.dtype == torch.int64 and
                    buf.is_contiguous() and buf.numel() >= need):
                raise ValueError(f"set_profile needs a contiguous int64 CUDA tensor of at least {need} words")
            if buf.device.index != self.desc.device:
                raise ValueError("set_profile: the buffer must live on the plan's device")
        st = lib().gz_gemm_plan_set_profile(self._h, _ptr(buf))
        if st != GZ_OK:
            raise GzError(st, "gz_gemm_plan_set_profile")

    def device_status(self, stream=None):
        """(status, detail[4]) after synchronising `stream`."""
        detail = (C.c_uint32 * 4)()
        st = lib().gz_last_device_status(self._h, _stream_handle(stream), C.byref(detail))
        return st, list(detail)

    def destroy(self):
        if self._h:
            lib().gz_gemm_plan_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.destroy()
        except Exception:
            pass


_TORCH_DT = None


def _torch_dtype_code(t):
    global _TORCH_DT
    if _TORCH_DT is None:
        import torch
        _TORCH_DT = {torch.float16: DT_F16, torch.bfloat16: DT_BF16, torch.float32: DT_F32,
                     torch.int8: DT_S8, torch.int32: DT_S32, torch.float8_e4m3fn: DT_E4M3,
                     torch.float8_e5m2: DT_E5M2}
    return _TORCH_DT[t]


class Sm100Gemm:
    """Mirror of the reference functor concept.

    Reference: ``Kernel kernel(m, n, k, properties); kernel(a, b, c, d, alpha, beta, stream);``
    (nvidia/utils/benchmark.cuh:54-57).  Defaults reproduce the reference
    convention: A row-major ld=k, B row-major ld=n, C/D row-major ld=n.
    """

    def __init__(self, m, n, k, in_dtype, out_dtype, layout_a=ROW_MAJOR, layout_b=ROW_MAJOR, lda=0,
                 ldb=0, ldc=0, ldd=0, device=0, config=CFG_AUTO, flags=0, wait_limit_ns=0, batch=1,
                 stride_a=0, stride_b=0, stride_c=0, stride_d=0):
        it = in_dtype if isinstance(in_dtype, int) else _torch_dtype_code(in_dtype)
        ot = out_dtype if isinstance(out_dtype, int) else _torch_dtype_code(out_dtype)
        self.desc = GemmDesc.make(it, ot, m, n, k, layout_a, layout_b, lda, ldb, ldc, ldd, device,
                                  config, flags, wait_limit_ns, batch, stride_a, stride_b, stride_c, stride_d)
        self.plan = Plan(self.desc)

    def __call__(self, a, b, c, d, alpha, beta, stream=None):
        self.plan.run(a, b, c, d, alpha, beta, stream)

    def info(self):
        return self.plan.info()


STATIC_SCRATCH_BYTES = 8 << 20


def gemm_skinny_static(desc: GemmDesc, a, b, c, d, alpha, beta, stream=None):
    """gz_gemm_skinny_static: the skinny split-K GEMM with its scratch in the library's fixed
    array, for hosts that must not allocate.  Returns the gz_status (0 = launched)."""
    al, be = _scalar(desc.in_type, alpha, desc.out_type), _scalar(desc.in_type, beta, desc.out_type)
    return lib().gz_gemm_skinny_static(C.byref(desc), _ptr(a), _ptr(b), _ptr(c), _ptr(d), C.byref(al),
                                       C.byref(be), _stream_handle(stream))


def static_device_status(device=0, stream=None):
    """gz_static_last_device_status: (status, detail[4]) of the gz_gemm_skinny_static launches on
    `device` after synchronising `stream`; a recorded timeout is cleared by the read."""
    detail = (C.c_uint32 * 4)()
    st = lib().gz_static_last_device_status(device, _stream_handle(stream), C.byref(detail))
    return st, list(detail)


def fill(t, seed, stream_id, dist, scale=1.0, stream=None):
    """Seeded fill of a contiguous torch CUDA tensor (see gz_fill)."""
    st = lib().gz_fill(t.data_ptr(), _torch_dtype_code(t.dtype), t.numel(), seed, stream_id, dist,
                       float(scale), _stream_handle(stream))
    if st != GZ_OK:
        raise GzError(st, "gz_fill")
    return t
