"""ctypes front end of libgz_cublaslt.so, the cuBLASLt comparator (bench and tests
only).  It stands where the reference's `kernel_functors::cublasLt_gemm` stands
(nvidia/kernel_functors/cublaslt_gemm.cuh:14-125): same constructor/call shape,
but the row-major problem is described truthfully, see cmp/cublaslt_cmp.cu.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

from .api import COL_MAJOR, DT_S8, ROW_MAJOR, _ptr, _scalar, _stream_handle, _torch_dtype_code

PKG = Path(__file__).resolve().parent
_lib = None


def lib():
    global _lib
    if _lib is None:
        p = PKG / "libgz_cublaslt.so"
        if not p.exists():
            raise RuntimeError(f"{p} is missing; build it with `python -m gemm_zoo_b200.build cublaslt`")
        L = C.CDLL(str(p))
        vp, i64 = C.c_void_p, C.c_int64
        L.gzc_create.argtypes = [C.POINTER(vp), C.c_int, C.c_int, C.c_int, C.c_int, i64, i64, i64, i64, i64,
                                 i64, i64, C.c_size_t, C.POINTER(C.c_int)]
        L.gzc_create.restype = C.c_int
        L.gzc_select.argtypes = [vp, C.c_int]
        L.gzc_select.restype = C.c_int
        L.gzc_run.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp]
        L.gzc_run.restype = C.c_int
        L.gzc_destroy.argtypes = [vp]
        L.gzc_destroy.restype = C.c_int
        _lib = L
    return _lib


class CublasLtGemm:
    def __init__(self, m, n, k, in_dtype, out_dtype, layout_a=ROW_MAJOR, layout_b=ROW_MAJOR, lda=0, ldb=0,
                 ldc=0, ldd=0, workspace_bytes=64 << 20):
        self.in_type = in_dtype if isinstance(in_dtype, int) else _torch_dtype_code(in_dtype)
        out_type = out_dtype if isinstance(out_dtype, int) else _torch_dtype_code(out_dtype)
        a_col, b_col = layout_a == COL_MAJOR, layout_b == COL_MAJOR
        lda = lda or (m if a_col else k)
        ldb = ldb or (k if b_col else n)
        self._h = C.c_void_p()
        n_algos = C.c_int(0)
        st = lib().gzc_create(C.byref(self._h), self.in_type, out_type, int(a_col), int(b_col), m, n, k, lda,
                              ldb, ldc or n, ldd or n, workspace_bytes, C.byref(n_algos))
        if st != 0:
            self._h = C.c_void_p()
            raise RuntimeError(f"cuBLASLt comparator could not be created (code {st})")
        self.num_algos = n_algos.value

    def select(self, index):
        if lib().gzc_select(self._h, index) != 0:
            raise IndexError(index)

    def __call__(self, a, b, c, d, alpha, beta, stream=None):
        al, be = _scalar(self.in_type, alpha), _scalar(self.in_type, beta)
        st = lib().gzc_run(self._h, _ptr(a), _ptr(b), _ptr(c), _ptr(d), C.byref(al), C.byref(be),
                           _stream_handle(stream))
        if st != 0:
            raise RuntimeError(f"cublasLtMatmul failed (code {st})")

    def destroy(self):
        if self._h:
            lib().gzc_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.destroy()
        except Exception:
            pass
