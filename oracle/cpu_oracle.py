"""TEST INFRASTRUCTURE — not part of the product.

ctypes front end of oracle/liboracle.so (the CPU restatement of the reference
project's naive GEMM, oracle/ref_gemm.cpp).  Only tests/, the smoke check and the
CPU-baseline leg of bench.py may import this module; nothing under
gemm_zoo_b200/ does.

Operands are numpy arrays.  16-bit float types travel as uint16 bit patterns:
use `bits_of(torch_tensor)` to get them from a torch tensor of any supported dtype.
"""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
DT_F16, DT_BF16, DT_F32, DT_S8, DT_S32, DT_E4M3, DT_E5M2 = 0, 1, 2, 3, 4, 5, 6
_NP_OF = {DT_F16: np.uint16, DT_BF16: np.uint16, DT_F32: np.float32, DT_S8: np.int8, DT_S32: np.int32}

_lib = None


def build(force: bool = False) -> Path:
    out = HERE / "liboracle.so"
    src = HERE / "ref_gemm.cpp"
    if force or not out.exists() or out.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(HERE), "liboracle.so"], check=True, capture_output=True)
    return out


def lib():
    global _lib
    if _lib is None:
        p = HERE / "liboracle.so"
        if not p.exists():
            build()
        L = C.CDLL(str(p))
        i64, vp, dbl = C.c_int64, C.c_void_p, C.c_double
        L.oracle_gemm_f64.argtypes = [C.c_int, C.c_int, vp, vp, vp, vp, i64, i64, i64, i64, i64, i64, i64,
                                      i64, dbl, dbl, C.c_int, vp, i64]
        L.oracle_gemm_f64.restype = C.c_int
        L.oracle_gemm_s8.argtypes = [vp, vp, vp, vp, i64, i64, i64, i64, i64, i64, i64, i64, i64,
                                     C.c_int32, C.c_int32, vp, i64]
        L.oracle_gemm_s8.restype = C.c_int
        L.oracle_gemm_f32seq.argtypes = [C.c_int, vp, vp, vp, vp, i64, i64, i64, i64, i64, i64, i64, i64,
                                         C.c_float, C.c_float]
        L.oracle_gemm_f32seq.restype = C.c_int
        L.oracle_abs_gemm.argtypes = [C.c_int, vp, vp, vp, i64, i64, i64, i64, i64, i64, i64, vp, i64]
        L.oracle_abs_gemm.restype = C.c_int
        L.oracle_num_threads.restype = C.c_int
        L.oracle_set_threads.argtypes = [C.c_int]
        _lib = L
    return _lib


def num_threads() -> int:
    return lib().oracle_num_threads()


def bits_of(t) -> np.ndarray:
    """numpy view of a CPU torch tensor; fp16/bf16 become uint16 bit patterns."""
    import torch
    t = t.detach().cpu().contiguous()
    if t.dtype in (torch.float16, torch.bfloat16):
        return t.view(torch.int16).numpy().view(np.uint16)
    if t.dtype in (torch.float8_e4m3fn, torch.float8_e5m2):
        return t.view(torch.uint8).numpy()
    return t.numpy()


def dtype_code(t) -> int:
    import torch
    return {torch.float16: DT_F16, torch.bfloat16: DT_BF16, torch.float32: DT_F32, torch.int8: DT_S8,
            torch.int32: DT_S32, torch.float8_e4m3fn: DT_E4M3, torch.float8_e5m2: DT_E5M2}[t.dtype]


def _strides(m, n, k, a_col_major, b_col_major, lda, ldb):
    """Element strides (a_sm, a_sk, b_sk, b_sn) for the given layouts."""
    lda = lda or (m if a_col_major else k)
    ldb = ldb or (k if b_col_major else n)
    a_sm, a_sk = (1, lda) if a_col_major else (lda, 1)
    b_sk, b_sn = (1, ldb) if b_col_major else (ldb, 1)
    return a_sm, a_sk, b_sk, b_sn


def _rows(rows):
    if rows is None:
        return None, 0, None
    r = np.ascontiguousarray(np.asarray(rows, dtype=np.int64))
    return r.ctypes.data, r.size, r


def gemm_f64(in_type, out_type, a, b, c, m, n, k, alpha=1.0, beta=0.0, a_col_major=False,
             b_col_major=False, lda=0, ldb=0, ldc=0, tf32_mode=0, rows=None) -> np.ndarray:
    """alpha*A*B + beta*C in double.  Returns (len(rows) or m) x n float64."""
    a = np.ascontiguousarray(a)
    b = np.ascontiguousarray(b)
    a_sm, a_sk, b_sk, b_sn = _strides(m, n, k, a_col_major, b_col_major, lda, ldb)
    rp, nr, keep = _rows(rows)
    out = np.empty(((nr if rows is not None else m), n), dtype=np.float64)
    cp = None
    if beta != 0.0:
        c = np.ascontiguousarray(c)
        cp = c.ctypes.data
    st = lib().oracle_gemm_f64(in_type, out_type, a.ctypes.data, b.ctypes.data, cp, out.ctypes.data, m, n, k,
                               a_sm, a_sk, b_sk, b_sn, ldc or n, float(alpha), float(beta), tf32_mode, rp, nr)
    if st != 0:
        raise RuntimeError("oracle_gemm_f64 failed")
    return out


def gemm_s8(a, b, c, m, n, k, alpha=1, beta=0, a_col_major=False, b_col_major=False, lda=0, ldb=0,
            ldc=0, rows=None) -> np.ndarray:
    a = np.ascontiguousarray(a, dtype=np.int8)
    b = np.ascontiguousarray(b, dtype=np.int8)
    a_sm, a_sk, b_sk, b_sn = _strides(m, n, k, a_col_major, b_col_major, lda, ldb)
    rp, nr, keep = _rows(rows)
    out = np.empty(((nr if rows is not None else m), n), dtype=np.int32)
    cp = None
    if beta != 0:
        c = np.ascontiguousarray(c, dtype=np.int32)
        cp = c.ctypes.data
    st = lib().oracle_gemm_s8(a.ctypes.data, b.ctypes.data, cp, out.ctypes.data, m, n, k, a_sm, a_sk, b_sk,
                              b_sn, ldc or n, n, int(alpha), int(beta), rp, nr)
    if st != 0:
        raise RuntimeError("oracle_gemm_s8 failed")
    return out


def gemm_f32seq(in_type, a, b, c, m, n, k, alpha=1.0, beta=0.0, a_col_major=False, b_col_major=False,
                lda=0, ldb=0, ldc=0) -> np.ndarray:
    a = np.ascontiguousarray(a)
    b = np.ascontiguousarray(b)
    a_sm, a_sk, b_sk, b_sn = _strides(m, n, k, a_col_major, b_col_major, lda, ldb)
    out = np.empty((m, n), dtype=np.float32)
    cp = None
    if beta != 0.0:
        c = np.ascontiguousarray(c, dtype=np.float32)
        cp = c.ctypes.data
    st = lib().oracle_gemm_f32seq(in_type, a.ctypes.data, b.ctypes.data, cp, out.ctypes.data, m, n, k, a_sm,
                                  a_sk, b_sk, b_sn, ldc or n, float(alpha), float(beta))
    if st != 0:
        raise RuntimeError("oracle_gemm_f32seq failed")
    return out


def abs_gemm(in_type, a, b, m, n, k, a_col_major=False, b_col_major=False, lda=0, ldb=0, rows=None):
    a = np.ascontiguousarray(a)
    b = np.ascontiguousarray(b)
    a_sm, a_sk, b_sk, b_sn = _strides(m, n, k, a_col_major, b_col_major, lda, ldb)
    rp, nr, keep = _rows(rows)
    out = np.empty(((nr if rows is not None else m), n), dtype=np.float64)
    st = lib().oracle_abs_gemm(in_type, a.ctypes.data, b.ctypes.data, out.ctypes.data, m, n, k, a_sm, a_sk,
                               b_sk, b_sn, rp, nr)
    if st != 0:
        raise RuntimeError("oracle_abs_gemm failed")
    return out


def round_to(out_type, x: np.ndarray):
    """Round float64 results once to the output type; returns a torch CPU tensor."""
    import torch
    t = torch.from_numpy(np.ascontiguousarray(x))
    if out_type == DT_F16:
        return t.to(torch.float16)
    if out_type == DT_BF16:
        return t.to(torch.bfloat16)
    if out_type == DT_F32:
        return t.to(torch.float32)
    raise ValueError(out_type)


ACT_NONE, ACT_RELU, ACT_GELU, ACT_GELU_TANH, ACT_SILU = 0, 1, 2, 3, 4


def activate_f64(x: np.ndarray, act: int) -> np.ndarray:
    """The activations of gz_activation (include/gemmzoo/gemm.h) in double."""
    import math
    if act == ACT_NONE:
        return x
    if act == ACT_RELU:
        return np.maximum(x, 0.0)
    if act == ACT_GELU:
        erf = np.vectorize(math.erf, otypes=[np.float64])
        return 0.5 * x * (1.0 + erf(x / math.sqrt(2.0)))
    if act == ACT_GELU_TANH:
        return 0.5 * x * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (x + 0.044715 * x ** 3)))
    if act == ACT_SILU:
        return x / (1.0 + np.exp(-x))
    raise ValueError(act)


def epilogue_f64(acc, c, alpha, beta, bias=None, row_scale=None, col_scale=None, act=ACT_NONE) -> np.ndarray:
    """act(alpha * row_scale[i] * col_scale[j] * acc + beta * C + bias[j]) in double.

    `acc` is the unscaled product A*B (gemm_f64 / gemm_s8 with alpha=1, beta=0).  The reference's
    kernels stop at alpha/beta (nvidia/kernels/generic_gemm.cuh:53-58); the extra terms follow the
    definition in include/gemmzoo/gemm.h (gz_epilogue)."""
    r = float(alpha) * np.asarray(acc, dtype=np.float64)
    if row_scale is not None:
        r = r * np.asarray(row_scale, dtype=np.float64)[:, None]
    if col_scale is not None:
        r = r * np.asarray(col_scale, dtype=np.float64)[None, :]
    if c is not None and beta != 0:
        r = r + float(beta) * np.asarray(c, dtype=np.float64)
    if bias is not None:
        r = r + np.asarray(bias, dtype=np.float64)[None, :]
    return activate_f64(r, act)
