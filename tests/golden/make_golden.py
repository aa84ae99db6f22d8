"""Generates tests/golden/ref_kernels.npz: outputs of the reference project's own
generic_gemm and naive_gemm kernels (compiled unmodified from its sources into
oracle/_ref/libref_kernels.so by oracle/Makefile) for small seeded inputs.

Run on a machine with a GPU, after `make -C oracle`:

    python tests/golden/make_golden.py [output.npz]

The inputs are stored beside the outputs, so the CPU test that checks the oracle
against this file (tests/test_oracle_cpu.py) needs neither the GPU nor the
reference sources.
"""
from __future__ import annotations

import ctypes as C
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent.parent.parent
DT = {"f16": 0, "bf16": 1, "f32": 2, "s8": 3, "s32": 4}
TORCH = {"f16": torch.float16, "bf16": torch.bfloat16, "f32": torch.float32, "s8": torch.int8, "s32": torch.int32}

# (kernel, in, out, m, n, k, alpha, beta, value kind)
CASES = [
    ("generic", "f32", "f32", 48, 40, 72, 1.5, -0.5, "normal"),
    ("generic", "f32", "f32", 33, 65, 100, 1.0, 0.0, "normal"),
    ("naive", "f32", "f32", 48, 40, 72, 1.5, -0.5, "normal"),
    ("generic", "bf16", "f32", 40, 56, 96, 1.0, 1.0, "normal"),
    ("generic", "f16", "f32", 40, 56, 96, 2.0, 0.0, "normal"),
    ("generic", "f16", "f16", 37, 29, 64, 1.0, 1.0, "int"),
    ("generic", "bf16", "bf16", 37, 29, 64, 1.0, 1.0, "int"),
    ("generic", "s8", "s32", 45, 52, 128, 3.0, -2.0, "s8small"),
    ("naive", "s8", "s32", 45, 52, 300, 3.0, -2.0, "s8full"),
]


def gen(shape, kind, dtype, rng):
    if dtype == "s8":
        lo, hi = (-128, 128) if kind == "s8full" else (-8, 9)
        return torch.from_numpy(rng.integers(lo, hi, size=shape, dtype=np.int8))
    if dtype == "s32":
        return torch.from_numpy(rng.integers(-1000, 1001, size=shape, dtype=np.int32))
    if kind == "int":
        x = rng.integers(-2, 3, size=shape).astype(np.float32)
    else:
        x = rng.standard_normal(size=shape).astype(np.float32)
    return torch.from_numpy(x).to(TORCH[dtype])


def bits(t):
    t = t.cpu().contiguous()
    if t.dtype in (torch.float16, torch.bfloat16):
        return t.view(torch.int16).numpy().view(np.uint16)
    return t.numpy()


def main():
    out = Path(sys.argv[1]) if len(sys.argv) > 1 else ROOT / "tests" / "golden" / "ref_kernels.npz"
    lib = C.CDLL(str(ROOT / "oracle" / "_ref" / "libref_kernels.so"))
    for fn in (lib.ref_generic_gemm, lib.ref_naive_gemm):
        fn.argtypes = [C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64,
                       C.c_int64, C.c_double, C.c_double, C.c_void_p]
        fn.restype = C.c_int
    store = {}
    meta = []
    for idx, (kern, it, ot, m, n, k, alpha, beta, kind) in enumerate(CASES):
        rng = np.random.default_rng([2025, idx])
        a, b, c = gen((m, k), kind, it, rng), gen((k, n), kind, it, rng), gen((m, n), kind, ot, rng)
        ad, bd, cd = a.cuda(), b.cuda(), c.cuda()
        dd = torch.zeros(m, n, dtype=TORCH[ot], device="cuda")
        fn = lib.ref_generic_gemm if kern == "generic" else lib.ref_naive_gemm
        rc = fn(DT[it], DT[ot], ad.data_ptr(), bd.data_ptr(), cd.data_ptr(), dd.data_ptr(), m, n, k, alpha, beta, None)
        torch.cuda.synchronize()
        assert rc == 0, (kern, it, ot, rc)
        store[f"a{idx}"], store[f"b{idx}"], store[f"c{idx}"], store[f"d{idx}"] = bits(a), bits(b), bits(c), bits(dd)
        meta.append(f"{kern},{it},{ot},{m},{n},{k},{alpha},{beta},{kind}")
    store["meta"] = np.array(meta)
    np.savez_compressed(out, **store)
    print("wrote", out, out.stat().st_size, "bytes")


if __name__ == "__main__":
    main()
