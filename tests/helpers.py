"""Shared machinery of the parity tests: build seeded operands in a given
layout, run the CUDA path through the C ABI, run the CPU oracle on the same
values, and compare.

Error bars:
  s8 -> s32                      bit-exact
  exact-integer inputs, any type bit-exact after one rounding to the output type
  fp16/bf16 inputs, random       |D - R| <= 2^-8 * |R| + 2^-20 * S   (bf16 out)
                                 |D - R| <= 2^-10 * |R| + 2^-20 * S  (fp16 out)
                                 |D - R| <= 2^-20 * S + 1e-6         (fp32 out)
  tf32 (fp32 in/out), random     |D - R| <= 2^-9 * S
  fp8 (e4m3/e5m2) inputs, random |D - R| <= u(out) * |R| + 2^-13 * S,  u = 2^-8 bf16, 2^-10 fp16, 0 fp32
where R is the fp64 oracle value and S = |alpha| * sum_k |a_ik||b_kj| + |beta||c_ij|.
"""
from __future__ import annotations

import dataclasses
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

import gemm_zoo_b200 as gz  # noqa: E402
from oracle import cpu_oracle as orc  # noqa: E402

SENTINEL = {"f": 777.0, "i": 0x5A5A5A5A}


@dataclasses.dataclass
class Case:
    in_type: int
    out_type: int
    m: int
    n: int
    k: int
    a_col: bool = False   # A column-major
    b_col: bool = False   # B column-major (the K-contiguous layout)
    alpha: float = 1.0
    beta: float = 0.0
    pad_a: int = 0        # extra elements added to the packed leading dimension
    pad_b: int = 0
    pad_c: int = 0
    pad_d: int = 0
    config: int = gz.CFG_AUTO
    flags: int = 0
    dist: str = "int"     # "int" small exact integers, "normal", "uniform"
    seed: int = 0
    scale_a: float = 1.0
    scale_b: float = 1.0
    inplace: bool = False  # D aliases C

    @property
    def lda(self):
        return (self.m if self.a_col else self.k) + self.pad_a

    @property
    def ldb(self):
        return (self.k if self.b_col else self.n) + self.pad_b

    @property
    def ldc(self):
        return self.n + (self.pad_d if self.inplace else self.pad_c)

    @property
    def ldd(self):
        return self.n + self.pad_d

    def name(self):
        dt = {0: "f16", 1: "bf16", 2: "f32", 3: "s8", 4: "s32"}
        dt.update({5: "e4m3", 6: "e5m2"})
        return (f"{dt[self.in_type]}->{dt[self.out_type]} {self.m}x{self.n}x{self.k} "
                f"A{'c' if self.a_col else 'r'}B{'c' if self.b_col else 'r'} a={self.alpha} b={self.beta} "
                f"cfg={self.config} fl={self.flags} {self.dist} pads={self.pad_a},{self.pad_b},{self.pad_c},{self.pad_d}"
                f"{' inplace' if self.inplace else ''}")


def torch_dtype(code):
    import torch
    return {gz.DT_F16: torch.float16, gz.DT_BF16: torch.bfloat16, gz.DT_F32: torch.float32,
            gz.DT_S8: torch.int8, gz.DT_S32: torch.int32, gz.DT_E4M3: torch.float8_e4m3fn,
            gz.DT_E5M2: torch.float8_e5m2}[code]


def _gen(shape, dtype_code, dist, seed, stream, scale):
    """Seeded host values (numpy Generator), rounded once to the storage type."""
    import torch
    rng = np.random.default_rng([seed, stream])
    if dtype_code == gz.DT_S8:
        lo, hi = (-128, 128) if dist != "int" else (-3, 4)
        return torch.from_numpy(rng.integers(lo, hi, size=shape, dtype=np.int8))
    if dtype_code == gz.DT_S32:
        return torch.from_numpy(rng.integers(-1000, 1001, size=shape, dtype=np.int32))
    if dist == "int":
        x = rng.integers(-2, 3, size=shape).astype(np.float32)
    elif dtype_code in (gz.DT_E4M3, gz.DT_E5M2) and dist == "full":
        # every finite byte pattern of the 8-bit format, scaled down so that sums stay in range
        bits = rng.integers(0, 256, size=shape, dtype=np.uint8)
        t = torch.from_numpy(bits).view(torch_dtype(dtype_code))
        f = t.float()
        f = torch.where(torch.isfinite(f), f, torch.zeros_like(f))
        f = torch.where(f.abs() > 240.0, torch.zeros_like(f), f)
        return f.to(torch_dtype(dtype_code))
    elif dist == "normal":
        x = (rng.standard_normal(size=shape) * scale).astype(np.float32)
    else:
        x = ((rng.random(size=shape) * 2 - 1) * scale).astype(np.float32)
    return torch.from_numpy(x).to(torch_dtype(dtype_code))


def make_operands(case: Case):
    """Host storage tensors: A (rows x lda), B (rows x ldb), C (m x ldc)."""
    a_rows = case.k if case.a_col else case.m
    b_rows = case.n if case.b_col else case.k
    a = _gen((a_rows, case.lda), case.in_type, case.dist, case.seed, 1, case.scale_a)
    b = _gen((b_rows, case.ldb), case.in_type, case.dist, case.seed, 2, case.scale_b)
    c = _gen((case.m, case.ldc), case.out_type, case.dist, case.seed, 3, 1.0)
    return a, b, c


def oracle_result(case: Case, a, b, c, rows=None, tf32_mode=0):
    """fp64 (or exact int32) oracle value for all rows or a sample; numpy array."""
    an, bn, cn = orc.bits_of(a), orc.bits_of(b), orc.bits_of(c)
    kw = dict(a_col_major=case.a_col, b_col_major=case.b_col, lda=case.lda, ldb=case.ldb, ldc=case.ldc,
              rows=rows)
    if case.in_type == gz.DT_S8:
        return orc.gemm_s8(an, bn, cn, case.m, case.n, case.k, alpha=int(case.alpha), beta=int(case.beta), **kw)
    return orc.gemm_f64(case.in_type, case.out_type, an, bn, cn, case.m, case.n, case.k, alpha=case.alpha,
                        beta=case.beta, tf32_mode=tf32_mode, **kw)


def error_scale(case: Case, a, b, c, rows=None):
    """S = |alpha| * sum_k |a||b| + |beta||c| for the rows checked (float64)."""
    an, bn = orc.bits_of(a), orc.bits_of(b)
    s = orc.abs_gemm(case.in_type, an, bn, case.m, case.n, case.k, a_col_major=case.a_col,
                     b_col_major=case.b_col, lda=case.lda, ldb=case.ldb, rows=rows)
    s *= abs(case.alpha)
    if case.beta != 0:
        cc = c[:, :case.n].double().numpy()
        s += abs(case.beta) * np.abs(cc if rows is None else cc[rows])
    return s


GUARD_ROWS = 2


def run_gpu(case: Case, a, b, c, device="cuda:0", plan=None):
    """Run through the C ABI.  Returns (d_host [m x n], guard_ok, plan_info, status)."""
    import torch
    dev = torch.device(device)
    ad, bd = a.to(dev), b.to(dev)
    odt = torch_dtype(case.out_type)
    sent = SENTINEL["i"] if case.out_type == gz.DT_S32 else SENTINEL["f"]
    # D sits between two guard bands; padding columns are guards too.
    dfull = torch.full((case.m + 2 * GUARD_ROWS, case.ldd), sent, dtype=odt, device=dev)
    dview = dfull[GUARD_ROWS:GUARD_ROWS + case.m]
    if case.inplace:
        dview[:, :case.n] = c[:, :case.n].to(dev)
        cd = dview
    else:
        cd = c.to(dev)
    own = plan is None
    if own:
        desc = gz.GemmDesc.make(case.in_type, case.out_type, case.m, case.n, case.k,
                                gz.COL_MAJOR if case.a_col else gz.ROW_MAJOR,
                                gz.COL_MAJOR if case.b_col else gz.ROW_MAJOR,
                                case.lda, case.ldb, case.ldc, case.ldd, dev.index or 0, case.config,
                                case.flags, wait_limit_ns=200_000_000)
        plan = gz.Plan(desc)
    info = plan.info()
    plan.run(ad, bd, cd if case.beta != 0 else None, dview, case.alpha, case.beta)
    status, detail = plan.device_status()
    torch.cuda.synchronize(dev)
    host = dfull.cpu()
    out = host[GUARD_ROWS:GUARD_ROWS + case.m, :case.n].contiguous()
    guards = [host[:GUARD_ROWS], host[GUARD_ROWS + case.m:], host[GUARD_ROWS:GUARD_ROWS + case.m, case.n:]]
    guard_ok = all(bool((g == sent).all()) for g in guards if g.numel())
    if own:
        plan.destroy()
    return out, guard_ok, info, (status, detail)


def tolerance(case: Case, ref, scale):
    """Per-element allowed |D - R| (float64 array), per the table in the module docstring."""
    if case.in_type == gz.DT_F32:
        return 2.0 ** -9 * scale + 1e-30
    if case.in_type in (gz.DT_E4M3, gz.DT_E5M2):
        # fp8 products are exact; the tensor core's fp32 accumulation of them is allowed 2^-13 * S
        unit = {gz.DT_BF16: 2.0 ** -8, gz.DT_F16: 2.0 ** -10, gz.DT_F32: 0.0}[case.out_type]
        return unit * np.abs(ref) + 2.0 ** -13 * scale + 1e-7
    if case.out_type == gz.DT_BF16:
        return 2.0 ** -8 * np.abs(ref) + 2.0 ** -20 * scale + 1e-30
    if case.out_type == gz.DT_F16:
        return 2.0 ** -10 * np.abs(ref) + 2.0 ** -20 * scale + 1e-7
    return 2.0 ** -20 * scale + 1e-6


def check(case: Case, device="cuda:0", rows=None):
    """Full parity check of one case.  Returns a dict with `ok` and diagnostics."""
    import torch
    a, b, c = make_operands(case)
    out, guard_ok, info, (status, detail) = run_gpu(case, a, b, c, device)
    res = {"case": case.name(), "config": info.config, "epilogue_tma": info.epilogue_tma, "split_k": info.split_k,
           "guard_ok": guard_ok, "status": status, "detail": detail}
    ref = oracle_result(case, a, b, c, rows=rows, tf32_mode=0)
    got = out if rows is None else out[rows]
    if case.in_type == gz.DT_S8:
        g = got.numpy()
        bad = int((g != ref).sum())
        res.update(mismatches=bad, ok=(bad == 0 and guard_ok and status == 0))
        if bad:
            idx = np.argwhere(g != ref)[:5]
            res["first_bad"] = [(int(i), int(j), int(g[i, j]), int(ref[i, j])) for i, j in idx]
        return res
    if case.dist == "int" and float(case.alpha).is_integer() and float(case.beta).is_integer():
        want = orc.round_to(case.out_type, ref)
        bad = int((got.view(torch.int16 if got.element_size() == 2 else torch.int32) !=
                   want.view(torch.int16 if want.element_size() == 2 else torch.int32)).sum())
        res.update(mismatches=bad, ok=(bad == 0 and guard_ok and status == 0))
        if bad:
            gd, wd = got.double().numpy(), want.double().numpy()
            idx = np.argwhere(gd != wd)[:5]
            res["first_bad"] = [(int(i), int(j), float(gd[i, j]), float(wd[i, j])) for i, j in idx]
            res["bad_rows"] = sorted(set(int(i) for i in np.argwhere(gd != wd)[:, 0]))[:8]
            res["bad_cols"] = sorted(set(int(j) for j in np.argwhere(gd != wd)[:, 1]))[:8]
        return res
    scale = error_scale(case, a, b, c, rows=rows)
    err = np.abs(got.double().numpy() - ref)
    tol = tolerance(case, ref, scale)
    bad = int((err > tol).sum()) + int((~np.isfinite(got.double().numpy())).sum())
    res.update(mismatches=bad, max_err=float(err.max()), max_rel_to_max=float(err.max() / max(np.abs(ref).max(), 1e-30)),
               max_err_over_scale=float((err / np.maximum(scale, 1e-30)).max()),
               ok=(bad == 0 and guard_ok and status == 0))
    return res
