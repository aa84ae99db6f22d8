"""CPU tests of the oracle (oracle/ref_gemm.cpp): against numpy on hand-checkable
cases (layouts, leading dimensions, alpha/beta, int32 wrap-around, row sampling)
and against tests/golden/ref_kernels.npz, which holds outputs of the reference
project's own generic_gemm / naive_gemm kernels run on a B200."""
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import cpu_oracle as orc

GOLDEN = Path(__file__).resolve().parent / "golden" / "ref_kernels.npz"


def _f(bits, dt):
    """float64 view of stored operand bits."""
    if dt == "bf16":
        return torch.from_numpy(bits.view(np.int16).copy()).view(torch.bfloat16).double().numpy()
    if dt == "f16":
        return torch.from_numpy(bits.view(np.int16).copy()).view(torch.float16).double().numpy()
    return bits.astype(np.float64)


def test_f64_matches_numpy_all_layouts():
    rng = np.random.default_rng(0)
    m, n, k = 37, 53, 71
    a = rng.standard_normal((m, k)).astype(np.float32)
    b = rng.standard_normal((k, n)).astype(np.float32)
    c = rng.standard_normal((m, n)).astype(np.float32)
    ref = 1.5 * (a.astype(np.float64) @ b.astype(np.float64)) - 0.5 * c
    for a_col in (False, True):
        for b_col in (False, True):
            aa = np.ascontiguousarray(a.T) if a_col else a
            bb = np.ascontiguousarray(b.T) if b_col else b
            r = orc.gemm_f64(orc.DT_F32, orc.DT_F32, aa, bb, c, m, n, k, alpha=1.5, beta=-0.5,
                             a_col_major=a_col, b_col_major=b_col)
            assert np.abs(r - ref).max() < 1e-12


def test_leading_dimensions_and_row_sample():
    rng = np.random.default_rng(1)
    m, n, k, lda, ldb, ldc = 9, 11, 13, 20, 17, 16
    a = rng.standard_normal((m, lda)).astype(np.float32)
    b = rng.standard_normal((k, ldb)).astype(np.float32)
    c = rng.standard_normal((m, ldc)).astype(np.float32)
    ref = a[:, :k].astype(np.float64) @ b[:, :n].astype(np.float64) + 2.0 * c[:, :n]
    r = orc.gemm_f64(orc.DT_F32, orc.DT_F32, a, b, c, m, n, k, alpha=1.0, beta=2.0, lda=lda, ldb=ldb, ldc=ldc)
    assert np.abs(r - ref).max() < 1e-12
    rows = [8, 0, 3]
    r2 = orc.gemm_f64(orc.DT_F32, orc.DT_F32, a, b, c, m, n, k, alpha=1.0, beta=2.0, lda=lda, ldb=ldb, ldc=ldc,
                      rows=rows)
    assert np.array_equal(r2, r[rows])


def test_beta_zero_does_not_read_c():
    a = np.ones((2, 3), np.float32)
    b = np.ones((3, 2), np.float32)
    r = orc.gemm_f64(orc.DT_F32, orc.DT_F32, a, b, None, 2, 2, 3, alpha=1.0, beta=0.0)
    assert np.array_equal(r, np.full((2, 2), 3.0))


def test_s8_exact_and_wraps():
    rng = np.random.default_rng(2)
    m, n, k = 21, 19, 300
    a = rng.integers(-128, 128, (m, k), dtype=np.int8)
    b = rng.integers(-128, 128, (k, n), dtype=np.int8)
    c = rng.integers(-2 ** 31, 2 ** 31, (m, n), dtype=np.int64).astype(np.int32)
    exact = a.astype(np.int64) @ b.astype(np.int64)
    r = orc.gemm_s8(a, b, c, m, n, k, alpha=3, beta=-2)
    assert np.array_equal(r, (3 * exact - 2 * c.astype(np.int64)).astype(np.int32))
    # alpha large enough to overflow: arithmetic is modulo 2^32
    r = orc.gemm_s8(a, b, c, m, n, k, alpha=2 ** 20, beta=7)
    want = ((2 ** 20) * exact + 7 * c.astype(np.int64)) & 0xFFFFFFFF
    assert np.array_equal(r.view(np.uint32).astype(np.int64), want)
    # column-major B
    r = orc.gemm_s8(a, np.ascontiguousarray(b.T), None, m, n, k, b_col_major=True)
    assert np.array_equal(r, exact.astype(np.int32))


def test_half_types_convert_exactly():
    m, n, k = 8, 8, 16
    ta = torch.randn(m, k, generator=torch.Generator().manual_seed(3))
    for tdt, code in ((torch.bfloat16, orc.DT_BF16), (torch.float16, orc.DT_F16)):
        a = ta.to(tdt)
        b = torch.randn(k, n, generator=torch.Generator().manual_seed(4)).to(tdt)
        r = orc.gemm_f64(code, code, orc.bits_of(a), orc.bits_of(b), None, m, n, k)
        assert np.abs(r - (a.double() @ b.double()).numpy()).max() == 0.0
    # fp16 subnormals, infinities' neighbours
    vals = torch.tensor([6e-8, -6e-8, 65504.0, 1e-5, 0.0, -0.0], dtype=torch.float16).repeat(1, 1)
    r = orc.gemm_f64(orc.DT_F16, orc.DT_F16, orc.bits_of(vals), orc.bits_of(torch.eye(6, dtype=torch.float16)),
                     None, 1, 6, 6)
    assert np.array_equal(r[0], vals.double().numpy()[0])


def test_tf32_modes():
    a = np.array([[1.0 + 2.0 ** -11, 1.0 + 2.0 ** -12]], dtype=np.float32)
    b = np.eye(2, dtype=np.float32)
    keep = orc.gemm_f64(orc.DT_F32, orc.DT_F32, a, b, None, 1, 2, 2, tf32_mode=0)
    trunc = orc.gemm_f64(orc.DT_F32, orc.DT_F32, a, b, None, 1, 2, 2, tf32_mode=1)
    rna = orc.gemm_f64(orc.DT_F32, orc.DT_F32, a, b, None, 1, 2, 2, tf32_mode=2)
    assert keep[0, 0] == 1.0 + 2.0 ** -11
    assert np.array_equal(trunc[0], [1.0, 1.0])
    assert np.array_equal(rna[0], [1.0 + 2.0 ** -10, 1.0])


def test_f32seq_is_close_to_f64():
    rng = np.random.default_rng(5)
    m, n, k = 16, 24, 512
    a = rng.standard_normal((m, k)).astype(np.float32)
    b = rng.standard_normal((k, n)).astype(np.float32)
    r64 = orc.gemm_f64(orc.DT_F32, orc.DT_F32, a, b, None, m, n, k)
    r32 = orc.gemm_f32seq(orc.DT_F32, a, b, None, m, n, k)
    assert np.abs(r32 - r64).max() < 1e-3


@pytest.mark.skipif(not GOLDEN.exists(), reason="golden fixture not generated yet")
def test_oracle_matches_reference_kernels_golden():
    """Pins the oracle to what the reference's own kernels computed on a B200."""
    z = np.load(GOLDEN)
    code = {"f16": orc.DT_F16, "bf16": orc.DT_BF16, "f32": orc.DT_F32, "s8": orc.DT_S8, "s32": orc.DT_S32}
    checked = 0
    for idx, line in enumerate(z["meta"]):
        kern, it, ot, m, n, k, alpha, beta, kind = str(line).split(",")
        m, n, k, alpha, beta = int(m), int(n), int(k), float(alpha), float(beta)
        a, b, c, d = z[f"a{idx}"], z[f"b{idx}"], z[f"c{idx}"], z[f"d{idx}"]
        if it == "s8":
            # generic_gemm sums in fp32 (exact while |sum| < 2^24), naive_gemm in int32
            r = orc.gemm_s8(a, b, c, m, n, k, alpha=int(alpha), beta=int(beta))
            assert np.array_equal(r, d), (idx, line)
        elif ot == "f32" and it == "f32" and kern == "generic":
            # same arithmetic as the kernel: fp32 fused multiply-add, k ascending -> bit-exact
            r = orc.gemm_f32seq(code[it], a, b, c, m, n, k, alpha=alpha, beta=beta)
            assert np.array_equal(r.view(np.uint32), d.view(np.uint32)), (idx, line)
        elif kind == "int":
            # small-integer inputs: every partial sum is exact in every type
            r = orc.gemm_f64(code[it], code[ot], a, b, c, m, n, k, alpha=alpha, beta=beta)
            assert np.array_equal(r, _f(d, ot)), (idx, line)
        else:
            r = orc.gemm_f64(code[it], code[ot], a, b, c, m, n, k, alpha=alpha, beta=beta)
            scale = np.abs(_f(a, it)) @ np.abs(_f(b, it)) * abs(alpha) + abs(beta) * np.abs(_f(c, ot))
            assert (np.abs(r - _f(d, ot)) <= 2.0 ** -20 * scale + 1e-6).all(), (idx, line)
        checked += 1
    assert checked == len(z["meta"]) >= 8


@pytest.mark.parametrize("tdt,code", [(torch.float8_e4m3fn, orc.DT_E4M3), (torch.float8_e5m2, orc.DT_E5M2)])
def test_fp8_decoding_matches_every_byte_pattern(tdt, code):
    allb = torch.arange(256, dtype=torch.uint8).view(tdt)
    vals = allb.float().double().numpy()
    one = torch.ones(1, 1).to(tdt)
    r = orc.gemm_f64(code, orc.DT_F32, orc.bits_of(allb.view(256, 1)), orc.bits_of(one), None, 256, 1, 1)[:, 0]
    assert bool(((r == vals) | (np.isnan(r) & np.isnan(vals))).all())
