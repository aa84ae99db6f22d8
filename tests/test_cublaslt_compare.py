"""This library against cuBLASLt (configured for the true row-major problem) on the
same operands: s8 bit for bit, floating point within twice the oracle tolerance."""
import numpy as np
import pytest
import torch

import gemm_zoo_b200 as gz

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TORCH = {gz.DT_F16: torch.float16, gz.DT_BF16: torch.bfloat16, gz.DT_F32: torch.float32, gz.DT_S8: torch.int8,
         gz.DT_S32: torch.int32}


@pytest.mark.parametrize("in_t,out_t,b_col", [(gz.DT_S8, gz.DT_S32, True), (gz.DT_BF16, gz.DT_BF16, True),
                                              (gz.DT_BF16, gz.DT_F32, False), (gz.DT_F16, gz.DT_F16, True),
                                              (gz.DT_F32, gz.DT_F32, False), (gz.DT_F32, gz.DT_F32, True)])
def test_agrees_with_cublaslt(in_t, out_t, b_col):
    from gemm_zoo_b200.cublaslt import CublasLtGemm
    m, n, k = 1024, 1536, 2048
    gen = torch.Generator(device=DEV).manual_seed(3)
    if in_t == gz.DT_S8:
        a = torch.randint(-128, 128, (m, k), dtype=torch.int8, device=DEV, generator=gen)
        b = torch.randint(-128, 128, (n, k) if b_col else (k, n), dtype=torch.int8, device=DEV, generator=gen)
        c = torch.randint(-1000, 1000, (m, n), dtype=torch.int32, device=DEV, generator=gen)
        alpha, beta = 2, 1
    else:
        a = torch.randn(m, k, device=DEV, generator=gen).to(TORCH[in_t])
        b = (torch.randn((n, k) if b_col else (k, n), device=DEV, generator=gen) * k ** -0.5).to(TORCH[in_t])
        c = torch.randn(m, n, device=DEV, generator=gen).to(TORCH[out_t])
        alpha, beta = 1.0, 0.5
    lb = gz.COL_MAJOR if b_col else gz.ROW_MAJOR
    d_own = torch.empty(m, n, dtype=TORCH[out_t], device=DEV)
    d_lt = torch.empty_like(d_own)
    gz.Sm100Gemm(m, n, k, in_t, out_t, layout_b=lb)(a, b, c, d_own, alpha, beta)
    try:
        lt = CublasLtGemm(m, n, k, in_t, out_t, layout_b=lb)
    except RuntimeError as e:
        pytest.skip(f"cuBLASLt has no algorithm for this case: {e}")
    lt(a, b, c, d_lt, alpha, beta)
    torch.cuda.synchronize()
    if in_t == gz.DT_S8:
        assert torch.equal(d_own, d_lt)
        return
    bm = b.t() if b_col else b
    scale = (a.double().abs() @ bm.double().abs() + 0.5 * c.double().abs()).cpu().numpy()
    err = (d_own.double() - d_lt.double()).abs().cpu().numpy()
    unit = {gz.DT_BF16: 2.0 ** -7, gz.DT_F16: 2.0 ** -9, gz.DT_F32: 0.0}[out_t]
    ref_mag = d_lt.double().abs().cpu().numpy()
    extra = 2.0 ** -8 if in_t == gz.DT_F32 else 2.0 ** -19
    assert (err <= unit * ref_mag + extra * scale + 1e-6).all()
