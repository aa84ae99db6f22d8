"""How the tf32 multiply treats the 13 low mantissa bits of its fp32 operands.

The reference feeds raw fp32 bit patterns to the tensor cores (B through `ld.shared.b32`, A
through `ldmatrix`, no `cvt.rna`: nvidia/kernels/sm_80/tf32_mma_gemm.cuh:138-155), so its
operands are TRUNCATED to tf32.  This library does the same: TMA copies the fp32 bits to shared
memory and `tcgen05.mma.kind::tf32` reads them from there.

The usual tf32 bar (|D - R| <= 2^-9 * S against the unrounded-input fp64 reference) cannot tell
truncation from round-to-nearest, nor notice a descriptor that drops more bits than it should.
This test can: every operand has all 13 low mantissa bits set and all operands are positive, so
truncation and rounding move every product the same way and the two fp64 references (inputs
truncated / inputs rounded to nearest, ties away) differ by about 2^-9 * S, while what is left
against the RIGHT reference is fp32 accumulation error only.  Bar: max |D - R| / S <= 1e-4 against
the truncated-input reference, and clearly above it against the rounded one.
S = sum_k |a_ik| |b_kj|.
"""
import numpy as np
import pytest
import torch

import gemm_zoo_b200 as gz
from oracle import cpu_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
BAR = 1e-4


def _operand(shape, seed):
    rng = np.random.default_rng(seed)
    x = (0.5 + 0.5 * rng.random(size=shape)).astype(np.float32)
    bits = x.view(np.uint32) | np.uint32(0x1FFF)  # all 13 bits below tf32's mantissa set
    return torch.from_numpy(bits.view(np.float32).copy())


@pytest.mark.parametrize("b_col", [False, True])
@pytest.mark.parametrize("config", [gz.CFG_AUTO, gz.CFG_1CTA_N128, gz.CFG_2CTA_N256, gz.CFG_2CTA_M512_N256])
def test_tf32_operands_are_truncated_like_the_reference(config, b_col):
    m, n, k = 512, 512, 512
    a = _operand((m, k), 1)
    b = _operand((n, k) if b_col else (k, n), 2)
    d = torch.empty(m, n, dtype=torch.float32, device=DEV)
    g = gz.Sm100Gemm(m, n, k, gz.DT_F32, gz.DT_F32, layout_b=gz.COL_MAJOR if b_col else gz.ROW_MAJOR, config=config)
    g(a.to(DEV), b.to(DEV), None, d, 1.0, 0.0)
    assert g.plan.device_status()[0] == 0
    got = d.cpu().double().numpy()
    an, bn = orc.bits_of(a), orc.bits_of(b)
    scale = orc.abs_gemm(gz.DT_F32, an, bn, m, n, k, b_col_major=b_col)
    err = {}
    for mode in (0, 1, 2):  # unrounded, truncated, rounded to nearest (ties away)
        ref = orc.gemm_f64(gz.DT_F32, gz.DT_F32, an, bn, None, m, n, k, b_col_major=b_col, tf32_mode=mode)
        err[mode] = float((np.abs(got - ref) / scale).max())
    # the general bar still holds ...
    assert err[0] <= 2.0 ** -9, err
    # ... and the operands were truncated, not rounded, with nothing more lost than the 13 bits
    assert err[1] <= BAR, err
    assert err[2] > 10 * BAR, err
