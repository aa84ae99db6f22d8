"""Size-independent properties checked on the GPU, some at the largest benchmark
size (bf16 16384^3): multiplying by the identity returns A bit for bit, a
column-partitioned run equals the unpartitioned one bit for bit, repeated runs are
bitwise identical, and integer GEMM is linear."""
import numpy as np
import pytest
import torch

import gemm_zoo_b200 as gz

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def test_identity_at_16384_cubed_bf16():
    n = 16384
    a = torch.empty(n, n, dtype=torch.bfloat16, device=DEV)
    gz.fill(a, 5, 1, 1, 1.0 / 128)
    eye = torch.zeros(n, n, dtype=torch.bfloat16, device=DEV)
    eye.diagonal().fill_(1.0)
    d = torch.empty(n, n, dtype=torch.bfloat16, device=DEV)
    g = gz.Sm100Gemm(n, n, n, gz.DT_BF16, gz.DT_BF16, layout_b=gz.COL_MAJOR)
    g(a, eye, None, d, 1.0, 0.0)
    assert g.plan.device_status()[0] == 0
    # bit for bit, except that -0 * 1 + (+0 + ...) is +0: zeros are compared by value
    same_bits = d.view(torch.int16) == a.view(torch.int16)
    assert bool((same_bits | ((d == 0) & (a == 0))).all())
    # and a column permutation: D[:, j] = A[:, perm[j]]  (B col-major: row j of the buffer is column j of B)
    perm = torch.randperm(n, device=DEV, generator=torch.Generator(device=DEV).manual_seed(1))
    pmat = torch.zeros(n, n, dtype=torch.bfloat16, device=DEV)
    pmat[torch.arange(n, device=DEV), perm] = 1.0
    g(a, pmat, None, d, 1.0, 0.0)
    want = a[:, perm].contiguous()
    assert bool(((d.view(torch.int16) == want.view(torch.int16)) | ((d == 0) & (want == 0))).all())


def test_identity_s8_8192():
    n = 8192
    a = torch.empty(n, n, dtype=torch.int8, device=DEV)
    gz.fill(a, 3, 1, 2)
    eye = torch.zeros(n, n, dtype=torch.int8, device=DEV)
    eye.diagonal().fill_(1)
    d = torch.empty(n, n, dtype=torch.int32, device=DEV)
    g = gz.Sm100Gemm(n, n, n, gz.DT_S8, gz.DT_S32, layout_b=gz.COL_MAJOR)
    g(a, eye, None, d, 1, 0)
    assert torch.equal(d, a.to(torch.int32))


def test_row_sum_checksum_bf16_8192():
    """sum_j D[i, j] == A[i, :] . (sum_j B[:, j]) — a checksum of the whole product."""
    m = n = k = 8192
    a = torch.empty(m, k, dtype=torch.bfloat16, device=DEV)
    b = torch.empty(n, k, dtype=torch.bfloat16, device=DEV)
    gz.fill(a, 9, 1, 1, 1.0)
    gz.fill(b, 9, 2, 1, k ** -0.5)
    d = torch.empty(m, n, dtype=torch.float32, device=DEV)
    g = gz.Sm100Gemm(m, n, k, gz.DT_BF16, gz.DT_F32, layout_b=gz.COL_MAJOR)
    g(a, b, None, d, 1.0, 0.0)
    got = d.double().sum(dim=1)
    want = a.double() @ b.double().sum(dim=0)
    scale = a.double().abs() @ b.double().abs().sum(dim=0)
    assert ((got - want).abs() <= 2.0 ** -18 * scale).all()


@pytest.mark.parametrize("parts", [2, 4, 8])
def test_column_partition_equals_full_run_bitwise(parts):
    m, n, k = 1024, 4096 + 256, 2048
    a = torch.empty(m, k, dtype=torch.bfloat16, device=DEV)
    b = torch.empty(n, k, dtype=torch.bfloat16, device=DEV)  # column-major: a shard is a contiguous block
    gz.fill(a, 11, 1, 1, 1.0)
    gz.fill(b, 11, 2, 1, k ** -0.5)
    full = torch.empty(m, n, dtype=torch.bfloat16, device=DEV)
    gz.Sm100Gemm(m, n, k, gz.DT_BF16, gz.DT_BF16, layout_b=gz.COL_MAJOR)(a, b, None, full, 1.0, 0.0)
    out = torch.zeros(m, n, dtype=torch.bfloat16, device=DEV)
    for p in range(parts):
        lo, hi = gz.partition_columns(n, parts, p, 8)
        if hi == lo:
            continue
        g = gz.Sm100Gemm(m, hi - lo, k, gz.DT_BF16, gz.DT_BF16, layout_b=gz.COL_MAJOR, ldd=n)
        g(a, b[lo:hi], None, out[:, lo:], 1.0, 0.0)
    torch.cuda.synchronize()
    assert torch.equal(out.view(torch.int16), full.view(torch.int16))


def test_repeated_runs_are_bitwise_identical():
    m, n, k = 2048, 2048, 4096
    a = torch.empty(m, k, dtype=torch.float16, device=DEV)
    b = torch.empty(n, k, dtype=torch.float16, device=DEV)
    gz.fill(a, 13, 1, 0, 1.0)
    gz.fill(b, 13, 2, 0, 1.0)
    g = gz.Sm100Gemm(m, n, k, gz.DT_F16, gz.DT_F16, layout_b=gz.COL_MAJOR)
    d1 = torch.empty(m, n, dtype=torch.float16, device=DEV)
    d2 = torch.empty_like(d1)
    g(a, b, None, d1, 1.0, 0.0)
    g(a, b, None, d2, 1.0, 0.0)
    assert torch.equal(d1.view(torch.int16), d2.view(torch.int16))
    # a different tile shape sums each output over k in the same order: still identical
    d3 = torch.empty_like(d1)
    gz.Sm100Gemm(m, n, k, gz.DT_F16, gz.DT_F16, layout_b=gz.COL_MAJOR, config=gz.CFG_1CTA_N128)(a, b, None, d3, 1.0, 0.0)
    assert torch.equal(d1.view(torch.int16), d3.view(torch.int16))


def test_integer_linearity():
    m, n, k = 512, 768, 1024
    gen = torch.Generator(device=DEV).manual_seed(17)
    a1 = torch.randint(-60, 60, (m, k), dtype=torch.int8, device=DEV, generator=gen)
    a2 = torch.randint(-60, 60, (m, k), dtype=torch.int8, device=DEV, generator=gen)
    b = torch.randint(-128, 128, (n, k), dtype=torch.int8, device=DEV, generator=gen)
    g = gz.Sm100Gemm(m, n, k, gz.DT_S8, gz.DT_S32, layout_b=gz.COL_MAJOR)
    d1, d2, d12 = (torch.empty(m, n, dtype=torch.int32, device=DEV) for _ in range(3))
    g(a1, b, None, d1, 1, 0)
    g(a2, b, None, d2, 1, 0)
    g((a1 + a2), b, None, d12, 1, 0)
    assert torch.equal(d12, d1 + d2)
    # accumulate through beta: D = A2*B + 1*D1
    g(a2, b, d1, d1, 1, 1)
    assert torch.equal(d1, d12)


def test_fill_is_deterministic_and_streams_differ():
    x = torch.empty(1 << 16, dtype=torch.float32, device=DEV)
    y = torch.empty_like(x)
    gz.fill(x, 1, 1, 0)
    gz.fill(y, 1, 1, 0)
    assert torch.equal(x, y)
    gz.fill(y, 1, 2, 0)
    assert not torch.equal(x, y)
    assert float(x.min()) >= -1.0 and float(x.max()) < 1.0
    gz.fill(x, 1, 1, 1, 2.0)
    assert abs(float(x.mean())) < 0.05 and abs(float(x.std()) - 2.0) < 0.05
    z = torch.empty(1 << 16, dtype=torch.int8, device=DEV)
    gz.fill(z, 1, 1, 2)
    assert int(z.min()) == -128 and int(z.max()) == 127
