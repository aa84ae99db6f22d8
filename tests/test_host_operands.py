"""gz_gemm_run_host: the end-to-end entry point that takes HOST operands.  Small problems use one
upload / launch / download; large ones are pipelined in column blocks over two copy streams.  Both
must equal the device-operand entry point bit for bit (the column blocks use the same kernels, and
each output element is summed over K in the same order)."""
import pytest
import torch

import gemm_zoo_b200 as gz

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.mark.parametrize("in_t,out_t,tin,tout", [(gz.DT_BF16, gz.DT_BF16, torch.bfloat16, torch.bfloat16),
                                                 (gz.DT_S8, gz.DT_S32, torch.int8, torch.int32),
                                                 (gz.DT_F32, gz.DT_F32, torch.float32, torch.float32)])
@pytest.mark.parametrize("m,n,k,b_col,beta", [(300, 520, 256, True, 0), (1024, 8192, 1024, True, 0),
                                              (1024, 8192 + 300, 1024, True, 1), (512, 6144, 2048, False, 1),
                                              (2048, 2048 + 8, 1024, False, 0)])
def test_host_operands_match_device_operands(in_t, out_t, tin, tout, m, n, k, b_col, beta):
    gen = torch.Generator().manual_seed(m + n)
    if tin == torch.int8:
        a = torch.randint(-128, 128, (m, k), dtype=tin, generator=gen)
        b = torch.randint(-128, 128, (n, k) if b_col else (k, n), dtype=tin, generator=gen)
        c = torch.randint(-1000, 1000, (m, n), dtype=tout, generator=gen)
        alpha = 2
    else:
        a = torch.randn(m, k, generator=gen).to(tin)
        b = (torch.randn((n, k) if b_col else (k, n), generator=gen) * k ** -0.5).to(tin)
        c = torch.randn(m, n, generator=gen).to(tout)
        alpha = 1.5
    a, b, c = a.pin_memory(), b.pin_memory(), c.pin_memory()
    g = gz.Sm100Gemm(m, n, k, in_t, out_t, layout_b=gz.COL_MAJOR if b_col else gz.ROW_MAJOR)
    want = torch.empty(m, n, dtype=tout, device=DEV)
    g(a.to(DEV), b.to(DEV), c.to(DEV) if beta else None, want, alpha, beta)
    torch.cuda.synchronize()
    for _ in range(2):  # the second call reuses the staging buffers, streams and block plans
        got = torch.full((m, n), 3, dtype=tout).pin_memory()
        g.plan.run_host(a, b, c if beta else None, got, alpha, beta)
        if tout == torch.float32:
            # column blocks may pick another tile shape; tf32 sums stay within a few ulps
            assert torch.allclose(got, want.cpu(), rtol=1e-5, atol=1e-4)
        else:
            assert torch.equal(got, want.cpu())
    assert g.plan.device_status()[0] == 0


@pytest.mark.parametrize("m,n,k", [(300, 520, 256), (1024, 8192 + 300, 1024)])
def test_resident_a_host_b_matches_device_operands(m, n, k):
    """gz_gemm_run_host_ex with GZ_HOST_A_ON_DEVICE: A already sits in the GPU's memory (the
    replicated operand of a column-partitioned run), B, C and D are host memory; the result equals
    the device-operand run bit for bit, also when A only becomes valid through work queued on the
    caller's stream just before the call (the call's own work is ordered after it)."""
    gen = torch.Generator().manual_seed(m)
    a = torch.randn(m, k, generator=gen).bfloat16().pin_memory()
    b = (torch.randn(n, k, generator=gen) * k ** -0.5).bfloat16().pin_memory()
    c = torch.randn(m, n, generator=gen).bfloat16().pin_memory()
    g = gz.Sm100Gemm(m, n, k, gz.DT_BF16, gz.DT_BF16, layout_b=gz.COL_MAJOR)
    want = torch.empty(m, n, dtype=torch.bfloat16, device=DEV)
    g(a.to(DEV), b.to(DEV), c.to(DEV), want, 1.5, 1.0)
    torch.cuda.synchronize()
    stream = torch.cuda.current_stream()
    a_dev = torch.zeros(m, k, dtype=torch.bfloat16, device=DEV)
    for call in range(2):
        a_dev.zero_()
        a_dev.copy_(a, non_blocking=True)  # queued on the caller's stream, not yet done when the call starts
        got = torch.full((m, n), 3, dtype=torch.bfloat16).pin_memory()
        g.plan.run_host(a_dev, b, c, got, 1.5, 1.0, stream, a_on_device=True)
        assert torch.equal(got.view(torch.int16), want.cpu().view(torch.int16)), call
    # the same plan still takes a host A afterwards
    got = torch.full((m, n), 3, dtype=torch.bfloat16).pin_memory()
    g.plan.run_host(a, b, c, got, 1.5, 1.0, stream)
    assert torch.equal(got.view(torch.int16), want.cpu().view(torch.int16))
    assert g.plan.device_status()[0] == 0
