"""The no-allocation entry point, gz_gemm_skinny_static.

Some hosts give all device memory to their own allocator at start-up and must not call cudaMalloc
afterwards (it can fail against their budget and it synchronises the device in a latency-critical
loop), so they cannot create a plan.  For them the skinny split-K GEMM exists once more with its
scratch memory (partial sums, arrival counters, status words) in a fixed array inside the library.

Checked here, through the C ABI: its output equals the output of the plan-based entry point (same
kernel, same K split, so the comparison is bit for bit) on two calls in a row — the second call
finds the array as the first one left it — for a floating-point and an integer problem; problems
whose partial sums exceed the array are refused; and no device memory is allocated by the calls.
This file is collected last so that a run that stops at the first failure has run everything else.
"""
import pytest
import torch

import gemm_zoo_b200 as gz
from gemm_zoo_b200 import api

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _operands(in_t, m, n, k, seed):
    gen = torch.Generator(device=DEV).manual_seed(seed)
    if in_t == gz.DT_S8:
        a = torch.randint(-128, 128, (m, k), dtype=torch.int8, device=DEV, generator=gen)
        b = torch.randint(-128, 128, (n, k), dtype=torch.int8, device=DEV, generator=gen)
        c = torch.randint(-1000, 1000, (m, n), dtype=torch.int32, device=DEV, generator=gen)
        return a, b, c, torch.int32, 3, -2
    a = torch.randn(m, k, device=DEV, generator=gen).bfloat16()
    b = (torch.randn(n, k, device=DEV, generator=gen) * k ** -0.5).bfloat16()
    c = torch.randn(m, n, device=DEV, generator=gen).bfloat16()
    return a, b, c, torch.bfloat16, 1.5, 0.5


@pytest.mark.parametrize("in_t,out_t,m,n,k", [(gz.DT_BF16, gz.DT_BF16, 16, 4096, 4096),
                                               (gz.DT_BF16, gz.DT_BF16, 64, 1000, 4096),
                                               (gz.DT_S8, gz.DT_S32, 33, 2048, 8192)])
def test_static_scratch_entry_point_matches_plan_entry_point_twice(in_t, out_t, m, n, k):
    a, b, c, odt, alpha, beta = _operands(in_t, m, n, k, seed=m)
    desc = gz.GemmDesc.make(in_t, out_t, m, n, k, layout_b=gz.COL_MAJOR)
    # Reference result: the existing entry point, told to split K the same way.
    want = torch.empty(m, n, dtype=odt, device=DEV)
    config = (gz.CFG_SWAP_M16 if m <= 16 else gz.CFG_SWAP_M32 if m <= 32 else gz.CFG_SWAP_M64 if m <= 64
              else gz.CFG_SWAP_M128)
    plan = gz.Sm100Gemm(m, n, k, in_t, out_t, layout_b=gz.COL_MAJOR, config=config, flags=gz.FLAG_SPLIT_K)
    assert plan.info().split_k == 1
    plan(a, b, c, want, alpha, beta)
    torch.cuda.synchronize()
    assert plan.plan.device_status()[0] == 0

    before = torch.cuda.memory_allocated()
    free_before, _ = torch.cuda.mem_get_info()
    for call in range(2):
        got = torch.full((m, n), 7, dtype=odt, device=DEV)
        st = gz.gemm_skinny_static(desc, a, b, c, got, alpha, beta)
        assert st == api.GZ_OK, gz.status_string(st)
        torch.cuda.synchronize()
        if odt == torch.int32:
            assert torch.equal(got, want), f"call {call}"
        else:
            assert torch.equal(got.view(torch.int16), want.view(torch.int16)), f"call {call}"
    # in place as well: D aliases C
    c2 = c.clone()
    assert gz.gemm_skinny_static(desc, a, b, c2, c2, alpha, beta) == api.GZ_OK
    torch.cuda.synchronize()
    assert torch.equal(c2, want)
    free_after, _ = torch.cuda.mem_get_info()
    # nothing but the two `got` tensors and the clone came from this test; the library allocated nothing
    assert free_before - free_after <= 3 * want.numel() * want.element_size() + (4 << 20)
    assert torch.cuda.memory_allocated() >= before


def test_static_scratch_refuses_what_does_not_fit_or_is_not_skinny():
    big = gz.GemmDesc.make(gz.DT_BF16, gz.DT_BF16, 128, 148 * 128, 128 * 64, layout_b=gz.COL_MAJOR)
    x = torch.zeros(16, dtype=torch.bfloat16, device=DEV)
    st = gz.gemm_skinny_static(big, x, x, None, x, 1.0, 0.0)
    assert st == api.GZ_ERR_TOO_LARGE
    assert b"static scratch too small" in gz.lib().gz_last_cuda_error()
    wide = gz.GemmDesc.make(gz.DT_BF16, gz.DT_BF16, 129, 4096, 4096, layout_b=gz.COL_MAJOR)
    assert gz.gemm_skinny_static(wide, x, x, None, x, 1.0, 0.0) == api.GZ_ERR_UNSUPPORTED
    odd = gz.GemmDesc.make(gz.DT_BF16, gz.DT_BF16, 16, 4096, 1001, layout_b=gz.COL_MAJOR)
    assert gz.gemm_skinny_static(odd, x, x, None, x, 1.0, 0.0) == api.GZ_ERR_MISALIGNED
    assert gz.lib().gz_gemm_skinny_static(None, None, None, None, None, None, None, None) == api.GZ_ERR_INVALID_ARG
