"""The no-allocation entry point, gz_gemm_skinny_static.

Some hosts give all device memory to their own allocator at start-up and must not call cudaMalloc
afterwards (it can fail against their budget and it synchronises the device in a latency-critical
loop), so they cannot create a plan.  For them the skinny split-K GEMM exists once more with its
scratch memory (partial sums, arrival counters, status words) in a fixed array inside the library.

Checked here, through the C ABI: its output equals the output of the plan-based entry point (same
kernel, same K split, so the comparison is bit for bit; the plan entry point is itself checked
against the CPU oracle in test_gemm_parity.py) on two calls in a row — the second call finds the
array as the first one left it — for floating-point, integer and dequantising problems; problems
whose partial sums exceed the array are refused; the calls leave the device's free-memory count
exactly where it was; and a bounded wait that expires on this path is reported by
gz_static_last_device_status, after which the entry point works again.
This file is collected last so that a run that stops at the first failure has run everything else.
"""
import pytest
import torch

import gemm_zoo_b200 as gz
from gemm_zoo_b200 import api

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _operands(in_t, out_t, m, n, k, seed):
    gen = torch.Generator(device=DEV).manual_seed(seed)
    if in_t == gz.DT_S8:
        a = torch.randint(-128, 128, (m, k), dtype=torch.int8, device=DEV, generator=gen)
        b = torch.randint(-128, 128, (n, k), dtype=torch.int8, device=DEV, generator=gen)
        if out_t == gz.DT_S32:
            c = torch.randint(-1000, 1000, (m, n), dtype=torch.int32, device=DEV, generator=gen)
            return a, b, c, torch.int32, 3, -2
        c = torch.randn(m, n, device=DEV, generator=gen).bfloat16()
        return a, b, c, torch.bfloat16, 2.0 ** -10, 0.5  # a dequantising scale: float scalars on s8 inputs
    a = torch.randn(m, k, device=DEV, generator=gen).bfloat16()
    b = (torch.randn(n, k, device=DEV, generator=gen) * k ** -0.5).bfloat16()
    c = torch.randn(m, n, device=DEV, generator=gen).bfloat16()
    return a, b, c, torch.bfloat16, 1.5, 0.5


def _swap_config(m):
    return (gz.CFG_SWAP_M16 if m <= 16 else gz.CFG_SWAP_M32 if m <= 32 else gz.CFG_SWAP_M64 if m <= 64
            else gz.CFG_SWAP_M128)


def _bits(t):
    return t.view(torch.int16) if t.element_size() == 2 else t.view(torch.int32)


@pytest.mark.parametrize("in_t,out_t,m,n,k", [(gz.DT_BF16, gz.DT_BF16, 16, 4096, 4096),
                                               (gz.DT_BF16, gz.DT_BF16, 64, 1000, 4096),
                                               (gz.DT_S8, gz.DT_S32, 33, 2048, 8192),
                                               (gz.DT_S8, gz.DT_BF16, 16, 2048, 4096)])
def test_static_scratch_entry_point_matches_plan_entry_point_twice(in_t, out_t, m, n, k):
    a, b, c, odt, alpha, beta = _operands(in_t, out_t, m, n, k, seed=m)
    desc = gz.GemmDesc.make(in_t, out_t, m, n, k, layout_b=gz.COL_MAJOR)
    # Reference result: the existing entry point, told to split K the same way.
    want = torch.empty(m, n, dtype=odt, device=DEV)
    plan = gz.Sm100Gemm(m, n, k, in_t, out_t, layout_b=gz.COL_MAJOR, config=_swap_config(m), flags=gz.FLAG_SPLIT_K)
    assert plan.info().split_k == 1
    plan(a, b, c, want, alpha, beta)
    torch.cuda.synchronize()
    assert plan.plan.device_status()[0] == 0
    assert bool(want.float().abs().sum() > 0)

    # Everything this test needs is allocated BEFORE the free-memory count is read, and the entry
    # point has run once (its first call on a device loads the kernel and takes the array's address).
    got = [torch.full((m, n), 7, dtype=odt, device=DEV) for _ in range(2)]
    c2 = c.clone()
    warm = torch.empty_like(want)
    assert gz.gemm_skinny_static(desc, a, b, c, warm, alpha, beta) == api.GZ_OK
    assert gz.static_device_status(0)[0] == api.GZ_OK
    torch.cuda.synchronize()
    allocated_before = torch.cuda.memory_allocated()
    free_before, _ = torch.cuda.mem_get_info()
    for call in range(2):
        st = gz.gemm_skinny_static(desc, a, b, c, got[call], alpha, beta)
        assert st == api.GZ_OK, gz.status_string(st)
    # in place as well: D aliases C
    assert gz.gemm_skinny_static(desc, a, b, c2, c2, alpha, beta) == api.GZ_OK
    st, detail = gz.static_device_status(0)
    assert st == api.GZ_OK, detail
    free_after, _ = torch.cuda.mem_get_info()
    # The split-K workspace of these problems is 0.3 - 1.6 MB: had the library allocated it (or
    # anything else), the driver's free count would have moved.
    assert free_after == free_before
    assert torch.cuda.memory_allocated() == allocated_before
    for call in range(2):
        assert torch.equal(_bits(got[call]), _bits(want)), f"call {call}"
    assert torch.equal(_bits(warm), _bits(want))
    assert torch.equal(_bits(c2), _bits(want))


def test_static_scratch_reports_an_expired_wait_and_works_again():
    m, n, k = 16, 2048, 4096
    a, b, c, odt, alpha, beta = _operands(gz.DT_BF16, gz.DT_BF16, m, n, k, seed=5)
    d = torch.zeros(m, n, dtype=odt, device=DEV)
    assert gz.static_device_status(0)[0] == api.GZ_OK
    # The library's own test knob: the MMA warp never signals "accumulator ready", so the epilogue's
    # bounded wait (2 ms here) runs out.  Nothing faults, traps or hangs.
    held = gz.GemmDesc.make(gz.DT_BF16, gz.DT_BF16, m, n, k, layout_b=gz.COL_MAJOR,
                            flags=gz.FLAG_TEST_WITHHOLD_ACC_READY, wait_limit_ns=2_000_000)
    assert gz.gemm_skinny_static(held, a, b, None, d, 1.0, 0.0) == api.GZ_OK  # the launch itself succeeds
    st, detail = gz.static_device_status(0)
    assert st == api.GZ_ERR_DEVICE_TIMEOUT
    assert detail[0] in (3, 4)  # the epilogue (or the MMA warp behind it) gave up
    assert gz.static_device_status(0)[0] == api.GZ_OK  # cleared by the read
    # The array and the context are intact: the next call is correct although the aborted launch
    # left arrival counters behind.
    desc = gz.GemmDesc.make(gz.DT_BF16, gz.DT_BF16, m, n, k, layout_b=gz.COL_MAJOR)
    want = torch.empty(m, n, dtype=odt, device=DEV)
    plan = gz.Sm100Gemm(m, n, k, gz.DT_BF16, gz.DT_BF16, layout_b=gz.COL_MAJOR, config=gz.CFG_SWAP_M16,
                        flags=gz.FLAG_SPLIT_K)
    plan(a, b, c, want, alpha, beta)
    assert gz.gemm_skinny_static(desc, a, b, c, d, alpha, beta) == api.GZ_OK
    assert gz.static_device_status(0)[0] == api.GZ_OK
    assert torch.equal(_bits(d), _bits(want))


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
