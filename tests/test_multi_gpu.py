"""N-column partition across the GPUs of one box: B sharded, A replicated, D shards
local, one plan per device, no collective.  The gathered result equals the
single-GPU result bit for bit (same kernel, same per-element summation order).
Skipped when fewer than two GPUs are visible."""
import pytest
import torch

import gemm_zoo_b200 as gz

pytestmark = pytest.mark.gpu


def test_partition_across_devices_bitwise():
    ndev = torch.cuda.device_count()
    if ndev < 2:
        pytest.skip("needs at least two GPUs")
    parts = min(ndev, 8)
    m, n, k = 2048, 8192, 4096
    a0 = torch.empty(m, k, dtype=torch.bfloat16, device="cuda:0")
    b0 = torch.empty(n, k, dtype=torch.bfloat16, device="cuda:0")
    gz.fill(a0, 21, 1, 1, 1.0)
    gz.fill(b0, 21, 2, 1, k ** -0.5)
    full = torch.empty(m, n, dtype=torch.bfloat16, device="cuda:0")
    gz.Sm100Gemm(m, n, k, gz.DT_BF16, gz.DT_BF16, layout_b=gz.COL_MAJOR, device=0)(a0, b0, None, full, 1.0, 0.0)
    shards = []
    for p in range(parts):
        lo, hi = gz.partition_columns(n, parts, p, 8)
        dev = torch.device("cuda", p)
        with torch.cuda.device(dev):
            a = torch.empty(m, k, dtype=torch.bfloat16, device=dev)
            gz.fill(a, 21, 1, 1, 1.0)                 # A regenerated in place on every GPU
            b = b0[lo:hi].to(dev)                      # this GPU's column block of B
            d = torch.empty(m, hi - lo, dtype=torch.bfloat16, device=dev)
            g = gz.Sm100Gemm(m, hi - lo, k, gz.DT_BF16, gz.DT_BF16, layout_b=gz.COL_MAJOR, device=p)
            g(a, b, None, d, 1.0, 0.0)
            assert g.plan.device_status()[0] == 0
            shards.append(d.cpu())
    got = torch.cat(shards, dim=1)
    assert torch.equal(got.view(torch.int16), full.cpu().view(torch.int16))


def test_entry_points_leave_the_current_device_alone():
    """Plans for another GPU are created, run, queried and destroyed while device 0 stays the
    calling thread's current device, and gz_fill runs on the GPU that owns the buffer."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least two GPUs")
    import ctypes as C
    rt = C.CDLL("libcudart.so.12")
    def current():
        d = C.c_int(-1)
        assert rt.cudaGetDevice(C.byref(d)) == 0
        return d.value
    torch.cuda.set_device(0)
    assert current() == 0
    m, n, k = 256, 512, 256
    a = torch.empty(m, k, dtype=torch.bfloat16, device="cuda:1")
    b = torch.empty(n, k, dtype=torch.bfloat16, device="cuda:1")
    gz.fill(a, 3, 1, 2, 3.0)
    gz.fill(b, 3, 2, 2, 3.0)
    assert current() == 0
    d = torch.zeros(m, n, dtype=torch.bfloat16, device="cuda:1")
    g = gz.Sm100Gemm(m, n, k, gz.DT_BF16, gz.DT_BF16, layout_b=gz.COL_MAJOR, device=1)
    assert current() == 0
    g(a, b, None, d, 1.0, 0.0)
    assert current() == 0
    assert g.plan.device_status()[0] == 0 and current() == 0
    g.plan.destroy()
    assert current() == 0
    want = (a.double() @ b.double().t()).to(torch.bfloat16)
    assert torch.equal(d.cpu(), want.cpu())
    # device 0 work right after is unaffected
    x = torch.empty(1 << 12, dtype=torch.float32, device="cuda:0")
    gz.fill(x, 1, 1, 0)
    torch.cuda.synchronize()
    assert x.abs().max().item() <= 1.0
