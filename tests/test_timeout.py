"""Bounded waits: a wait that can never complete makes the launch report
GZ_ERR_DEVICE_TIMEOUT instead of hanging, and the context stays usable.  The
condition is produced with the library's own test knob (the MMA warp withholds
the accumulator-ready signal); nothing faults or traps."""
import pytest
import torch

import gemm_zoo_b200 as gz
from gemm_zoo_b200 import api
from tests.helpers import Case, check

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("config", [gz.CFG_1CTA_N128, gz.CFG_2CTA_N256, gz.CFG_2CTA_M512_N256])
def test_withheld_signal_times_out_and_context_survives(config):
    m, n, k = 512, 512, 256
    a = torch.ones(m, k, dtype=torch.bfloat16, device="cuda:0")
    b = torch.ones(n, k, dtype=torch.bfloat16, device="cuda:0")
    d = torch.zeros(m, n, dtype=torch.bfloat16, device="cuda:0")
    g = gz.Sm100Gemm(m, n, k, gz.DT_BF16, gz.DT_BF16, layout_b=gz.COL_MAJOR, config=config,
                     flags=gz.FLAG_TEST_WITHHOLD_ACC_READY, wait_limit_ns=2_000_000)
    g(a, b, None, d, 1.0, 0.0)
    status, detail = g.plan.device_status()
    assert status == api.GZ_ERR_DEVICE_TIMEOUT
    assert detail[0] in (3, 4)  # the epilogue (or the MMA warp behind it) gave up
    # the status word is cleared by the read
    assert g.plan.device_status()[0] == api.GZ_OK
    # the context is intact: a normal GEMM right after is correct
    torch.cuda.synchronize()
    r = check(Case(gz.DT_BF16, gz.DT_BF16, 300, 520, 256, b_col=True, config=config))
    assert r["ok"], r
