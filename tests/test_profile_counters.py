"""Stall counters and timeline (gz_gemm_plan_set_profile): the kernel writes
GZ_PROFILE_WORDS_PER_CTA words per CTA and nothing beyond them, the timeline is ordered, and the
binding refuses buffers that are too small or of the wrong kind."""
import pytest
import torch

import gemm_zoo_b200 as gz
from gemm_zoo_b200 import api

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.mark.parametrize("config", [gz.CFG_2CTA_N256, gz.CFG_2CTA_M512_N256, gz.CFG_1CTA_N64])
def test_counters_stay_inside_their_words_per_cta(config):
    m = n = 2048
    k = 512
    a = torch.randn(m, k, device=DEV).bfloat16()
    b = torch.randn(n, k, device=DEV).bfloat16()
    d = torch.empty(m, n, dtype=torch.bfloat16, device=DEV)
    g = gz.Sm100Gemm(m, n, k, gz.DT_BF16, gz.DT_BF16, layout_b=gz.COL_MAJOR, config=config)
    grid = g.info().grid
    guard = 1024
    sentinel = 0x5A5A5A5A5A5A5A5A
    W = gz.PROFILE_WORDS_PER_CTA
    buf = torch.full((W * grid + guard,), sentinel, dtype=torch.int64, device=DEV)
    g.plan.set_profile(buf)
    g(a, b, None, d, 1.0, 0.0)
    torch.cuda.synchronize()
    assert g.plan.device_status()[0] == api.GZ_OK
    words = buf.cpu()
    assert bool((words[W * grid:] == sentinel).all()), "the kernel wrote past its words per CTA"
    per_cta = words[:W * grid].view(grid, W)
    assert bool((per_cta[:, 15] != sentinel).all())  # every CTA recorded its lifetime
    assert bool((per_cta[:, 15] > 0).all())
    # the timeline of every CTA is ordered: entry <= dependencies satisfied <= exit
    assert bool((per_cta[:, 16] <= per_cta[:, 17]).all()) and bool((per_cta[:, 17] <= per_cta[:, 23]).all())
    lead = per_cta[per_cta[:, 18] != sentinel]  # CTAs whose MMA warp issued (the leader of a pair)
    assert len(lead) > 0
    assert bool((lead[:, 17] <= lead[:, 18]).all()) and bool((lead[:, 18] <= lead[:, 19]).all())
    assert bool((lead[:, 19] <= lead[:, 23]).all())
    # profiled and plain launches compute the same thing
    g.plan.set_profile(None)
    d2 = torch.empty_like(d)
    g(a, b, None, d2, 1.0, 0.0)
    torch.cuda.synchronize()
    assert torch.equal(d.view(torch.int16), d2.view(torch.int16))


def test_binding_refuses_buffers_the_kernel_would_overrun():
    g = gz.Sm100Gemm(1024, 1024, 256, gz.DT_BF16, gz.DT_BF16, layout_b=gz.COL_MAJOR, config=gz.CFG_2CTA_N256)
    grid = g.info().grid
    with pytest.raises(ValueError):
        g.plan.set_profile(torch.zeros(16 * grid, dtype=torch.int64, device=DEV))  # too small
    with pytest.raises(ValueError):
        g.plan.set_profile(torch.zeros(24 * grid, dtype=torch.int32, device=DEV))  # wrong element type
    with pytest.raises(ValueError):
        g.plan.set_profile(torch.zeros(24 * grid, dtype=torch.int64))              # host memory
    with pytest.raises(ValueError):
        g.plan.set_profile(12345)                                                  # a raw address
    g.plan.set_profile(torch.zeros(gz.PROFILE_WORDS_PER_CTA * grid, dtype=torch.int64, device=DEV))
    g.plan.set_profile(None)
