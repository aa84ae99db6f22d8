"""The die-aware tile order.

A B200 is two dies; the plan measures once per device which die each SM sits on (a pointer chase
through L2-resident lines from every SM, classified on the host) and, for problems of several
waves of tiles, lets the CTA pairs of one die take neighbouring tiles.  Checked here:
  CPU   the host-side classification on a matrix of clocks recorded on a B200 (70 + 78 SMs), and
        that it refuses pictures that are not two-sided;
  GPU   the measurement agrees with itself, the order is on for large problems and off where it
        cannot pay, results are bit for bit those of the plain order, the ticket counters clean up
        after themselves over more launches than there are counter sets, and two launches in flight
        at once on different streams do not disturb each other."""
from pathlib import Path

import numpy as np
import pytest
import torch

import gemm_zoo_b200 as gz
from gemm_zoo_b200 import api

GOLDEN = Path(__file__).resolve().parent / "golden" / "b200_sm_line_clocks.npy"
# SMs of the recorded part that share a die with SM 0 (the other 78 share the other die)
DIE0 = ([0, 1, 2, 3] + list(range(12, 20)) + list(range(28, 36)) + list(range(44, 52)) + list(range(60, 68)) +
        list(range(76, 82)) + list(range(90, 96)) + list(range(104, 110)) + list(range(118, 124)) +
        list(range(132, 136)) + list(range(138, 144)))


def test_classification_of_a_recorded_b200():
    clocks = np.load(GOLDEN)  # [148 SMs][96 lines], clocks per dependent load
    assert clocks.shape == (148, 96)
    st, dies, counts = gz.classify_dies(clocks)
    assert st == api.GZ_OK and counts == [70, 78]
    assert [s for s, d in enumerate(dies) if d == 0] == DIE0
    # half of the lines are enough, and the answer does not depend on which SM is listed first
    st, dies48, counts48 = gz.classify_dies(clocks[:, :48])
    assert st == api.GZ_OK and dies48 == dies
    st, rolled, counts_r = gz.classify_dies(np.roll(clocks, -4, axis=0))  # SM 4 (other die) comes first
    assert st == api.GZ_OK and counts_r == [78, 70]
    assert [1 - d for d in np.roll(np.array(rolled), 4)] == dies


def test_classification_refuses_what_is_not_two_sided():
    clocks = np.load(GOLDEN)
    rng = np.random.default_rng(0)
    assert gz.classify_dies(rng.integers(250, 300, size=(148, 48), dtype=np.uint32))[0] == api.GZ_ERR_UNSUPPORTED
    assert gz.classify_dies(np.full((148, 48), 260, dtype=np.uint32))[0] == api.GZ_ERR_UNSUPPORTED
    one_die = np.repeat(clocks[:1], 148, axis=0)
    assert gz.classify_dies(one_die)[0] == api.GZ_ERR_UNSUPPORTED
    mixed = clocks.copy()
    mixed[100:] = clocks[100:, ::-1]  # a third of the SMs see the lines in another order
    assert gz.classify_dies(mixed)[0] == api.GZ_ERR_UNSUPPORTED
    lopsided = clocks.copy()
    lopsided[[s for s in range(148) if s not in DIE0][8:]] = clocks[0]  # only 8 SMs left on the second die
    assert gz.classify_dies(lopsided)[0] == api.GZ_ERR_UNSUPPORTED


DEV = "cuda:0"


def _operands(m, n, k, seed):
    a = torch.empty(m, k, dtype=torch.bfloat16, device=DEV)
    b = torch.empty(n, k, dtype=torch.bfloat16, device=DEV)
    gz.fill(a, seed, 1, 1, 1.0)
    gz.fill(b, seed, 2, 1, k ** -0.5)
    return a, b


def _need_placement():
    """The probe times L2 hits; where it cannot classify a chip (after its retries) the library runs
    without the die-aware order, which is correct behaviour and leaves nothing to test here."""
    if gz.device_placement(0)[0] != api.GZ_OK:
        pytest.skip("die placement of this chip could not be measured: the die-aware order is off")


@pytest.mark.gpu
def test_measured_placement_is_two_dies_and_stable():
    _need_placement()
    st, dies, counts = gz.device_placement(0)
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    assert sum(counts) == sms and min(counts) * 4 >= sms
    assert all(dies[s] == dies[s ^ 1] for s in range(sms))  # the two SMs of a TPC share a die
    assert gz.device_placement(0)[1] == dies  # measured once per process


@pytest.mark.gpu
def test_order_is_on_where_it_pays_and_results_do_not_depend_on_it():
    _need_placement()
    m = n = 4096
    k = 1024
    a, b = _operands(m, n, k, 41)
    on = gz.Sm100Gemm(m, n, k, gz.DT_BF16, gz.DT_BF16, layout_b=gz.COL_MAJOR, config=gz.CFG_2CTA_N128)
    off = gz.Sm100Gemm(m, n, k, gz.DT_BF16, gz.DT_BF16, layout_b=gz.COL_MAJOR, config=gz.CFG_2CTA_N128,
                       flags=gz.FLAG_NO_DIE_ORDER)
    assert on.info().die_order == 1 and off.info().die_order == 0  # 512 tiles on 74 CTA pairs
    small = gz.Sm100Gemm(1024, 1024, 1024, gz.DT_BF16, gz.DT_BF16, layout_b=gz.COL_MAJOR)
    skinny = gz.Sm100Gemm(16, 14336, 4096, gz.DT_BF16, gz.DT_BF16, layout_b=gz.COL_MAJOR)
    assert small.info().die_order == 0 and skinny.info().die_order == 0
    want = torch.empty(m, n, dtype=torch.bfloat16, device=DEV)
    off(a, b, None, want, 1.0, 0.0)
    torch.cuda.synchronize()
    # more launches than the plan has counter sets: every set is used again after it cleaned itself up
    for i in range(2 * 32 + 3):
        got = torch.zeros(m, n, dtype=torch.bfloat16, device=DEV)
        on(a, b, None, got, 1.0, 0.0)
        if i % 16 == 0 or i > 60:
            assert torch.equal(got.view(torch.int16), want.view(torch.int16)), i
    assert on.plan.device_status()[0] == 0


@pytest.mark.gpu
@pytest.mark.parametrize("config", [gz.CFG_2CTA_M512_N256, gz.CFG_2CTA_N256, gz.CFG_1CTA_N128])
def test_every_tile_family_with_the_order_on(config):
    _need_placement()
    m, n, k = 8192, 4096 + 256, 512
    a, b = _operands(m, n, k, 43)
    c = torch.randn(m, n, device=DEV).bfloat16()
    on = gz.Sm100Gemm(m, n, k, gz.DT_BF16, gz.DT_BF16, layout_b=gz.COL_MAJOR, config=config)
    off = gz.Sm100Gemm(m, n, k, gz.DT_BF16, gz.DT_BF16, layout_b=gz.COL_MAJOR, config=config,
                       flags=gz.FLAG_NO_DIE_ORDER)
    assert on.info().die_order == 1
    want, got = (torch.zeros(m, n, dtype=torch.bfloat16, device=DEV) for _ in range(2))
    off(a, b, c, want, 1.5, 0.5)
    on(a, b, c, got, 1.5, 0.5)
    torch.cuda.synchronize()
    assert torch.equal(got.view(torch.int16), want.view(torch.int16))
    assert on.plan.device_status()[0] == 0


@pytest.mark.gpu
def test_two_launches_in_flight_on_two_streams():
    _need_placement()
    m = n = 4096
    k = 2048
    a, b = _operands(m, n, k, 47)
    a2, b2 = _operands(m, n, k, 53)
    g = gz.Sm100Gemm(m, n, k, gz.DT_BF16, gz.DT_BF16, layout_b=gz.COL_MAJOR)
    assert g.info().die_order == 1
    ref = gz.Sm100Gemm(m, n, k, gz.DT_BF16, gz.DT_BF16, layout_b=gz.COL_MAJOR, flags=gz.FLAG_NO_DIE_ORDER)
    want1, want2 = (torch.empty(m, n, dtype=torch.bfloat16, device=DEV) for _ in range(2))
    ref(a, b, None, want1, 1.0, 0.0)
    ref(a2, b2, None, want2, 1.0, 0.0)
    torch.cuda.synchronize()
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
    for _ in range(5):
        d1, d2 = (torch.zeros(m, n, dtype=torch.bfloat16, device=DEV) for _ in range(2))
        torch.cuda.synchronize()
        g(a, b, None, d1, 1.0, 0.0, s1)   # the two launches share the plan and compete for the SMs
        g(a2, b2, None, d2, 1.0, 0.0, s2)
        torch.cuda.synchronize()
        assert torch.equal(d1.view(torch.int16), want1.view(torch.int16))
        assert torch.equal(d2.view(torch.int16), want2.view(torch.int16))
    assert g.plan.device_status()[0] == 0
