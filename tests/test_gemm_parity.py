"""GPU parity tests: the CUDA path, called through the C ABI, against the CPU
oracle on the same seeded operands.  Integer work and exact-integer float inputs
are compared bit for bit; random float inputs within the bars in tests/helpers.py.
Every output buffer is wrapped in sentinel guard bands that must stay untouched."""
import pytest

import gemm_zoo_b200 as gz
from tests.helpers import Case, check

pytestmark = pytest.mark.gpu

F16, BF16, F32, S8, S32 = gz.DT_F16, gz.DT_BF16, gz.DT_F32, gz.DT_S8, gz.DT_S32
DIRECT, TMA = gz.FLAG_EPILOGUE_DIRECT, gz.FLAG_EPILOGUE_TMA
TC_CONFIGS = [gz.CFG_1CTA_N256, gz.CFG_1CTA_N128, gz.CFG_1CTA_N64, gz.CFG_2CTA_N256, gz.CFG_2CTA_N128]


def run(case):
    r = check(case)
    assert r["ok"], r
    return r


@pytest.mark.parametrize("config", TC_CONFIGS)
@pytest.mark.parametrize("flags", [DIRECT, TMA])
def test_single_and_multi_tile_bf16(config, flags):
    run(Case(BF16, BF16, 256, 256, 64, b_col=True, config=config, flags=flags))
    run(Case(BF16, F32, 384, 768, 320, b_col=True, config=config, flags=flags, alpha=2, beta=-1))
    run(Case(BF16, BF16, 100, 200, 72, b_col=True, config=config, flags=flags))


@pytest.mark.parametrize("config", TC_CONFIGS)
@pytest.mark.parametrize("in_t,out_t", [(F16, F16), (F16, F32), (BF16, BF16), (F32, F32), (S8, S32)])
def test_every_dtype_pair_k_major(config, in_t, out_t):
    dist = "full" if in_t == S8 else "int"
    run(Case(in_t, out_t, 300, 520, 400, b_col=True, config=config, dist=dist, alpha=3, beta=-2))


@pytest.mark.parametrize("a_col,b_col", [(False, False), (True, False), (True, True), (False, True)])
@pytest.mark.parametrize("in_t,out_t", [(BF16, F32), (F16, F16), (F32, F32), (S8, S32)])
@pytest.mark.parametrize("config", [gz.CFG_1CTA_N256, gz.CFG_2CTA_N256, gz.CFG_1CTA_N128])
def test_every_layout(a_col, b_col, in_t, out_t, config):
    dist = "full" if in_t == S8 else "int"
    run(Case(in_t, out_t, 384, 512, 384, a_col=a_col, b_col=b_col, config=config, dist=dist, alpha=1, beta=1))


@pytest.mark.parametrize("alpha,beta", [(1, 0), (1, 1), (1, 0.5), (0, 1), (-2, 3)])
@pytest.mark.parametrize("in_t,out_t", [(BF16, BF16), (F32, F32), (S8, S32)])
def test_alpha_beta(alpha, beta, in_t, out_t):
    if in_t == S8 and beta == 0.5:
        pytest.skip("integer scalars only")
    dist = "full" if in_t == S8 else ("normal" if beta == 0.5 else "int")
    run(Case(in_t, out_t, 200, 264, 192, b_col=True, dist=dist, alpha=alpha, beta=beta))


@pytest.mark.parametrize("m,n,k", [(1, 8, 8), (1, 1000, 64), (7, 16, 24), (128, 128, 8), (129, 257, 72),
                                   (255, 8, 1000), (300, 296, 136), (61, 1016, 40)])
@pytest.mark.parametrize("in_t,out_t", [(BF16, BF16), (F32, F32), (S8, S32)])
def test_ragged_shapes_auto_config(m, n, k, in_t, out_t):
    mult = 16 // {BF16: 2, F32: 4, S8: 1}[in_t]
    kk = -(-k // mult) * mult  # K-contiguous rows must be 16-byte sized for the tensor-core path
    dist = "full" if in_t == S8 else "int"
    r = run(Case(in_t, out_t, m, n, kk, b_col=True, dist=dist, alpha=1, beta=1, pad_d=(8 if n % 8 else 0)))
    assert r["config"] != gz.CFG_SIMT


@pytest.mark.parametrize("in_t,out_t", [(BF16, BF16), (F16, F32), (F32, F32), (S8, S32)])
@pytest.mark.parametrize("a_col,b_col", [(False, False), (True, True)])
def test_misaligned_operands_use_simt_kernel(in_t, out_t, a_col, b_col):
    dist = "full" if in_t == S8 else "int"
    r = run(Case(in_t, out_t, 33, 77, 45, a_col=a_col, b_col=b_col, dist=dist, alpha=2, beta=-1, pad_a=1, pad_b=3,
                 pad_c=1, pad_d=5))
    assert r["config"] == gz.CFG_SIMT


def test_leading_dimensions_larger_than_extents():
    run(Case(BF16, BF16, 200, 264, 192, b_col=True, pad_a=64, pad_b=8, pad_c=24, pad_d=40, alpha=1, beta=1))
    run(Case(F32, F32, 200, 264, 192, pad_a=4, pad_b=12, pad_c=4, pad_d=8, alpha=1, beta=1))
    # D rows not 16-byte sized: the direct-store epilogue takes over
    r = run(Case(BF16, BF16, 200, 261, 192, b_col=True, pad_d=2, alpha=1, beta=1))
    assert r["epilogue_tma"] == 0


def test_in_place_update():
    run(Case(BF16, BF16, 384, 768, 320, b_col=True, alpha=2, beta=-1, inplace=True, flags=TMA))
    run(Case(S8, S32, 300, 520, 256, b_col=True, dist="full", alpha=1, beta=1, inplace=True, flags=DIRECT))


@pytest.mark.parametrize("in_t,out_t,dist", [(BF16, BF16, "normal"), (F16, F16, "uniform"), (BF16, F32, "normal"),
                                             (F32, F32, "uniform")])
def test_random_inputs_within_tolerance(in_t, out_t, dist):
    r = run(Case(in_t, out_t, 1000, 1032, 2048, b_col=True, dist=dist, alpha=1.0, beta=0.5, scale_b=2048 ** -0.5))
    assert r["mismatches"] == 0


def test_many_tiles_persistent_loop():
    # more tiles than CTAs: every CTA walks several tiles and both accumulators
    for config in (gz.CFG_1CTA_N64, gz.CFG_2CTA_N128):
        run(Case(BF16, BF16, 2048, 4096, 256, b_col=True, config=config))
    run(Case(S8, S32, 4096, 4096, 256, b_col=True, dist="full", config=gz.CFG_2CTA_N256))
