"""GPU parity tests: the CUDA path, called through the C ABI, against the CPU
oracle on the same seeded operands.  Integer work and exact-integer float inputs
are compared bit for bit; random float inputs within the bars in tests/helpers.py.
Every output buffer is wrapped in sentinel guard bands that must stay untouched."""
import pytest

import gemm_zoo_b200 as gz
from tests.helpers import Case, check

pytestmark = pytest.mark.gpu

F16, BF16, F32, S8, S32 = gz.DT_F16, gz.DT_BF16, gz.DT_F32, gz.DT_S8, gz.DT_S32
E4M3, E5M2 = gz.DT_E4M3, gz.DT_E5M2
DIRECT, TMA = gz.FLAG_EPILOGUE_DIRECT, gz.FLAG_EPILOGUE_TMA
TC_CONFIGS = [gz.CFG_1CTA_N256, gz.CFG_1CTA_N128, gz.CFG_1CTA_N64, gz.CFG_2CTA_N256, gz.CFG_2CTA_N128,
              gz.CFG_2CTA_M512_N256]


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
@pytest.mark.parametrize("config", [gz.CFG_1CTA_N256, gz.CFG_2CTA_N256, gz.CFG_1CTA_N128, gz.CFG_2CTA_M512_N256])
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


SWAP_CONFIGS = [(gz.CFG_SWAP_M16, 16), (gz.CFG_SWAP_M32, 32), (gz.CFG_SWAP_M64, 64), (gz.CFG_SWAP_M128, 128)]


@pytest.mark.parametrize("config,mmax", SWAP_CONFIGS)
@pytest.mark.parametrize("in_t,out_t", [(BF16, BF16), (F16, F32), (F32, F32), (S8, S32)])
def test_swapped_operand_tiles(config, mmax, in_t, out_t):
    """Skinny problems: B rides the 128-row side of the MMA, A the narrow side."""
    dist = "full" if in_t == S8 else "int"
    for m in sorted({1, mmax // 2 + 1, mmax}):
        run(Case(in_t, out_t, m, 1000 if in_t != S8 else 1008, 512, b_col=True, config=config, dist=dist,
                 alpha=2, beta=-1, pad_d=8))
    # B row-major (N contiguous) on the wide side
    run(Case(in_t, out_t, mmax, 640, 384, b_col=False, config=config, dist=dist, alpha=1, beta=1))


def test_swapped_tiles_are_chosen_for_skinny_problems():
    for m, want in ((1, gz.CFG_SWAP_M16), (16, gz.CFG_SWAP_M16), (17, gz.CFG_SWAP_M32)):
        r = run(Case(BF16, BF16, m, 2048, 1024, b_col=True, dist="normal", beta=0.5, inplace=(m == 16)))
        assert r["config"] == want
    # A column-major with a narrow tile cannot be fetched in 128-byte chunks: falls back to a wide tile
    r = run(Case(BF16, BF16, 16, 2048, 1024, a_col=True, b_col=True))
    assert r["config"] not in (gz.CFG_SWAP_M16, gz.CFG_SWAP_M32, gz.CFG_SIMT)


@pytest.mark.parametrize("in_t,out_t", [(BF16, BF16), (F16, F32), (F32, F32), (S8, S32)])
@pytest.mark.parametrize("m,n,k", [(16, 14336, 4096), (5, 1000, 8192), (1, 136, 16384), (32, 4096, 2048),
                                   (64, 640, 4096), (16, 128, 128 * 148 * 2), (100, 1024, 8192)])
def test_split_k_last_arriver_reduction(in_t, out_t, m, n, k):
    """K ranges shared between CTAs: partial sums parked in the plan's workspace, finished by the
    last CTA to arrive.  Exact-integer inputs make the result independent of how K was cut."""
    dist = "int"
    if in_t == S8:
        dist = "int"  # small values keep |sum| far below 2^31
        n = -(-n // 16) * 16
    config = (gz.CFG_SWAP_M16 if m <= 16 else gz.CFG_SWAP_M32 if m <= 32 else gz.CFG_SWAP_M64 if m <= 64
              else gz.CFG_SWAP_M128)
    r = run(Case(in_t, out_t, m, n, k, b_col=True, dist=dist, alpha=1, beta=1, config=config, flags=gz.FLAG_SPLIT_K))
    assert r["split_k"] == 1


def test_split_k_is_reproducible_and_reusable():
    """Same plan called repeatedly (the arrival counters reset themselves) gives identical bits,
    for random inputs too."""
    import torch
    m, n, k = 16, 4096, 4096   # 32 tiles for 148 SMs: the plan splits K on its own
    a = torch.randn(m, k, device="cuda:0").bfloat16()
    b = (torch.randn(n, k, device="cuda:0") * 0.02).bfloat16()
    g = gz.Sm100Gemm(m, n, k, BF16, BF16, layout_b=gz.COL_MAJOR)
    assert g.info().split_k == 1 and g.info().workspace_bytes > 0 and g.info().grid > 32
    outs = []
    for _ in range(4):
        d = torch.empty(m, n, dtype=torch.bfloat16, device="cuda:0")
        g(a, b, None, d, 1.0, 0.0)
        outs.append(d)
    torch.cuda.synchronize()
    assert g.plan.device_status()[0] == 0
    for d in outs[1:]:
        assert torch.equal(d.view(torch.int16), outs[0].view(torch.int16))
    ref = (a.double() @ b.double().t())
    assert ((outs[0].double() - ref).abs() <= 2.0 ** -8 * ref.abs() + 1e-3).all()
    # and agrees with the unsplit kernel to within fp32 summation-order effects
    d2 = torch.empty(m, n, dtype=torch.float32, device="cuda:0")
    d3 = torch.empty_like(d2)
    gz.Sm100Gemm(m, n, k, BF16, gz.DT_F32, layout_b=gz.COL_MAJOR, flags=gz.FLAG_NO_SPLIT_K)(a, b, None, d2, 1.0, 0.0)
    gz.Sm100Gemm(m, n, k, BF16, gz.DT_F32, layout_b=gz.COL_MAJOR, flags=gz.FLAG_SPLIT_K)(a, b, None, d3, 1.0, 0.0)
    assert ((d2 - d3).abs() <= 1e-4).all()


@pytest.mark.parametrize("config,m,n", [(gz.CFG_2CTA_N256, 1536, 3584),   # 84 tiles on 74 pairs: 10 tail tiles in 4 strips
                                        (gz.CFG_2CTA_N256, 2048, 3328),   # 104 tiles: 30 tail tiles in 2 strips
                                        (gz.CFG_1CTA_N256, 2048, 2560 + 256),  # 176 tiles on 148 CTAs
                                        (gz.CFG_1CTA_N128, 2176, 1280),   # 170 tiles: 22 tail tiles, 2 strips of 64
                                        (gz.CFG_2CTA_N128, 2560, 1024 + 128),
                                        (gz.CFG_2CTA_M512_N256, 3072, 3584),  # 84 tiles of 512x256: 10 tail tiles in 4 strips
                                        (gz.CFG_2CTA_M512_N256, 4096, 3328)])  # 104 tiles: 30 tail tiles in 2 strips
@pytest.mark.parametrize("in_t,out_t,b_col", [(BF16, BF16, True), (BF16, F32, False), (F32, F32, False),
                                              (S8, S32, True)])
def test_tail_wave_is_cut_into_column_strips(config, m, n, in_t, out_t, b_col):
    """Problems whose last wave of tiles would be mostly empty: those tiles are computed as narrower
    column strips.  Results must not change."""
    dist = "full" if in_t == S8 else "int"
    run(Case(in_t, out_t, m, n, 256, b_col=b_col, config=config, dist=dist, alpha=2, beta=1))
    run(Case(in_t, out_t, m - 8, n - 24, 192, b_col=b_col, config=config, dist=dist, alpha=1, beta=0))


ALL_CONFIGS = TC_CONFIGS + [gz.CFG_SWAP_M64]


@pytest.mark.parametrize("in_t", [E4M3, E5M2])
@pytest.mark.parametrize("out_t", [F16, BF16, F32])
@pytest.mark.parametrize("config", ALL_CONFIGS)
def test_fp8_inputs_exact_integers(in_t, out_t, config):
    """8-bit float inputs (kind::f8f6f4): small integers are exact in e4m3 and e5m2."""
    m = 64 if config == gz.CFG_SWAP_M64 else 300
    run(Case(in_t, out_t, m, 528, 512, b_col=True, config=config, dist="int", alpha=2, beta=-1))


@pytest.mark.parametrize("in_t", [E4M3, E5M2])
@pytest.mark.parametrize("a_col,b_col", [(False, False), (True, False), (True, True), (False, True)])
def test_fp8_layouts(in_t, a_col, b_col):
    run(Case(in_t, F32, 384, 512, 384, a_col=a_col, b_col=b_col, dist="int", alpha=1, beta=1))
    run(Case(in_t, BF16, 256, 384, 256, a_col=a_col, b_col=b_col, config=gz.CFG_2CTA_N256, dist="int"))


@pytest.mark.parametrize("in_t", [E4M3, E5M2])
@pytest.mark.parametrize("out_t", [F16, F32])
def test_fp8_every_byte_pattern_within_tolerance(in_t, out_t):
    """Operands drawn from all finite byte patterns of the format (subnormals included)."""
    r = run(Case(in_t, out_t, 512, 640, 1024, b_col=True, dist="full", alpha=2.0 ** -10, beta=0.5))
    assert r["mismatches"] == 0
    r = run(Case(in_t, out_t, 33, 77, 45, dist="full", alpha=2.0 ** -10, beta=0.0, pad_a=1, pad_b=3, pad_d=5))
    assert r["config"] == gz.CFG_SIMT
