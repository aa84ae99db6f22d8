"""Epilogue terms beyond alpha/beta (gz_gemm_run_ex): bias, per-row and per-column scales,
activations, and the dequantising s8 GEMM with floating-point output.

    D = act(alpha * row_scale[i] * col_scale[j] * acc + beta * C + bias[j])

Checked against the CPU oracle (product in fp64 / exact int32, then the same formula in double).
Integer operands with power-of-two scales and ReLU must be bit-exact after the one rounding to the
output type; the transcendental activations are held to fp32 accuracy."""
import numpy as np
import pytest
import torch

import gemm_zoo_b200 as gz
from gemm_zoo_b200 import api
from oracle import cpu_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TORCH = {gz.DT_F16: torch.float16, gz.DT_BF16: torch.bfloat16, gz.DT_F32: torch.float32, gz.DT_S8: torch.int8,
         gz.DT_S32: torch.int32, gz.DT_E4M3: torch.float8_e4m3fn}


def _operands(in_t, out_t, m, n, k, seed, wide=False):
    rng = np.random.default_rng(seed)
    lo, hi = ((-128, 128) if wide else (-3, 4))
    a = torch.from_numpy(rng.integers(lo, hi, (m, k)).astype(np.float32)).to(TORCH[in_t])
    b = torch.from_numpy(rng.integers(lo, hi, (n, k)).astype(np.float32)).to(TORCH[in_t])   # column-major K x N
    c = torch.from_numpy(rng.integers(-8, 9, (m, n)).astype(np.float32)).to(TORCH[out_t])
    bias = torch.from_numpy(rng.integers(-16, 17, n).astype(np.float32))
    rs = torch.from_numpy(2.0 ** rng.integers(-3, 2, m).astype(np.float32))
    cs = torch.from_numpy(2.0 ** rng.integers(-2, 3, n).astype(np.float32))
    return a, b, c, bias, rs, cs


def _oracle(in_t, out_t, a, b, c, m, n, k, alpha, beta, bias, rs, cs, act):
    if in_t == gz.DT_S8:
        acc = orc.gemm_s8(a.numpy(), b.numpy(), None, m, n, k, b_col_major=True)
    else:
        acc = orc.gemm_f64(in_t, out_t, orc.bits_of(a), orc.bits_of(b), None, m, n, k, b_col_major=True)
    c64 = c.double().numpy() if beta else None
    return orc.epilogue_f64(acc, c64, alpha, beta, None if bias is None else bias.numpy(),
                            None if rs is None else rs.numpy(), None if cs is None else cs.numpy(), act)


def _run(in_t, out_t, m, n, k, alpha, beta, use, act, config=gz.CFG_AUTO, flags=0, seed=0, wide=False):
    a, b, c, bias, rs, cs = _operands(in_t, out_t, m, n, k, seed, wide)
    bias = bias if "bias" in use else None
    rs = rs if "rs" in use else None
    cs = cs if "cs" in use else None
    g = gz.Sm100Gemm(m, n, k, in_t, out_t, layout_b=gz.COL_MAJOR, config=config, flags=flags)
    dev = lambda t: None if t is None else t.to(DEV)
    d = torch.full((m, n), 7, dtype=TORCH[out_t], device=DEV)
    g.plan.run_ex(a.to(DEV), b.to(DEV), dev(c) if beta else None, d, alpha, beta, dev(bias), dev(rs), dev(cs), act)
    torch.cuda.synchronize()
    assert g.plan.device_status()[0] == api.GZ_OK
    want = _oracle(in_t, out_t, a, b, c, m, n, k, alpha, beta, bias, rs, cs, act)
    return d.cpu(), want, g.info().config


@pytest.mark.parametrize("config,m", [(gz.CFG_AUTO, 300), (gz.CFG_1CTA_N128, 300), (gz.CFG_1CTA_N64, 130),
                                      (gz.CFG_2CTA_N256, 300), (gz.CFG_2CTA_M512_N256, 700),
                                      (gz.CFG_SWAP_M64, 64), (gz.CFG_SIMT, 70)])
@pytest.mark.parametrize("in_t,out_t", [(gz.DT_BF16, gz.DT_BF16), (gz.DT_F16, gz.DT_F32), (gz.DT_S8, gz.DT_BF16),
                                        (gz.DT_S8, gz.DT_F32)])
def test_bias_scales_relu_exact(config, m, in_t, out_t):
    got, want, _ = _run(in_t, out_t, m, 520, 256, 2, -1, {"bias", "rs", "cs"}, gz.ACT_RELU, config=config)
    assert torch.equal(got, orc.round_to(out_t, want))


@pytest.mark.parametrize("use", [{"bias"}, {"rs"}, {"cs"}, set()])
def test_each_term_alone(use):
    got, want, _ = _run(gz.DT_BF16, gz.DT_F32, 200, 264, 192, 1, 1, use, gz.ACT_RELU if not use else gz.ACT_NONE)
    assert torch.equal(got, orc.round_to(gz.DT_F32, want))


@pytest.mark.parametrize("act", [gz.ACT_GELU, gz.ACT_GELU_TANH, gz.ACT_SILU])
@pytest.mark.parametrize("in_t,out_t", [(gz.DT_BF16, gz.DT_F32), (gz.DT_S8, gz.DT_F16)])
def test_transcendental_activations(act, in_t, out_t):
    got, want, _ = _run(in_t, out_t, 256, 384, 128, 0.125, 0.5, {"bias", "cs"}, act)
    want_t = torch.from_numpy(want)
    tol = 1e-5 if out_t == gz.DT_F32 else 2.0 ** -10
    assert ((got.double() - want_t).abs() <= tol * want_t.abs() + 1e-5).all()


def test_dequantising_gemm_full_range_s8():
    """Every s8 value, K large enough that the int32 sums exceed 2^24: the accumulator is converted
    from int32 exactly once."""
    got, want, _ = _run(gz.DT_S8, gz.DT_F32, 256, 512, 4096, 1, 0, {"rs", "cs"}, gz.ACT_NONE, wide=True)
    want_t = torch.from_numpy(want)
    assert ((got.double() - want_t).abs() <= 2.0 ** -23 * want_t.abs()).all()


def test_split_k_skinny_with_terms():
    got, want, cfg = _run(gz.DT_S8, gz.DT_BF16, 16, 1024, 8192, 1, 0, {"bias", "rs", "cs"}, gz.ACT_RELU,
                          flags=gz.FLAG_SPLIT_K)
    assert torch.equal(got, orc.round_to(gz.DT_BF16, want))


def test_integer_output_refuses_the_terms():
    g = gz.Sm100Gemm(128, 128, 128, gz.DT_S8, gz.DT_S32, layout_b=gz.COL_MAJOR)
    a = torch.zeros(128, 128, dtype=torch.int8, device=DEV)
    d = torch.zeros(128, 128, dtype=torch.int32, device=DEV)
    bias = torch.zeros(128, device=DEV)
    with pytest.raises(gz.GzError) as e:
        g.plan.run_ex(a, a, None, d, 1, 0, bias=bias)
    assert e.value.status == api.GZ_ERR_UNSUPPORTED
    g.plan.run_ex(a, a, None, d, 1, 0)   # no terms: same as gz_gemm_run
