"""Batched (strided) GEMM: `batch` problems of one shape in a single launch.

Every problem of the batch must equal the same problem run alone through the oracle; integer
operands make that a bit-exact comparison.  Covers packed and padded batch strides, a shared
(broadcast) operand, every tile family (1-CTA, 2-CTA, 512x256, swapped skinny tiles with split-K,
the CUDA-core kernel), beta with a batched C, and the epilogue terms."""
import numpy as np
import pytest
import torch

import gemm_zoo_b200 as gz
from gemm_zoo_b200 import api
from oracle import cpu_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TORCH = {gz.DT_F16: torch.float16, gz.DT_BF16: torch.bfloat16, gz.DT_F32: torch.float32, gz.DT_S8: torch.int8,
         gz.DT_S32: torch.int32}


def _ints(shape, dtype, seed, lo=-3, hi=4):
    rng = np.random.default_rng(seed)
    return torch.from_numpy(rng.integers(lo, hi, shape).astype(np.float32)).to(TORCH[dtype])


def _one(in_t, out_t, a, b, c, m, n, k, alpha, beta, b_col):
    if in_t == gz.DT_S8:
        r = orc.gemm_s8(a.numpy(), b.numpy(), None if c is None else c.numpy(), m, n, k, alpha, beta,
                        b_col_major=b_col)
        return torch.from_numpy(r)
    r = orc.gemm_f64(in_t, out_t, orc.bits_of(a), orc.bits_of(b), None if c is None else orc.bits_of(c), m, n, k,
                     alpha, beta, b_col_major=b_col)
    return orc.round_to(out_t, r)


@pytest.mark.parametrize("in_t,out_t,m,n,k,batch,config,b_col,beta,pad", [
    (gz.DT_BF16, gz.DT_BF16, 300, 520, 256, 5, gz.CFG_AUTO, True, 0, 0),
    (gz.DT_BF16, gz.DT_BF16, 256, 512, 128, 7, gz.CFG_1CTA_N128, True, -1, 64),     # padded batch strides, batched C
    (gz.DT_F16, gz.DT_F32, 384, 768, 192, 3, gz.CFG_2CTA_N256, False, 1, 0),        # row-major B
    (gz.DT_BF16, gz.DT_BF16, 1024, 512, 256, 40, gz.CFG_2CTA_M512_N256, True, 0, 0),  # 160 tiles: tail strips cross problems
    (gz.DT_F32, gz.DT_F32, 200, 264, 96, 4, gz.CFG_1CTA_N64, False, 0, 32),         # tf32, both row-major
    (gz.DT_S8, gz.DT_S32, 130, 256, 512, 6, gz.CFG_2CTA_N128, True, 2, 0),
    (gz.DT_BF16, gz.DT_BF16, 16, 256, 2048, 3, gz.CFG_SWAP_M16, True, 0, 0),        # skinny tiles, split-K across the batch
    (gz.DT_BF16, gz.DT_F32, 64, 384, 1024, 9, gz.CFG_SWAP_M64, True, 1, 128),
    (gz.DT_BF16, gz.DT_BF16, 33, 77, 45, 5, gz.CFG_AUTO, True, 1, 0),               # rows TMA cannot describe: CUDA-core kernel
])
def test_every_problem_of_the_batch(in_t, out_t, m, n, k, batch, config, b_col, beta, pad):
    lo, hi = (-128, 128) if in_t == gz.DT_S8 else (-3, 4)
    b_shape = (n, k) if b_col else (k, n)
    sa, sb, sc = m * k + pad, b_shape[0] * b_shape[1] + pad, m * n + pad
    a = _ints((batch, sa), in_t, 1, lo, hi)
    b = _ints((batch, sb), in_t, 2, lo, hi)
    c = _ints((batch, sc), out_t, 3, -4, 5)
    d = torch.full((batch, sc), 55, dtype=TORCH[out_t], device=DEV)
    flags = gz.FLAG_SPLIT_K if config in (gz.CFG_SWAP_M16, gz.CFG_SWAP_M64) else 0
    g = gz.Sm100Gemm(m, n, k, in_t, out_t, layout_b=gz.COL_MAJOR if b_col else gz.ROW_MAJOR, config=config,
                     flags=flags, batch=batch, stride_a=sa, stride_b=sb, stride_c=sc, stride_d=sc)
    info = g.info()
    if m == 33:
        assert info.config == gz.CFG_SIMT
    g(a.to(DEV), b.to(DEV), c.to(DEV) if beta else None, d, 2, beta)
    torch.cuda.synchronize()
    assert g.plan.device_status()[0] == api.GZ_OK
    got = d.cpu()
    for i in range(batch):
        ai = a[i, :m * k].reshape(m, k)
        bi = b[i, :b_shape[0] * b_shape[1]].reshape(b_shape)
        ci = c[i, :m * n].reshape(m, n) if beta else None
        want = _one(in_t, out_t, ai, bi, ci, m, n, k, 2, beta, b_col)
        assert torch.equal(got[i, :m * n].reshape(m, n), want), (i, info.config)
        if pad:
            assert (got[i, m * n:] == 55).all()   # nothing written between the problems


def test_shared_operand_and_epilogue_terms():
    """One B for the whole batch (weights), a different A per problem, bias and ReLU in the epilogue."""
    m, n, k, batch = 128, 384, 256, 6
    a = _ints((batch, m * k), gz.DT_BF16, 1)
    b = _ints((n, k), gz.DT_BF16, 2)
    bias = torch.from_numpy(np.random.default_rng(3).integers(-9, 10, n).astype(np.float32))
    d = torch.zeros(batch, m * n, dtype=torch.bfloat16, device=DEV)
    g = gz.Sm100Gemm(m, n, k, gz.DT_BF16, gz.DT_BF16, layout_b=gz.COL_MAJOR, batch=batch, flags=gz.FLAG_BROADCAST_B)
    g.plan.run_ex(a.to(DEV), b.to(DEV), None, d, 1, 0, bias=bias.to(DEV), activation=gz.ACT_RELU)
    torch.cuda.synchronize()
    for i in range(batch):
        acc = orc.gemm_f64(gz.DT_BF16, gz.DT_BF16, orc.bits_of(a[i].reshape(m, k)), orc.bits_of(b), None, m, n, k,
                           b_col_major=True)
        want = orc.round_to(gz.DT_BF16, orc.epilogue_f64(acc, None, 1, 0, bias.numpy(), None, None, orc.ACT_RELU))
        assert torch.equal(d[i].cpu().reshape(m, n), want), i


def test_batch_is_one_launch_and_argument_errors():
    st, info = gz.validate(gz.GemmDesc.make(gz.DT_BF16, gz.DT_BF16, 256, 256, 256, layout_b=gz.COL_MAJOR, batch=100), 148)
    assert st == api.GZ_OK and info.tiles % 100 == 0 and info.tiles >= 100 and info.grid <= 148
    st, _ = gz.validate(gz.GemmDesc.make(gz.DT_BF16, gz.DT_BF16, 256, 256, 256, batch=-1), 148)
    assert st == api.GZ_ERR_INVALID_ARG
    # a batch stride TMA cannot describe falls back to the CUDA-core kernel
    st, info = gz.validate(gz.GemmDesc.make(gz.DT_BF16, gz.DT_BF16, 256, 256, 256, batch=3, stride_a=256 * 256 + 3), 148)
    assert st == api.GZ_OK and info.config == gz.CFG_SIMT
    # host-operand runs move one problem
    g = gz.Sm100Gemm(128, 128, 128, gz.DT_BF16, gz.DT_BF16, batch=2)
    x = torch.zeros(2, 128 * 128, dtype=torch.bfloat16)
    with pytest.raises(gz.GzError) as e:
        g.plan.run_host(x, x, None, x.clone(), 1, 0)
    assert e.value.status == api.GZ_ERR_UNSUPPORTED
