"""Stream order between consecutive launches.

Every GEMM launch allows programmatic dependent launch: it may start while the kernel before it in
the stream still runs, sets itself up, and each of its roles waits for that kernel inside the
kernel, as late as it can (the producers just before their first load, the epilogue before its first
store).  What a caller relies on is plain stream order, so these tests chain launches that depend
on one another in every direction and compare, bit for bit, with the same chain run with a device
synchronisation after every launch:
  read-after-write   the output of one GEMM is the A (or B) operand of the next;
  write-after-read   a GEMM overwrites a buffer the GEMM before it reads as an operand;
  write-after-write  two GEMMs write the same output, the second must win;
and the same chains replayed from a CUDA graph, for the tile families that differ in who loads and
who stores (one CTA, CTA pair, two row blocks, swapped skinny tiles with and without split-K).
"""
import pytest
import torch

import gemm_zoo_b200 as gz

DEV = "cuda:0"

# (m, n == k, config, why)
CHAINS = [
    (256, 512, gz.CFG_AUTO, "one small tile family, many idle SMs: the next launch starts at once"),
    (1024, 1024, gz.CFG_1CTA_N64, "128 CTAs of one tile each"),
    (1024, 1024, gz.CFG_2CTA_N128, "CTA pairs"),
    (2048, 2048, gz.CFG_2CTA_M512_N256, "two row blocks per CTA"),
    (16, 2048, gz.CFG_AUTO, "swapped skinny tiles, split-K"),
    (128, 4096, gz.CFG_AUTO, "swapped skinny tiles, whole tiles"),
]


def _weights(n, seed):
    w = torch.empty(n, n, dtype=torch.bfloat16, device=DEV)
    gz.fill(w, seed, 2, 1, n ** -0.5)  # N(0, 1/n): activations keep their scale along the chain
    return w


def _chain(g, x0, w, steps, sync):
    """x_{i+1} = x_i . w^T, ping-pong between two buffers: every launch reads what the one before
    wrote and overwrites what the one before read."""
    bufs = [x0.clone(), torch.zeros_like(x0)]
    for i in range(steps):
        g(bufs[i & 1], w, None, bufs[(i + 1) & 1], 1.0, 0.0)
        if sync:
            torch.cuda.synchronize()
    torch.cuda.synchronize()
    return bufs[steps & 1]


@pytest.mark.gpu
@pytest.mark.parametrize("m,n,config,why", CHAINS)
def test_chain_of_dependent_gemms(m, n, config, why):
    g = gz.Sm100Gemm(m, n, n, gz.DT_BF16, gz.DT_BF16, layout_b=gz.COL_MAJOR, config=config)
    x0 = torch.empty(m, n, dtype=torch.bfloat16, device=DEV)
    gz.fill(x0, 11, 1, 1, 1.0)
    w = _weights(n, 13)
    steps = 9
    want = _chain(g, x0, w, steps, sync=True)
    assert float(want.float().abs().max()) > 0.0
    for _ in range(3):
        got = _chain(g, x0, w, steps, sync=False)
        assert torch.equal(got.view(torch.int16), want.view(torch.int16)), why
    assert g.plan.device_status()[0] == 0


@pytest.mark.gpu
@pytest.mark.parametrize("m,n,config,why", CHAINS)
def test_chain_replayed_from_a_graph(m, n, config, why):
    g = gz.Sm100Gemm(m, n, n, gz.DT_BF16, gz.DT_BF16, layout_b=gz.COL_MAJOR, config=config)
    x0 = torch.empty(m, n, dtype=torch.bfloat16, device=DEV)
    gz.fill(x0, 17, 1, 1, 1.0)
    w = _weights(n, 19)
    steps = 8  # even: the result lands in the buffer the chain started from
    want = _chain(g, x0, w, steps, sync=True)
    bufs = [x0.clone(), torch.zeros_like(x0)]
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        g(bufs[0], w, None, bufs[1], 1.0, 0.0, stream=stream)  # warm-up outside the capture
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for i in range(steps):
                g(bufs[i & 1], w, None, bufs[(i + 1) & 1], 1.0, 0.0, stream=stream)
    for _ in range(3):
        bufs[0].copy_(x0)
        bufs[1].zero_()
        torch.cuda.synchronize()
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(bufs[0].view(torch.int16), want.view(torch.int16)), why
    assert g.plan.device_status()[0] == 0


@pytest.mark.gpu
def test_later_launch_wins_the_output_and_an_operand_written_in_between_is_seen():
    m, n, k = 512, 768, 1024
    g = gz.Sm100Gemm(m, n, k, gz.DT_BF16, gz.DT_BF16, layout_b=gz.COL_MAJOR)
    a1, a2 = (torch.empty(m, k, dtype=torch.bfloat16, device=DEV) for _ in range(2))
    b = torch.empty(n, k, dtype=torch.bfloat16, device=DEV)
    gz.fill(a1, 23, 1, 1, 1.0)
    gz.fill(a2, 23, 3, 1, 1.0)
    gz.fill(b, 23, 2, 1, k ** -0.5)
    want = torch.empty(m, n, dtype=torch.bfloat16, device=DEV)
    g(a2, b, None, want, 1.0, 0.0)
    torch.cuda.synchronize()
    for _ in range(5):
        d = torch.zeros(m, n, dtype=torch.bfloat16, device=DEV)
        a = a1.clone()
        torch.cuda.synchronize()
        g(a, b, None, d, 1.0, 0.0)   # first result, to be overwritten
        a.copy_(a2)                  # another kernel rewrites the operand in between
        g(a, b, None, d, 1.0, 0.0)   # must read the new operand and win the output
        torch.cuda.synchronize()
        assert torch.equal(d.view(torch.int16), want.view(torch.int16))


@pytest.mark.gpu
def test_accumulating_into_the_output_of_the_launch_before():
    """beta != 0 with C == D: launch i + 1 reads as C what launch i stored as D."""
    m, n, k = 1024, 1024, 512
    g = gz.Sm100Gemm(m, n, k, gz.DT_BF16, gz.DT_F32, layout_b=gz.COL_MAJOR)
    a = torch.empty(m, k, dtype=torch.bfloat16, device=DEV)
    b = torch.empty(n, k, dtype=torch.bfloat16, device=DEV)
    gz.fill(a, 29, 1, 2, 4.0)  # integers in [-4, 4]: every partial sum is exact in fp32
    gz.fill(b, 29, 2, 2, 4.0)
    once = torch.zeros(m, n, dtype=torch.float32, device=DEV)
    g(a, b, None, once, 1.0, 0.0)
    torch.cuda.synchronize()
    d = torch.zeros(m, n, dtype=torch.float32, device=DEV)
    steps = 7
    for _ in range(steps):
        g(a, b, d, d, 1.0, 1.0)
    torch.cuda.synchronize()
    assert torch.equal(d, once * steps)


@pytest.mark.gpu
def test_time_spent_waiting_for_the_previous_kernel_does_not_count_against_the_wait_limit():
    """A launch whose CTAs are resident early (idle SMs, the kernel before it has signalled that
    dependents may start) sits out the rest of that kernel inside `griddepcontrol.wait`; its bounded
    waits start only afterwards, so a small wait limit does not turn a long predecessor into a
    timeout."""
    k_long = 1 << 22
    slow = gz.Sm100Gemm(128, 128, k_long, gz.DT_BF16, gz.DT_BF16, layout_b=gz.COL_MAJOR, config=gz.CFG_1CTA_N128)
    assert slow.info().grid == 1  # one CTA walks 65536 K blocks: about 15 ms, 147 SMs idle
    a = torch.zeros(128, k_long, dtype=torch.bfloat16, device=DEV)
    b = torch.zeros(128, k_long, dtype=torch.bfloat16, device=DEV)
    d_slow = torch.empty(128, 128, dtype=torch.bfloat16, device=DEV)
    m, n, k = 1024, 1024, 256
    quick = gz.Sm100Gemm(m, n, k, gz.DT_BF16, gz.DT_BF16, layout_b=gz.COL_MAJOR, wait_limit_ns=1_000_000)
    x = torch.empty(m, k, dtype=torch.bfloat16, device=DEV)
    w = torch.empty(n, k, dtype=torch.bfloat16, device=DEV)
    gz.fill(x, 31, 1, 1, 1.0)
    gz.fill(w, 31, 2, 1, k ** -0.5)
    want = torch.empty(m, n, dtype=torch.bfloat16, device=DEV)
    quick(x, w, None, want, 1.0, 0.0)
    slow(a, b, None, d_slow, 1.0, 0.0)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    got = torch.zeros(m, n, dtype=torch.bfloat16, device=DEV)
    e0.record()
    slow(a, b, None, d_slow, 1.0, 0.0)
    quick(x, w, None, got, 1.0, 0.0)  # directly behind: an event record in between would end the overlap
    e1.record()
    torch.cuda.synchronize()
    if e0.elapsed_time(e1) < 2.0:
        pytest.skip("the long kernel finished within twice the wait limit: nothing to show")
    st, detail = quick.plan.device_status()
    assert st == 0, (st, detail)
    assert torch.equal(got.view(torch.int16), want.view(torch.int16))
