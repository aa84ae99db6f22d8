"""The C++ side of the drop-in boundary: a bench main written against the reference's
harness entry point compiles with the sm100_gemm functor (CPU check), and runs and
verifies itself against cuBLASLt on a GPU."""
import subprocess
from pathlib import Path

import pytest

from gemm_zoo_b200 import build as b

BENCH = b.PKG / "nvidia" / "bench"


def test_bench_mains_compile_against_the_functor(tmp_path):
    src = tmp_path / "drop_in.cu"
    # The reference's own call pattern (nvidia/bench/bench_tf32_mma_gemm.cu:9-28) with the functor swapped.
    src.write_text('''
#include "kernel_functors/sm100_gemm.cuh"
#include "utils/benchmark.cuh"
#include <tuple>
int main() {
  float alpha = 1.0f;
  float beta = 1.0f;
  using kernel_functor_struct = nvidia::kernel_functors::sm100_gemm<float, float>;
  benchmark::benchmark<kernel_functor_struct, float, float>({{128, 128, 128}, {256, 256, 256}}, alpha, beta);
}
''')
    lib = b.build_lib()
    out = tmp_path / "drop_in"
    cmd = [b.nvcc_path(), *b.ARCH, *b.NVCC_COMMON, f"-I{b.INCLUDE}", f"-I{b.PKG / 'nvidia'}", "-o", str(out), str(src),
           f"-L{b.PKG}", "-lgemmzoo", f"-Xlinker=-rpath={b.PKG}", "-lcublasLt"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-2000:]
    assert out.exists() and lib.exists()
    assert len(list(BENCH.glob("bench_sm100_*.cu"))) >= 5


@pytest.mark.gpu
def test_bench_main_runs_and_verifies():
    exe = BENCH / "build" / "bench_sm100_tf32"
    if not exe.exists():
        b.build_bench()
    r = subprocess.run([str(exe)], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, (r.stdout[-1500:], r.stderr[-1500:])
    lines = [l for l in r.stdout.splitlines() if l.startswith("GEMM Problem:")]
    assert len(lines) == 7 and "verification failed" not in r.stdout
