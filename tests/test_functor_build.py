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


DEQUANT_MAIN = r'''
// sm100_gemm<int8_t, float>: s8 operands, int32 accumulation, float scalars and output.
#include "kernel_functors/sm100_gemm.cuh"
#include <cstdio>
#include <cstdint>
#include <vector>
int main() {
  const int m = 96, n = 200, k = 320;
  std::vector<int8_t> a(m * k), b(k * n);
  for (int i = 0; i < m * k; ++i) a[i] = (int8_t)((i * 37 + 11) % 255 - 127);
  for (int i = 0; i < k * n; ++i) b[i] = (int8_t)((i * 53 + 7) % 251 - 125);
  std::vector<float> c(m * n), d(m * n, -1.0f);
  for (int i = 0; i < m * n; ++i) c[i] = (float)((i % 17) - 8);
  int8_t *da, *db; float *dc, *dd;
  cudaMalloc(&da, a.size()); cudaMalloc(&db, b.size()); cudaMalloc(&dc, c.size() * 4); cudaMalloc(&dd, d.size() * 4);
  cudaMemcpy(da, a.data(), a.size(), cudaMemcpyHostToDevice);
  cudaMemcpy(db, b.data(), b.size(), cudaMemcpyHostToDevice);
  cudaMemcpy(dc, c.data(), c.size() * 4, cudaMemcpyHostToDevice);
  cudaDeviceProp prop; cudaGetDeviceProperties(&prop, 0);
  nvidia::kernel_functors::sm100_gemm<int8_t, float> gemm(m, n, k, prop);  // reference convention: all row-major
  const float alpha = 0.25f, beta = -2.0f;
  gemm(da, db, dc, dd, alpha, beta, nullptr);
  if (cudaDeviceSynchronize() != cudaSuccess || gemm.device_status(nullptr) != GZ_OK) { printf("FAILED launch\n"); return 1; }
  cudaMemcpy(d.data(), dd, d.size() * 4, cudaMemcpyDeviceToHost);
  long bad = 0;
  for (int i = 0; i < m; ++i)
    for (int j = 0; j < n; ++j) {
      int acc = 0;
      for (int l = 0; l < k; ++l) acc += (int)a[i * k + l] * (int)b[l * n + j];
      const float want = alpha * (float)acc + beta * c[i * n + j];  // exact in fp32 for these magnitudes
      if (d[i * n + j] != want) { if (bad < 5) printf("bad %d %d got %g want %g\n", i, j, d[i * n + j], want); ++bad; }
    }
  printf(bad ? "FAILED %ld\n" : "DEQUANT OK %ld\n", bad);
  return bad ? 1 : 0;
}
'''


def _compile(tmp_path, name, text):
    src = tmp_path / f"{name}.cu"
    src.write_text(text)
    b.build_lib()
    out = tmp_path / name
    cmd = [b.nvcc_path(), *b.ARCH, *b.NVCC_COMMON, f"-I{b.INCLUDE}", f"-I{b.PKG / 'nvidia'}", "-o", str(out), str(src),
           f"-L{b.PKG}", "-lgemmzoo", f"-Xlinker=-rpath={b.PKG}"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-2000:]
    return out


def test_dequantising_functor_compiles(tmp_path):
    assert _compile(tmp_path, "dequant", DEQUANT_MAIN).exists()


@pytest.mark.gpu
def test_dequantising_functor_passes_float_scalars(tmp_path):
    """sm100_gemm<int8_t, float>: alpha and beta must reach the C ABI as floats (the C ABI reads
    int32 scalars only for s32 outputs); checked against an exact host loop."""
    exe = _compile(tmp_path, "dequant", DEQUANT_MAIN)
    r = subprocess.run([str(exe)], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "DEQUANT OK" in r.stdout, (r.stdout[-1500:], r.stderr[-1500:])
