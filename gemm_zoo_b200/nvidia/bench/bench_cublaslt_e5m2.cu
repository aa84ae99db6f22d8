// Benchmark of cuBLASLt (the comparator): fp8 e5m2 inputs, fp32 accumulate, fp16 output, A row-major / B column-major;
// the dtype pair and sizes of nvidia/bench/bench_cublaslt_e5m2.cu:6-21.
// Same shape as the reference's bench mains: pick the functor, call the harness.
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include <tuple>

#include "kernel_functors/cublaslt_gemm.cuh"
#include "kernel_functors/sm100_gemm.cuh"
#include "utils/benchmark.cuh"

int main() {
  using TIn = __nv_fp8_e5m2;
  using TOut = __half;
  const TOut alpha = __half(1.0f);
  const TOut beta = __half(1.0f);
  using kernel_functor_struct = nvidia::kernel_functors::cublasLt_gemm<TIn, TOut, nvidia::kernel_functors::RowMajor, nvidia::kernel_functors::ColMajor>;
  benchmark::benchmark<kernel_functor_struct, TIn, TOut>(
      {{128, 128, 128}, {256, 256, 256}, {512, 512, 512}, {1024, 1024, 1024}, {2048, 2048, 2048}, {4096, 4096, 4096}, {8192, 8192, 8192}},
      alpha, beta);
}
