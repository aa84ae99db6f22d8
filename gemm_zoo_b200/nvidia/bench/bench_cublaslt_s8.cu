// Benchmark of cuBLASLt (the comparator): s8 x s8 -> s32, the contract of bench/bench_xe_gemm_s8_s8_s32_m8k16.cpp:10-18; B column-major.
// Same shape as the reference's bench mains: pick the functor, call the harness.
#include <cuda_runtime.h>
#include <cstdint>

#include <tuple>

#include "kernel_functors/cublaslt_gemm.cuh"
#include "kernel_functors/sm100_gemm.cuh"
#include "utils/benchmark.cuh"

int main() {
  using TIn = std::int8_t;
  using TOut = std::int32_t;
  const TOut alpha = 1;
  const TOut beta = 1;
  using kernel_functor_struct = nvidia::kernel_functors::cublasLt_gemm<TIn, TOut, nvidia::kernel_functors::RowMajor, nvidia::kernel_functors::ColMajor>;
  benchmark::benchmark<kernel_functor_struct, TIn, TOut>({{1024, 1024, 1024}, {2048, 2048, 2048}, {4096, 4096, 4096}, {8192, 8192, 8192}}, alpha, beta);
}
