// Benchmark of cuBLASLt (the comparator): bf16, A row-major / B column-major, beta = 0: the headline layout and the inference-shaped sweep.
// Same shape as the reference's bench mains: pick the functor, call the harness.
#include <cuda_runtime.h>
#include <cuda_bf16.h>

#include <tuple>

#include "kernel_functors/cublaslt_gemm.cuh"
#include "kernel_functors/sm100_gemm.cuh"
#include "utils/benchmark.cuh"

int main() {
  using TIn = __nv_bfloat16;
  using TOut = __nv_bfloat16;
  const TOut alpha = __float2bfloat16(1.0f);
  const TOut beta = __float2bfloat16(0.0f);
  using kernel_functor_struct = nvidia::kernel_functors::cublasLt_gemm<TIn, TOut, nvidia::kernel_functors::RowMajor, nvidia::kernel_functors::ColMajor>;
  benchmark::benchmark<kernel_functor_struct, TIn, TOut>({{4096, 4096, 4096}, {8192, 8192, 8192}, {16, 14336, 4096}, {128, 14336, 4096}, {2048, 14336, 4096}, {16384, 14336, 4096}}, alpha, beta);
}
