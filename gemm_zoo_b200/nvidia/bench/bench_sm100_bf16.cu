// Benchmark of this library's sm_100a kernel: bf16 in, fp32 accumulate, bf16 out; sizes of nvidia/bench/bench_bf16_mma_gemm.cu:21-27.
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
  const TOut beta = __float2bfloat16(1.0f);
  using kernel_functor_struct = nvidia::kernel_functors::sm100_gemm<TIn, TOut, nvidia::kernel_functors::RowMajor, nvidia::kernel_functors::RowMajor>;
  benchmark::benchmark<kernel_functor_struct, TIn, TOut>({{256, 256, 256}, {512, 512, 512}, {1024, 1024, 1024}, {2048, 2048, 2048}, {4096, 4096, 4096}, {8192, 8192, 8192}}, alpha, beta);
}
