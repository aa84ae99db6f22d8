// Benchmark of this library's sm_100a kernel: fp32 storage, tf32 multiply; sizes of nvidia/bench/bench_tf32_mma_gemm.cu:19-25.
// Same shape as the reference's bench mains: pick the functor, call the harness.
#include <cuda_runtime.h>


#include <tuple>

#include "kernel_functors/cublaslt_gemm.cuh"
#include "kernel_functors/sm100_gemm.cuh"
#include "utils/benchmark.cuh"

int main() {
  using TIn = float;
  using TOut = float;
  const TOut alpha = 1.0f;
  const TOut beta = 1.0f;
  using kernel_functor_struct = nvidia::kernel_functors::sm100_gemm<TIn, TOut, nvidia::kernel_functors::RowMajor, nvidia::kernel_functors::RowMajor>;
  benchmark::benchmark<kernel_functor_struct, TIn, TOut>({{128, 128, 128}, {256, 256, 256}, {512, 512, 512}, {1024, 1024, 1024}, {2048, 2048, 2048}, {4096, 4096, 4096}, {8192, 8192, 8192}}, alpha, beta);
}
