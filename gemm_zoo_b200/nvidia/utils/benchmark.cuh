// Benchmark harness with the entry point of the reference
// (nvidia/utils/benchmark.cuh:111-126):
//
//   benchmark::benchmark<Kernel, TIn, TOut>({{m, n, k}, ...}, alpha, beta, repetitions = 50);
//
// For every problem: operands are rotated through enough buffer sets that no
// repetition finds its inputs in L2 (as nvidia/utils/benchmark.cuh:27-34 does),
// the kernel's result is verified once, then each repetition is timed with a
// pair of CUDA events on the stream.  Differences from the reference:
//   - A, B and C are filled from different random streams, and the verification
//     kernel is cuBLASLt configured for the true layout (falling back to this
//     library's CUDA-core kernel), so operand-order mistakes are caught;
//   - the report line keeps the reference's format (same FLOP convention
//     m*n*(2k+3), nvidia/utils/benchmark.cuh:91-92) and is followed by a JSON
//     line with median/min times and TFLOP/s by 2*m*n*k;
//   - layouts follow the Kernel: a functor may expose
//     `static constexpr bool b_col_major` / `a_col_major` (default: row-major).
#ifndef GZ_NVIDIA_UTILS_BENCHMARK_CUH
#define GZ_NVIDIA_UTILS_BENCHMARK_CUH

#include <cuda_runtime.h>

#include <algorithm>
#include <cstddef>
#include <cstdio>
#include <stdexcept>
#include <tuple>
#include <type_traits>
#include <vector>

#include "compare.cuh"
#include "defines.hpp"
#include "fill_data.cuh"
#include "kernel_functors/cublaslt_gemm.cuh"
#include "kernel_functors/sm100_gemm.cuh"

namespace benchmark {
namespace detail {

template <class K, class = void>
struct a_is_col : std::false_type {};
template <class K>
struct a_is_col<K, std::void_t<decltype(K::a_col_major)>> : std::bool_constant<K::a_col_major> {};
template <class K, class = void>
struct b_is_col : std::false_type {};
template <class K>
struct b_is_col<K, std::void_t<decltype(K::b_col_major)>> : std::bool_constant<K::b_col_major> {};

template <class Kernel, typename TIn, typename TOut>
void benchmark_impl(std::size_t m, std::size_t n, std::size_t k, TOut alpha, TOut beta,
                    cudaStream_t stream, const int num_repetitions) {
  namespace kf = nvidia::kernel_functors;
  int device_id = 0;
  checkCudaError(cudaGetDevice(&device_id));
  cudaDeviceProp properties;
  checkCudaError(cudaGetDeviceProperties(&properties, device_id));

  const std::size_t problem_bytes = (m * k + k * n) * sizeof(TIn) + m * n * sizeof(TOut);
  const std::size_t sets = static_cast<std::size_t>(properties.l2CacheSize) / problem_bytes + 1;
  const std::size_t reps = std::max<std::size_t>(num_repetitions, sets);

  std::vector<TIn*> a(sets), b(sets);
  std::vector<TOut*> c(sets);
  TOut *d_out = nullptr, *d_ref = nullptr;
  for (std::size_t i = 0; i < sets; ++i) {
    checkCudaError(cudaMalloc(&a[i], m * k * sizeof(TIn)));
    checkCudaError(cudaMalloc(&b[i], k * n * sizeof(TIn)));
    checkCudaError(cudaMalloc(&c[i], m * n * sizeof(TOut)));
    utils::populate_with_random(a[i], m * k, stream, 2025, static_cast<std::uint32_t>(3 * i + 1));
    utils::populate_with_random(b[i], k * n, stream, 2025, static_cast<std::uint32_t>(3 * i + 2));
    utils::populate_with_random(c[i], m * n, stream, 2025, static_cast<std::uint32_t>(3 * i + 3));
  }
  checkCudaError(cudaMalloc(&d_out, m * n * sizeof(TOut)));
  checkCudaError(cudaMalloc(&d_ref, m * n * sizeof(TOut)));

  Kernel kernel(m, n, k, properties);
  kernel(a[0], b[0], c[0], d_out, alpha, beta, stream);
  checkCudaError(cudaGetLastError());
  checkCudaError(cudaStreamSynchronize(stream));

  using LA = std::conditional_t<a_is_col<Kernel>::value, kf::ColMajor, kf::RowMajor>;
  using LB = std::conditional_t<b_is_col<Kernel>::value, kf::ColMajor, kf::RowMajor>;
  try {
    kf::cublasLt_gemm<TIn, TOut, LA, LB> reference(m, n, k, properties);
    reference(a[0], b[0], c[0], d_ref, alpha, beta, stream);
  } catch (const std::exception&) {
    kf::sm100_gemm<TIn, TOut, LA, LB, GZ_CFG_SIMT> reference(m, n, k, properties);
    reference(a[0], b[0], c[0], d_ref, alpha, beta, stream);
  }
  checkCudaError(cudaGetLastError());
  checkCudaError(cudaStreamSynchronize(stream));
  utils::compare_results(d_out, d_ref, m * n, stream, k);

  cudaEvent_t start, stop;
  checkCudaError(cudaEventCreate(&start));
  checkCudaError(cudaEventCreate(&stop));
  for (int w = 0; w < 5; ++w) kernel(a[w % sets], b[w % sets], c[w % sets], d_out, alpha, beta, stream);
  std::vector<float> times(reps);
  for (std::size_t i = 0; i < reps; ++i) {
    const std::size_t s = (i + 1) % sets;
    checkCudaError(cudaEventRecord(start, stream));
    kernel(a[s], b[s], c[s], d_out, alpha, beta, stream);
    checkCudaError(cudaEventRecord(stop, stream));
    checkCudaError(cudaEventSynchronize(stop));
    checkCudaError(cudaEventElapsedTime(&times[i], start, stop));
  }
  checkCudaError(cudaEventDestroy(start));
  checkCudaError(cudaEventDestroy(stop));

  double total = 0;
  for (float t : times) total += t;
  const double mean_ms = total / reps;
  std::vector<float> sorted = times;
  std::sort(sorted.begin(), sorted.end());
  const double median_ms = sorted[reps / 2], min_ms = sorted[0];
  const double ref_flops = static_cast<double>(m) * n * (2.0 * k + 3.0);
  const double flops = 2.0 * m * n * k;
  std::printf("GEMM Problem: [m: %lu n: %lu k: %lu], GFLOPS: %f  Time in ms: %f\n", (unsigned long)m,
              (unsigned long)n, (unsigned long)k, ref_flops * 1e-9 / (mean_ms * 1e-3), mean_ms);
  std::printf("{\"m\": %lu, \"n\": %lu, \"k\": %lu, \"reps\": %lu, \"buffer_sets\": %lu, \"ms_mean\": %.6f, "
              "\"ms_median\": %.6f, \"ms_min\": %.6f, \"tflops_median\": %.2f, \"tflops_best\": %.2f, "
              "\"tflops_mean_reference_convention\": %.2f}\n",
              (unsigned long)m, (unsigned long)n, (unsigned long)k, (unsigned long)reps, (unsigned long)sets,
              mean_ms, median_ms, min_ms, flops * 1e-12 / (median_ms * 1e-3), flops * 1e-12 / (min_ms * 1e-3),
              ref_flops * 1e-12 / (mean_ms * 1e-3));

  checkCudaError(cudaFree(d_out));
  checkCudaError(cudaFree(d_ref));
  for (std::size_t i = 0; i < sets; ++i) {
    checkCudaError(cudaFree(a[i]));
    checkCudaError(cudaFree(b[i]));
    checkCudaError(cudaFree(c[i]));
  }
}
}  // namespace detail

template <class Kernel, typename TIn, typename TOut>
void benchmark(std::vector<std::tuple<int, int, int>> problem_sizes, TOut alpha, TOut beta,
               const int num_repetitions = 50) {
  cudaStream_t stream;
  if (cudaStreamCreate(&stream) != cudaSuccess) throw std::runtime_error("Failed to create CUDA stream:");
  for (const auto& size_tuple : problem_sizes) {
    auto [m, n, k] = size_tuple;
    detail::benchmark_impl<Kernel, TIn, TOut>(m, n, k, alpha, beta, stream, num_repetitions);
  }
  cudaStreamDestroy(stream);
}

}  // namespace benchmark
#endif
