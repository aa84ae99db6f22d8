// Result check for the harness.  The reference flags |out - ref| > 0.5
// (nvidia/utils/compare.cuh:19-22), an absolute bar that means nothing once the
// result grows like sqrt(k); here integers must match exactly and floating
// point must satisfy |out - ref| <= atol + rtol * |ref| with the bars scaled to
// the output type and to k.
#ifndef GZ_NVIDIA_UTILS_COMPARE_CUH
#define GZ_NVIDIA_UTILS_COMPARE_CUH

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cmath>
#include <cstddef>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <stdexcept>
#include <type_traits>

#include "defines.hpp"

namespace utils {

namespace detail {
template <typename T>
__device__ __forceinline__ double as_double(T v) {
  if constexpr (std::is_same_v<T, __half>) return static_cast<double>(__half2float(v));
  else if constexpr (std::is_same_v<T, __nv_bfloat16>) return static_cast<double>(__bfloat162float(v));
  else return static_cast<double>(v);
}
}  // namespace detail

struct compare_report {
  unsigned long long mismatches;
  double max_abs_err;
  unsigned long long first_index;
};

template <typename T>
__global__ void compare_results_kernel(const T* output, const T* reference, std::size_t num_elements,
                                       double atol, double rtol, unsigned long long* mismatches,
                                       unsigned long long* max_err_bits, unsigned long long* first_index) {
  const std::size_t stride = static_cast<std::size_t>(gridDim.x) * blockDim.x;
  for (std::size_t i = static_cast<std::size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < num_elements;
       i += stride) {
    const double o = detail::as_double(output[i]), r = detail::as_double(reference[i]);
    const double err = fabs(o - r);
    if (!(err <= atol + rtol * fabs(r))) {  // also catches NaN
      atomicAdd(mismatches, 1ull);
      atomicMin(first_index, static_cast<unsigned long long>(i));
    }
    if (err == err) atomicMax(max_err_bits, static_cast<unsigned long long>(__double_as_longlong(err)));
  }
}

// Throws std::runtime_error("verification failed") like the reference (nvidia/utils/compare.cuh:44-46).
// k scales the tolerance: two correct kernels may sum k products in different orders.
template <typename T>
compare_report compare_results(const T* output, const T* reference, std::size_t num_elements,
                               cudaStream_t stream, std::size_t k = 1, bool throw_on_mismatch = true) {
  double atol = 0.0, rtol = 0.0;
  if constexpr (std::is_same_v<T, __nv_bfloat16>) rtol = 1.0 / 64, atol = 1e-2 * std::sqrt(double(k));
  else if constexpr (std::is_same_v<T, __half>) rtol = 1.0 / 256, atol = 2e-3 * std::sqrt(double(k));
  else if constexpr (std::is_same_v<T, float>) rtol = 1.0 / 128, atol = 1e-2 * std::sqrt(double(k));  // tf32 products
  unsigned long long* dev = nullptr;
  checkCudaError(cudaMalloc(&dev, 3 * sizeof(unsigned long long)));
  const unsigned long long init[3] = {0ull, 0ull, ~0ull};
  checkCudaError(cudaMemcpyAsync(dev, init, sizeof(init), cudaMemcpyHostToDevice, stream));
  const int block = 256;
  const std::size_t want = (num_elements + block - 1) / block;
  const int grid = static_cast<int>(want < 4096 ? (want ? want : 1) : 4096);
  compare_results_kernel<<<grid, block, 0, stream>>>(output, reference, num_elements, atol, rtol, dev, dev + 1,
                                                     dev + 2);
  checkCudaError(cudaGetLastError());
  unsigned long long host[3];
  checkCudaError(cudaMemcpyAsync(host, dev, sizeof(host), cudaMemcpyDeviceToHost, stream));
  checkCudaError(cudaStreamSynchronize(stream));
  checkCudaError(cudaFree(dev));
  compare_report rep;
  rep.mismatches = host[0];
  long long bits = static_cast<long long>(host[1]);
  double e;
  static_assert(sizeof(e) == sizeof(bits));
  std::memcpy(&e, &bits, sizeof(e));
  rep.max_abs_err = e;
  rep.first_index = host[2];
  if (rep.mismatches && throw_on_mismatch) {
    std::printf("verification failed: %llu of %zu elements differ (first at %llu, max abs err %g)\n",
                rep.mismatches, num_elements, rep.first_index, rep.max_abs_err);
    std::fflush(stdout);
    throw std::runtime_error("verification failed");
  }
  return rep;
}
}  // namespace utils
#endif
