// TEST INFRASTRUCTURE — not part of the product.
//
// Launch glue around the reference project's OWN kernels, which are included
// from the reference source tree where it lies (-I<reference>/nvidia); no
// reference source is copied into this repository.  The result,
// oracle/_ref/libref_kernels.so, is used
//   - to pin the CPU oracle (oracle/ref_gemm.cpp) against what the reference's
//     generic_gemm / naive_gemm kernels actually compute, and
//   - as a secondary GPU comparator (the reference's mma.sync kernels
//     recompiled for sm_100a) in the benchmark report.
//
// Functors wrapped, with the template arguments their bench mains use:
//   nvidia/kernel_functors/generic_gemm.cuh:13-43   generic_gemm<TIn,TOut>
//   nvidia/kernel_functors/naive_gemm.cuh:11-33     naive_gemm<TIn,TOut>
//   nvidia/kernel_functors/bf16_mma_gemm.cuh:15-72  compiled but never launched (see ref_mma_gemm)
//   nvidia/kernel_functors/fp16_mma_gemm.cuh:15-70  <half,half,256,256,32>   (nvidia/bench/bench_fp16_mma_gemm.cu:10-18)
//   nvidia/kernel_functors/tf32_mma_gemm.cuh:14-61  <float,float,128,128,32> (nvidia/bench/bench_tf32_mma_gemm.cu:9-17)
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <type_traits>

#include "kernel_functors/bf16_mma_gemm.cuh"
#include "kernel_functors/fp16_mma_gemm.cuh"
#include "kernel_functors/generic_gemm.cuh"
#include "kernel_functors/naive_gemm.cuh"
#include "kernel_functors/tf32_mma_gemm.cuh"

namespace {
enum { DT_F16 = 0, DT_BF16 = 1, DT_F32 = 2, DT_S8 = 3, DT_S32 = 4 };

template <typename T>
T scalar_from(double v) {
  if constexpr (std::is_same_v<T, __half>) return __float2half(static_cast<float>(v));
  else if constexpr (std::is_same_v<T, __nv_bfloat16>) return __float2bfloat16(static_cast<float>(v));
  else return static_cast<T>(v);
}

template <typename TIn, typename TOut>
int run_generic(const void* a, const void* b, const void* c, void* d, size_t m, size_t n, size_t k,
                double alpha, double beta, cudaStream_t s) {
  nvidia::kernel_functors::generic_gemm<TIn, TOut> f(m, n, k);
  f(static_cast<const TIn*>(a), static_cast<const TIn*>(b), static_cast<const TOut*>(c),
    static_cast<TOut*>(d), scalar_from<TOut>(alpha), scalar_from<TOut>(beta), s);
  return static_cast<int>(cudaGetLastError());
}

template <typename TIn, typename TOut>
int run_naive(const void* a, const void* b, const void* c, void* d, size_t m, size_t n, size_t k,
              double alpha, double beta, cudaStream_t s) {
  cudaDeviceProp prop;
  int dev = 0;
  cudaGetDevice(&dev);
  cudaGetDeviceProperties(&prop, dev);
  nvidia::kernel_functors::naive_gemm<TIn, TOut> f(m, n, k, prop);
  f(static_cast<const TIn*>(a), static_cast<const TIn*>(b), static_cast<const TOut*>(c),
    static_cast<TOut*>(d), scalar_from<TOut>(alpha), scalar_from<TOut>(beta), s);
  return static_cast<int>(cudaGetLastError());
}
}  // namespace

extern "C" {

// Reference convention only: A row-major ld=k, B row-major ld=n, C/D row-major ld=n.
int ref_generic_gemm(int in_type, int out_type, const void* a, const void* b, const void* c, void* d,
                     int64_t m, int64_t n, int64_t k, double alpha, double beta, void* stream) {
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (in_type == DT_F32 && out_type == DT_F32) return run_generic<float, float>(a, b, c, d, m, n, k, alpha, beta, s);
  if (in_type == DT_BF16 && out_type == DT_F32) return run_generic<__nv_bfloat16, float>(a, b, c, d, m, n, k, alpha, beta, s);
  if (in_type == DT_F16 && out_type == DT_F32) return run_generic<__half, float>(a, b, c, d, m, n, k, alpha, beta, s);
  if (in_type == DT_F16 && out_type == DT_F16) return run_generic<__half, __half>(a, b, c, d, m, n, k, alpha, beta, s);
  if (in_type == DT_BF16 && out_type == DT_BF16) return run_generic<__nv_bfloat16, __nv_bfloat16>(a, b, c, d, m, n, k, alpha, beta, s);
  if (in_type == DT_S8 && out_type == DT_S32) return run_generic<int8_t, int32_t>(a, b, c, d, m, n, k, alpha, beta, s);
  return -1;
}

int ref_naive_gemm(int in_type, int out_type, const void* a, const void* b, const void* c, void* d,
                   int64_t m, int64_t n, int64_t k, double alpha, double beta, void* stream) {
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (in_type == DT_F32 && out_type == DT_F32) return run_naive<float, float>(a, b, c, d, m, n, k, alpha, beta, s);
  if (in_type == DT_S8 && out_type == DT_S32) return run_naive<int8_t, int32_t>(a, b, c, d, m, n, k, alpha, beta, s);
  return -1;
}

// The reference's tensor-core kernels; m, n, k must be multiples of the tile and
// the tile grid a power-of-two square (its Hilbert rasteriser), as in its benches.
int ref_mma_gemm(int in_type, const void* a, const void* b, const void* c, void* d, int64_t m,
                 int64_t n, int64_t k, double alpha, double beta, void* stream) {
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaDeviceProp prop;
  int dev = 0;
  cudaGetDevice(&dev);
  cudaGetDeviceProperties(&prop, dev);
  if (in_type == DT_BF16) {
    // Not run: nvidia/kernel_functors/bf16_mma_gemm.cuh:34-35 sizes the epilogue staging area with
    // sizeof(bf16) while nvidia/kernels/sm_80/bf16_mma_gemm.cuh:34-35 strides it as float, so the
    // kernel writes 1 KB past its shared-memory allocation.
    return -3;
  } else if (in_type == DT_F16) {
    if (m % 256 || n % 256 || k % 32) return -2;
    nvidia::kernel_functors::fp16_mma_gemm<__half, __half, 256, 256, 32> f(m, n, k, prop);
    f(static_cast<const __half*>(a), static_cast<const __half*>(b), static_cast<const __half*>(c),
      static_cast<__half*>(d), __float2half(static_cast<float>(alpha)),
      __float2half(static_cast<float>(beta)), s);
  } else if (in_type == DT_F32) {
    if (m % 128 || n % 128 || k % 32) return -2;
    nvidia::kernel_functors::tf32_mma_gemm<float, float, 128, 128, 32> f(m, n, k, prop);
    f(static_cast<const float*>(a), static_cast<const float*>(b), static_cast<const float*>(c),
      static_cast<float*>(d), static_cast<float>(alpha), static_cast<float>(beta), s);
  } else {
    return -1;
  }
  return static_cast<int>(cudaGetLastError());
}

}  // extern "C"
