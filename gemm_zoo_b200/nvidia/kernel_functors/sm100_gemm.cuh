// Host functor for the sm_100a GEMM, satisfying the functor concept of the
// reference's nvidia/kernel_functors (e.g. bf16_mma_gemm.cuh:15-72):
//
//   Kernel kernel(m, n, k, properties);                 // nvidia/utils/benchmark.cuh:54
//   kernel(a, b, c, d, alpha, beta, stream);            // nvidia/utils/benchmark.cuh:56-57
//
// so it can be handed to benchmark::benchmark<Kernel, TIn, TOut> unchanged.
// Differences from the reference functors:
//   - one template serves every dtype pair: (half,half), (half,float),
//     (bf16,bf16), (bf16,float), (float,float) = tf32 multiply, (int8,int32),
//     (fp8 e4m3 / e5m2, half | bf16 | float);
//   - A and B may each be row- or column-major (template tags) and an extended
//     constructor takes lda/ldb/ldc/ldd; the 4-argument constructor keeps the
//     reference convention A[m x k] ld=k, B[k x n] ld=n, C/D[m x n] ld=n
//     (nvidia/kernels/naive_gemm.cuh:18-20);
//   - no divisibility requirement on m, n, k;
//   - alpha/beta arrive as TOut (as in the reference) and are applied in fp32
//     (int32 for s8) on top of an fp32 (int32) accumulator;
//   - construction failures throw std::runtime_error instead of assert/exit.
// All work is delegated to the C ABI in gemmzoo/gemm.h.
#ifndef GZ_NVIDIA_KERNEL_FUNCTORS_SM100_GEMM_CUH
#define GZ_NVIDIA_KERNEL_FUNCTORS_SM100_GEMM_CUH

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>
#include <type_traits>

#include "defines.hpp"
#include "gemmzoo/gemm.h"

namespace nvidia::kernel_functors {

struct RowMajor {};
struct ColMajor {};

namespace detail {
template <typename T>
constexpr int gz_dtype_of() {
  if constexpr (std::is_same_v<T, __half>) return GZ_DT_F16;
  else if constexpr (std::is_same_v<T, __nv_bfloat16>) return GZ_DT_BF16;
  else if constexpr (std::is_same_v<T, float>) return GZ_DT_F32;
  else if constexpr (std::is_same_v<T, std::int8_t>) return GZ_DT_S8;
  else if constexpr (std::is_same_v<T, std::int32_t>) return GZ_DT_S32;
  else if constexpr (std::is_same_v<T, __nv_fp8_e4m3>) return GZ_DT_E4M3;
  else if constexpr (std::is_same_v<T, __nv_fp8_e5m2>) return GZ_DT_E5M2;
  else static_assert(sizeof(T) == 0, "unsupported element type");
}
template <typename T>
inline float scalar_to_float(T v) {
  if constexpr (std::is_same_v<T, __half>) return __half2float(v);
  else if constexpr (std::is_same_v<T, __nv_bfloat16>) return __bfloat162float(v);
  else return static_cast<float>(v);
}
}  // namespace detail

template <typename TIn, typename TOut, typename LayoutA = RowMajor, typename LayoutB = RowMajor,
          int Config = GZ_CFG_AUTO>
struct sm100_gemm {
  static constexpr bool a_col_major = std::is_same_v<LayoutA, ColMajor>;
  static constexpr bool b_col_major = std::is_same_v<LayoutB, ColMajor>;

  sm100_gemm(std::size_t m, std::size_t n, std::size_t k, const cudaDeviceProp& properties)
      : sm100_gemm(m, n, k, 0, 0, 0, 0, properties) {}

  // Leading dimensions in elements; 0 selects the packed value for the layout.
  sm100_gemm(std::size_t m, std::size_t n, std::size_t k, std::size_t lda, std::size_t ldb,
             std::size_t ldc, std::size_t ldd, const cudaDeviceProp&) {
    gz_gemm_desc desc{};
    desc.struct_size = sizeof(desc);
    desc.in_type = detail::gz_dtype_of<TIn>();
    desc.out_type = detail::gz_dtype_of<TOut>();
    desc.layout_a = std::is_same_v<LayoutA, ColMajor> ? GZ_COL_MAJOR : GZ_ROW_MAJOR;
    desc.layout_b = std::is_same_v<LayoutB, ColMajor> ? GZ_COL_MAJOR : GZ_ROW_MAJOR;
    int device = 0;
    checkCudaError(cudaGetDevice(&device));
    desc.device = device;
    desc.config = Config;
    desc.m = static_cast<std::int64_t>(m);
    desc.n = static_cast<std::int64_t>(n);
    desc.k = static_cast<std::int64_t>(k);
    desc.lda = static_cast<std::int64_t>(lda);
    desc.ldb = static_cast<std::int64_t>(ldb);
    desc.ldc = static_cast<std::int64_t>(ldc);
    desc.ldd = static_cast<std::int64_t>(ldd);
    checkGzStatus(gz_gemm_plan_create(&plan_, &desc), "sm100_gemm");
  }

  sm100_gemm(const sm100_gemm&) = delete;
  sm100_gemm& operator=(const sm100_gemm&) = delete;
  sm100_gemm(sm100_gemm&& o) noexcept : plan_(o.plan_) { o.plan_ = nullptr; }

  ~sm100_gemm() {
    if (plan_) gz_gemm_plan_destroy(plan_);
  }

  // One asynchronous launch on `stream`; D may alias C; C is not read when beta == 0.
  void operator()(const TIn* a, const TIn* b, const TOut* c, TOut* d, const TOut alpha,
                  const TOut beta, cudaStream_t stream) {
    // The C ABI reads int32 scalars exactly when the OUTPUT type is s32; an s8 GEMM with a
    // floating-point output (dequantising) takes float scalars like every other float output.
    if constexpr (std::is_same_v<TOut, std::int32_t>) {
      const std::int32_t al = static_cast<std::int32_t>(alpha), be = static_cast<std::int32_t>(beta);
      checkGzStatus(gz_gemm_run(plan_, a, b, c, d, &al, &be, stream), "sm100_gemm::operator()");
    } else {
      const float al = detail::scalar_to_float(alpha), be = detail::scalar_to_float(beta);
      checkGzStatus(gz_gemm_run(plan_, a, b, c, d, &al, &be, stream), "sm100_gemm::operator()");
    }
  }

  gz_plan_info info() const {
    gz_plan_info i{};
    gz_gemm_plan_info(plan_, &i);
    return i;
  }

  // GZ_OK, or GZ_ERR_DEVICE_TIMEOUT if a bounded in-kernel wait expired (synchronises `stream`).
  gz_status device_status(cudaStream_t stream) { return gz_last_device_status(plan_, stream, nullptr); }

 private:
  gz_plan* plan_ = nullptr;
};

}  // namespace nvidia::kernel_functors
#endif
