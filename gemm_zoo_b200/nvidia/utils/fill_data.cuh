// Seeded operand fill for the harness.  Same entry point as the reference's
// utils::populate_with_random (nvidia/utils/fill_data.cuh:33-49) — which keeps a
// 48-byte generator state per element and gives every buffer the same values —
// but stateless: element i of a buffer depends only on (seed, stream_id, i), and
// callers pass a different stream_id per operand.
#ifndef GZ_NVIDIA_UTILS_FILL_DATA_CUH
#define GZ_NVIDIA_UTILS_FILL_DATA_CUH

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>
#include <type_traits>

#include "defines.hpp"
#include "gemmzoo/gemm.h"

namespace utils {

template <typename T>
constexpr int gz_dtype_code() {
  if constexpr (std::is_same_v<T, __half>) return GZ_DT_F16;
  else if constexpr (std::is_same_v<T, __nv_bfloat16>) return GZ_DT_BF16;
  else if constexpr (std::is_same_v<T, float>) return GZ_DT_F32;
  else if constexpr (std::is_same_v<T, std::int8_t>) return GZ_DT_S8;
  else if constexpr (std::is_same_v<T, std::int32_t>) return GZ_DT_S32;
  else if constexpr (std::is_same_v<T, __nv_fp8_e4m3>) return GZ_DT_E4M3;
  else if constexpr (std::is_same_v<T, __nv_fp8_e5m2>) return GZ_DT_E5M2;
  else static_assert(sizeof(T) == 0, "unsupported element type");
}

// N(0, scale^2) for floating types; uniform integers for s8 (full range) and s32 ([-scale, scale]).
template <typename T>
void populate_with_random(T* device_ptr, std::size_t num_elements, cudaStream_t stream,
                          std::uint64_t seed = 2025, std::uint32_t stream_id = 0, float scale = 1.0f) {
  constexpr bool is_int = std::is_integral_v<T>;
  checkGzStatus(gz_fill(device_ptr, gz_dtype_code<T>(), static_cast<std::int64_t>(num_elements), seed,
                        stream_id, is_int ? 2 : 1, is_int ? 100.0f * scale : scale, stream),
                "populate_with_random");
}

}  // namespace utils
#endif
