// CUDA-core GEMM used only when an operand cannot be described to TMA
// (base pointer not 16-byte aligned, or a leading dimension whose byte size is
// not a multiple of 16).  It plays the role the reference gives to
// nvidia::kernels::generic_gemm (nvidia/kernels/generic_gemm.cuh:5-60): any
// dtype, any extent, bounds-checked, C skipped when beta == 0 — extended with
// element strides so that row- and column-major A and B share one kernel, and
// with an exact int32 path for s8.
#ifndef GZ_SIMT_GEMM_CUH
#define GZ_SIMT_GEMM_CUH

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <type_traits>

namespace gz {

struct SimtParams {
  const void* a;
  const void* b;
  const void* c;
  void* d;
  int64_t m, n, k;
  int64_t a_sm, a_sk;  // element strides of A along m and k
  int64_t b_sk, b_sn;  // element strides of B along k and n
  int64_t ldc, ldd;
  int64_t batch, stride_a, stride_b, stride_c, stride_d;  // problems along blockIdx.z, strides in elements
  float alpha_f, beta_f;
  int32_t alpha_i, beta_i;
  // optional epilogue terms (float outputs): D = act(alpha * rs[i] * cs[j] * acc + beta * C + bias[j])
  uint32_t epi_flags, act;
  const float* bias;
  const float* row_scale;
  const float* col_scale;
};

namespace detail {
template <typename T>
__device__ __forceinline__ float simt_to_f(T v) {
  return static_cast<float>(v);
}
template <>
__device__ __forceinline__ float simt_to_f<__half>(__half v) {
  return __half2float(v);
}
template <>
__device__ __forceinline__ float simt_to_f<__nv_bfloat16>(__nv_bfloat16 v) {
  return __bfloat162float(v);
}
template <>
__device__ __forceinline__ float simt_to_f<__nv_fp8_e4m3>(__nv_fp8_e4m3 v) {
  return static_cast<float>(v);
}
template <>
__device__ __forceinline__ float simt_to_f<__nv_fp8_e5m2>(__nv_fp8_e5m2 v) {
  return static_cast<float>(v);
}
template <typename T>
__device__ __forceinline__ T simt_from_f(float v) {
  return static_cast<T>(v);
}
template <>
__device__ __forceinline__ __half simt_from_f<__half>(float v) {
  return __float2half_rn(v);
}
template <>
__device__ __forceinline__ __nv_bfloat16 simt_from_f<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}
__device__ __forceinline__ float simt_activate(float x, uint32_t act) {
  switch (act) {
    case 1: return fmaxf(x, 0.0f);
    case 2: return 0.5f * x * (1.0f + erff(x * 0.70710678118654752f));
    case 3: {
      const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
      return 0.5f * x * (1.0f + tanhf(u));
    }
    case 4: return x / (1.0f + __expf(-x));
    default: return x;
  }
}
}  // namespace detail

// 64x64 output tile per 256-thread block, 16-deep K slices, 4x4 outputs per thread.
template <typename TIn, typename TOut>
__global__ void __launch_bounds__(256) simt_gemm_kernel(const SimtParams p) {
  constexpr int TM = 64, TN = 64, TK = 16;
  constexpr bool INT = std::is_same<TIn, int8_t>::value;
  using Acc = typename std::conditional<INT, int32_t, float>::type;
  __shared__ Acc sa[TK][TM + 1];
  __shared__ Acc sb[TK][TN + 1];

  const TIn* a = static_cast<const TIn*>(p.a) + static_cast<int64_t>(blockIdx.z) * p.stride_a;
  const TIn* b = static_cast<const TIn*>(p.b) + static_cast<int64_t>(blockIdx.z) * p.stride_b;
  const int64_t m0 = static_cast<int64_t>(blockIdx.y) * TM;
  const int64_t n0 = static_cast<int64_t>(blockIdx.x) * TN;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;

  Acc acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0;

  for (int64_t k0 = 0; k0 < p.k; k0 += TK) {
    for (int e = threadIdx.x; e < TM * TK; e += 256) {
      // Walk the contiguous dimension with the fastest-varying index.
      const int mm = (p.a_sk == 1) ? e / TK : e % TM;
      const int kk = (p.a_sk == 1) ? e % TK : e / TM;
      const int64_t gm = m0 + mm, gk = k0 + kk;
      Acc v = 0;
      if (gm < p.m && gk < p.k) {
        if constexpr (INT) v = static_cast<int32_t>(a[gm * p.a_sm + gk * p.a_sk]);
        else v = detail::simt_to_f(a[gm * p.a_sm + gk * p.a_sk]);
      }
      sa[kk][mm] = v;
    }
    for (int e = threadIdx.x; e < TN * TK; e += 256) {
      const int nn = (p.b_sk == 1) ? e / TK : e % TN;
      const int kk = (p.b_sk == 1) ? e % TK : e / TN;
      const int64_t gn = n0 + nn, gk = k0 + kk;
      Acc v = 0;
      if (gn < p.n && gk < p.k) {
        if constexpr (INT) v = static_cast<int32_t>(b[gk * p.b_sk + gn * p.b_sn]);
        else v = detail::simt_to_f(b[gk * p.b_sk + gn * p.b_sn]);
      }
      sb[kk][nn] = v;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < TK; ++kk) {
      Acc av[4], bv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) av[i] = sa[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) bv[j] = sb[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] += av[i] * bv[j];
    }
    __syncthreads();
  }

  const TOut* c = static_cast<const TOut*>(p.c) + static_cast<int64_t>(blockIdx.z) * p.stride_c;
  TOut* d = static_cast<TOut*>(p.d) + static_cast<int64_t>(blockIdx.z) * p.stride_d;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int64_t gm = m0 + ty * 4 + i;
    if (gm >= p.m) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int64_t gn = n0 + tx * 4 + j;
      if (gn >= p.n) continue;
      if constexpr (std::is_same<TOut, int32_t>::value) {
        uint32_t v = static_cast<uint32_t>(p.alpha_i) * static_cast<uint32_t>(acc[i][j]);
        if (p.beta_i != 0)
          v += static_cast<uint32_t>(p.beta_i) * static_cast<uint32_t>(c[gm * p.ldc + gn]);
        d[gm * p.ldd + gn] = static_cast<int32_t>(v);
      } else {
        float v = p.alpha_f * static_cast<float>(acc[i][j]);
        if (p.epi_flags) {
          if (p.row_scale) v *= p.row_scale[gm];
          if (p.col_scale) v *= p.col_scale[gn];
        }
        if (p.beta_f != 0.0f) v = fmaf(p.beta_f, detail::simt_to_f(c[gm * p.ldc + gn]), v);
        if (p.epi_flags) {
          if (p.bias) v += p.bias[gn];
          v = detail::simt_activate(v, p.act);
        }
        d[gm * p.ldd + gn] = detail::simt_from_f<TOut>(v);
      }
    }
  }
}

}  // namespace gz
#endif
