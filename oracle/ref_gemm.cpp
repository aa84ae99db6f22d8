// TEST INFRASTRUCTURE — not part of the product.  Only tests/, the smoke check
// and the CPU-baseline leg of bench.py may load this library.
//
// CPU restatement of the reference project's GEMM arithmetic.  AD2605/gemm-zoo
// has no host GEMM; its "reference" results come from three naive DEVICE
// kernels, whose arithmetic is restated here as plain loops:
//
//   intel/utils/reference_kernel.hpp:16-27  and  nvidia/kernels/naive_gemm.cuh:9-20
//       acc = 0; for i < k: acc += a[row*k+i] * b[i*n+col];
//       d[row*n+col] = alpha*acc + beta*c[row*n+col];
//   nvidia/kernels/generic_gemm.cuh:29-59
//       float sum over k ascending (tiles of 32, same order), leading dimensions,
//       val = TOut(sum)*alpha; if (beta != 0) val += beta*c[row*ldc+col]; d[row*ldd+col] = val;
//
// Three variants:
//   oracle_gemm_s8      int8 x int8 -> int32, exact (two's-complement wrap), the
//                       contract of intel/kernels/xe_gemm_s8_s8_s32_m8k16.hpp:19,68-71
//   oracle_gemm_f64     inputs converted exactly, products and sums in double,
//                       alpha/beta in double, result returned as double (the
//                       caller rounds once to the output type): the tolerance oracle
//   oracle_gemm_f32seq  generic_gemm's own arithmetic: fp32 fused multiply-add over k
//                       ascending, epilogue in fp32 — reference-faithful, used to
//                       pin this file against the reference kernels themselves
//
// Parity pin: the reference ships no golden vectors.  This file is pinned by
// tests/golden/*.npz, which hold outputs of the reference's generic_gemm and
// naive_gemm kernels (compiled unmodified from the reference sources by
// oracle/ref_kernels_wrap.cu and run on a B200) for the seeded inputs that
// tests/golden/make_golden.py generates.
//
// Operands are addressed with element strides so that row- and column-major A
// and B use one code path:  A(i,kk) = a[i*a_sm + kk*a_sk],  B(kk,j) = b[kk*b_sk + j*b_sn].
#include <omp.h>
#include <stdint.h>
#include <string.h>

#include <cmath>
#include <vector>

namespace {

enum { DT_F16 = 0, DT_BF16 = 1, DT_F32 = 2, DT_S8 = 3, DT_S32 = 4, DT_E4M3 = 5, DT_E5M2 = 6 };

inline float bf16_to_f32(uint16_t h) {
  uint32_t u = static_cast<uint32_t>(h) << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

inline float f16_to_f32(uint16_t h) {
  const uint32_t sign = (h >> 15) & 1u, exp = (h >> 10) & 0x1Fu, man = h & 0x3FFu;
  float v;
  if (exp == 0) v = std::ldexp(static_cast<float>(man), -24);
  else if (exp == 31) v = man ? NAN : INFINITY;
  else v = std::ldexp(static_cast<float>(man | 0x400u), static_cast<int>(exp) - 25);
  return sign ? -v : v;
}

// 8-bit floats.  e4m3 (the "fn" flavour CUDA uses): bias 7, no infinities, S.1111.111 is NaN.
inline float e4m3_to_f32(uint8_t v) {
  const uint32_t sign = v >> 7, exp = (v >> 3) & 0xFu, man = v & 0x7u;
  float f;
  if (exp == 0) f = std::ldexp(static_cast<float>(man), -9);
  else if (exp == 15 && man == 7) f = NAN;
  else f = std::ldexp(static_cast<float>(man | 0x8u), static_cast<int>(exp) - 10);
  return sign ? -f : f;
}
// e5m2: bias 15, IEEE-style infinities and NaNs (it is the top byte of an fp16).
inline float e5m2_to_f32(uint8_t v) { return f16_to_f32(static_cast<uint16_t>(v) << 8); }

// tf32 views of an fp32 value: mode 1 drops the low 13 mantissa bits, mode 2
// rounds to nearest with ties away from zero (cvt.rna.tf32.f32).
inline float to_tf32(float f, int mode) {
  if (mode == 0) return f;
  uint32_t u;
  memcpy(&u, &f, 4);
  if (mode == 2 && ((u >> 23) & 0xFFu) != 0xFFu) u += 0x1000u;
  u &= 0xFFFFE000u;
  memcpy(&f, &u, 4);
  return f;
}

inline float load_as_f32(const void* p, int dt, int64_t idx) {
  switch (dt) {
    case DT_F16: return f16_to_f32(static_cast<const uint16_t*>(p)[idx]);
    case DT_BF16: return bf16_to_f32(static_cast<const uint16_t*>(p)[idx]);
    case DT_F32: return static_cast<const float*>(p)[idx];
    case DT_S8: return static_cast<float>(static_cast<const int8_t*>(p)[idx]);
    case DT_S32: return static_cast<float>(static_cast<const int32_t*>(p)[idx]);
    case DT_E4M3: return e4m3_to_f32(static_cast<const uint8_t*>(p)[idx]);
    case DT_E5M2: return e5m2_to_f32(static_cast<const uint8_t*>(p)[idx]);
  }
  return 0.f;
}

inline double load_as_f64(const void* p, int dt, int64_t idx) {
  if (dt == DT_S32) return static_cast<double>(static_cast<const int32_t*>(p)[idx]);
  return static_cast<double>(load_as_f32(p, dt, idx));
}

// Pack all of B as fp32 (exact for every supported input type), row-major with n contiguous.
void pack_b(std::vector<float>& out, const void* b, int dt, int64_t k, int64_t n, int64_t b_sk,
            int64_t b_sn, int tf32_mode) {
  out.resize(static_cast<size_t>(k) * n);
#pragma omp parallel for schedule(static)
  for (int64_t kk = 0; kk < k; ++kk)
    for (int64_t j = 0; j < n; ++j)
      out[kk * n + j] = to_tf32(load_as_f32(b, dt, kk * b_sk + j * b_sn), tf32_mode);
}

}  // namespace

extern "C" {

int oracle_num_threads() { return omp_get_max_threads(); }
void oracle_set_threads(int n) {
  if (n > 0) omp_set_num_threads(n);
}

// Rows may be restricted to a list (row_idx, nrows) so that large problems can
// be checked on a sample; row_idx == NULL means all m rows.  Output row r of
// `d` (ld = n) corresponds to row_idx[r].
int oracle_gemm_f64(int in_type, int out_type, const void* a, const void* b, const void* c,
                    double* d, int64_t m, int64_t n, int64_t k, int64_t a_sm, int64_t a_sk,
                    int64_t b_sk, int64_t b_sn, int64_t ldc, double alpha, double beta,
                    int tf32_mode, const int64_t* row_idx, int64_t nrows) {
  if (!a || !b || !d || m <= 0 || n <= 0 || k <= 0) return 1;
  if (beta != 0.0 && !c) return 1;
  if (!row_idx) nrows = m;
  std::vector<float> bp;
  pack_b(bp, b, in_type, k, n, b_sk, b_sn, tf32_mode);
  const int64_t IB = 8;
#pragma omp parallel
  {
    std::vector<double> acc(static_cast<size_t>(IB) * n);
    std::vector<float> arow(static_cast<size_t>(IB) * k);
#pragma omp for schedule(dynamic, 1)
    for (int64_t r0 = 0; r0 < nrows; r0 += IB) {
      const int64_t rb = (nrows - r0 < IB) ? (nrows - r0) : IB;
      for (int64_t r = 0; r < rb; ++r) {
        const int64_t i = row_idx ? row_idx[r0 + r] : (r0 + r);
        for (int64_t kk = 0; kk < k; ++kk)
          arow[r * k + kk] = to_tf32(load_as_f32(a, in_type, i * a_sm + kk * a_sk), tf32_mode);
      }
      std::fill(acc.begin(), acc.end(), 0.0);
      // k ascending for every output; the product of two values with <= 24-bit
      // significands is exact in double, so each step is one rounding.
      for (int64_t kk = 0; kk < k; ++kk) {
        const float* brow = &bp[kk * n];
        for (int64_t r = 0; r < rb; ++r) {
          const double av = static_cast<double>(arow[r * k + kk]);
          double* ar = &acc[r * n];
#pragma omp simd
          for (int64_t j = 0; j < n; ++j) ar[j] += av * static_cast<double>(brow[j]);
        }
      }
      for (int64_t r = 0; r < rb; ++r) {
        const int64_t i = row_idx ? row_idx[r0 + r] : (r0 + r);
        for (int64_t j = 0; j < n; ++j) {
          double v = alpha * acc[r * n + j];
          if (beta != 0.0) v += beta * load_as_f64(c, out_type, i * ldc + j);
          d[(r0 + r) * n + j] = v;
        }
      }
    }
  }
  return 0;
}

// Exact s8 x s8 -> s32 with int32 alpha/beta; arithmetic wraps modulo 2^32.
int oracle_gemm_s8(const int8_t* a, const int8_t* b, const int32_t* c, int32_t* d, int64_t m,
                   int64_t n, int64_t k, int64_t a_sm, int64_t a_sk, int64_t b_sk, int64_t b_sn,
                   int64_t ldc, int64_t ldd, int32_t alpha, int32_t beta, const int64_t* row_idx,
                   int64_t nrows) {
  if (!a || !b || !d || m <= 0 || n <= 0 || k <= 0) return 1;
  if (beta != 0 && !c) return 1;
  if (!row_idx) nrows = m;
  std::vector<int16_t> bp(static_cast<size_t>(k) * n);
#pragma omp parallel for schedule(static)
  for (int64_t kk = 0; kk < k; ++kk)
    for (int64_t j = 0; j < n; ++j) bp[kk * n + j] = b[kk * b_sk + j * b_sn];
  const int64_t IB = 8;
#pragma omp parallel
  {
    std::vector<uint32_t> acc(static_cast<size_t>(IB) * n);
#pragma omp for schedule(dynamic, 1)
    for (int64_t r0 = 0; r0 < nrows; r0 += IB) {
      const int64_t rb = (nrows - r0 < IB) ? (nrows - r0) : IB;
      std::fill(acc.begin(), acc.end(), 0u);
      for (int64_t kk = 0; kk < k; ++kk) {
        const int16_t* brow = &bp[kk * n];
        for (int64_t r = 0; r < rb; ++r) {
          const int64_t i = row_idx ? row_idx[r0 + r] : (r0 + r);
          const int32_t av = a[i * a_sm + kk * a_sk];
          uint32_t* ar = &acc[r * n];
#pragma omp simd
          for (int64_t j = 0; j < n; ++j)
            ar[j] += static_cast<uint32_t>(av * static_cast<int32_t>(brow[j]));
        }
      }
      for (int64_t r = 0; r < rb; ++r) {
        const int64_t i = row_idx ? row_idx[r0 + r] : (r0 + r);
        for (int64_t j = 0; j < n; ++j) {
          uint32_t v = static_cast<uint32_t>(alpha) * acc[r * n + j];
          if (beta != 0) v += static_cast<uint32_t>(beta) * static_cast<uint32_t>(c[i * ldc + j]);
          d[(r0 + r) * ldd + j] = static_cast<int32_t>(v);
        }
      }
    }
  }
  return 0;
}

// generic_gemm's arithmetic (nvidia/kernels/generic_gemm.cuh:29-59) for fp32
// output: sum = fma(a, b, sum) over k ascending in fp32 (nvcc contracts
// `sum += x * y` into one FFMA); val = sum * alpha; if (beta != 0)
// val = fma(beta, c, val).  Result as fp32 (ld = n).
int oracle_gemm_f32seq(int in_type, const void* a, const void* b, const float* c, float* d,
                       int64_t m, int64_t n, int64_t k, int64_t a_sm, int64_t a_sk, int64_t b_sk,
                       int64_t b_sn, int64_t ldc, float alpha, float beta) {
  if (!a || !b || !d || m <= 0 || n <= 0 || k <= 0) return 1;
  if (beta != 0.0f && !c) return 1;
  std::vector<float> bp;
  pack_b(bp, b, in_type, k, n, b_sk, b_sn, 0);
#pragma omp parallel
  {
    std::vector<float> acc(static_cast<size_t>(n));
#pragma omp for schedule(dynamic, 4)
    for (int64_t i = 0; i < m; ++i) {
      std::fill(acc.begin(), acc.end(), 0.0f);
      for (int64_t kk = 0; kk < k; ++kk) {
        const float av = load_as_f32(a, in_type, i * a_sm + kk * a_sk);
        const float* brow = &bp[kk * n];
        for (int64_t j = 0; j < n; ++j) acc[j] = std::fmaf(av, brow[j], acc[j]);
      }
      for (int64_t j = 0; j < n; ++j) {
        float v = acc[j] * alpha;
        if (beta != 0.0f) v = std::fmaf(beta, c[i * ldc + j], v);
        d[i * n + j] = v;
      }
    }
  }
  return 0;
}

// Sum over k of |a_ik| * |b_kj| for sampled rows (the scale of the componentwise
// error bound), as double, ld = n.
int oracle_abs_gemm(int in_type, const void* a, const void* b, double* d, int64_t m, int64_t n,
                    int64_t k, int64_t a_sm, int64_t a_sk, int64_t b_sk, int64_t b_sn,
                    const int64_t* row_idx, int64_t nrows) {
  if (!a || !b || !d) return 1;
  if (!row_idx) nrows = m;
  std::vector<float> bp;
  pack_b(bp, b, in_type, k, n, b_sk, b_sn, 0);
#pragma omp parallel
  {
    std::vector<double> acc(static_cast<size_t>(n));
#pragma omp for schedule(dynamic, 4)
    for (int64_t r = 0; r < nrows; ++r) {
      const int64_t i = row_idx ? row_idx[r] : r;
      std::fill(acc.begin(), acc.end(), 0.0);
      for (int64_t kk = 0; kk < k; ++kk) {
        const double av = std::fabs(static_cast<double>(load_as_f32(a, in_type, i * a_sm + kk * a_sk)));
        const float* brow = &bp[kk * n];
#pragma omp simd
        for (int64_t j = 0; j < n; ++j) acc[j] += av * std::fabs(static_cast<double>(brow[j]));
      }
      for (int64_t j = 0; j < n; ++j) d[r * n + j] = acc[j];
    }
  }
  return 0;
}

}  // extern "C"
