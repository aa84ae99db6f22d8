// cuBLASLt comparator functor: same constructor/call shape as the sm100_gemm
// functor, so both can be handed to benchmark::benchmark<Kernel, TIn, TOut>.
//
// Takes the place of the reference's comparator functor and one-shot helper
// (nvidia/kernel_functors/cublaslt_gemm.cuh:14-125, nvidia/utils/cublaslt_gemm.cuh:52-129)
// with three corrections: the row-major problem is described truthfully (the
// reference hands row-major buffers to default column-major layouts, which
// computes B*A and only verifies because it fills A and B identically); the
// compute types are the accurate ones (fp32 accumulate for fp16, int32 for s8);
// and everything the object owns is released.
//
// Row-major C/D (m x n, ld) is the column-major matrix D^T (n x m, ld), so the
// library is asked for  D^T = op(Bmem) * op(Amem):
//   B row-major (k x n, ldb)  = column-major n x k  -> no transpose
//   B col-major (ld >= k)     = column-major k x n  -> transpose
//   A row-major (m x k, lda)  = column-major k x m  -> no transpose
//   A col-major (ld >= m)     = column-major m x k  -> transpose
#ifndef GZ_NVIDIA_KERNEL_FUNCTORS_CUBLASLT_GEMM_CUH
#define GZ_NVIDIA_KERNEL_FUNCTORS_CUBLASLT_GEMM_CUH

#include <cublasLt.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>
#include <cstdio>
#include <stdexcept>
#include <string>
#include <type_traits>

namespace nvidia::kernel_functors {

struct RowMajor;
struct ColMajor;

// Runtime-typed core (dtype codes as gz_dtype: 0 f16, 1 bf16, 2 f32, 3 s8, 4 s32, 5 e4m3, 6 e5m2).
// fp8 inputs use fp32 compute (the reference's CUBLAS_COMPUTE_16F for fp8,
// nvidia/kernel_functors/cublaslt_gemm.cuh:106-109, is not a combination cuBLASLt offers).
class cublaslt_core {
 public:
  cublaslt_core(int in_type, int out_type, bool a_col_major, bool b_col_major, std::int64_t m,
                std::int64_t n, std::int64_t k, std::int64_t lda, std::int64_t ldb, std::int64_t ldc,
                std::int64_t ldd, std::size_t workspace_bytes)
      : in_type_(in_type) {
    if (lda == 0) lda = a_col_major ? m : k;
    if (ldb == 0) ldb = b_col_major ? k : n;
    if (ldc == 0) ldc = n;
    if (ldd == 0) ldd = n;
    cublasComputeType_t compute;
    cudaDataType_t scale;
    if (in_type == 3) {
      compute = CUBLAS_COMPUTE_32I;
      scale = CUDA_R_32I;
    } else if (in_type == 2) {
      compute = CUBLAS_COMPUTE_32F_FAST_TF32;
      scale = CUDA_R_32F;
    } else {
      compute = CUBLAS_COMPUTE_32F;
      scale = CUDA_R_32F;
    }
    try {
      check(cublasLtCreate(&handle_), "cublasLtCreate");
      check(cublasLtMatmulDescCreate(&op_, compute, scale), "cublasLtMatmulDescCreate");
      const cublasOperation_t op_first = b_col_major ? CUBLAS_OP_T : CUBLAS_OP_N;   // B memory
      const cublasOperation_t op_second = a_col_major ? CUBLAS_OP_T : CUBLAS_OP_N;  // A memory
      check(cublasLtMatmulDescSetAttribute(op_, CUBLASLT_MATMUL_DESC_TRANSA, &op_first, sizeof(op_first)),
            "set TRANSA");
      check(cublasLtMatmulDescSetAttribute(op_, CUBLASLT_MATMUL_DESC_TRANSB, &op_second, sizeof(op_second)),
            "set TRANSB");
      const cudaDataType_t tin = cuda_type(in_type), tout = cuda_type(out_type);
      check(b_col_major ? cublasLtMatrixLayoutCreate(&la_, tin, k, n, ldb)
                        : cublasLtMatrixLayoutCreate(&la_, tin, n, k, ldb), "layout B");
      check(a_col_major ? cublasLtMatrixLayoutCreate(&lb_, tin, m, k, lda)
                        : cublasLtMatrixLayoutCreate(&lb_, tin, k, m, lda), "layout A");
      check(cublasLtMatrixLayoutCreate(&lc_, tout, n, m, ldc), "layout C");
      check(cublasLtMatrixLayoutCreate(&ld_, tout, n, m, ldd), "layout D");
      if (workspace_bytes) {
        if (cudaMalloc(&workspace_, workspace_bytes) != cudaSuccess)
          throw std::runtime_error("cuBLASLt comparator: workspace allocation failed");
        workspace_bytes_ = workspace_bytes;
      }
      check(cublasLtMatmulPreferenceCreate(&pref_), "preference");
      check(cublasLtMatmulPreferenceSetAttribute(pref_, CUBLASLT_MATMUL_PREF_MAX_WORKSPACE_BYTES,
                                                 &workspace_bytes_, sizeof(workspace_bytes_)),
            "preference workspace");
      const cublasStatus_t hs = cublasLtMatmulAlgoGetHeuristic(handle_, op_, la_, lb_, lc_, ld_, pref_, 16,
                                                               results_, &nresults_);
      if (hs != CUBLAS_STATUS_SUCCESS || nresults_ == 0)
        throw std::runtime_error("cuBLASLt comparator: no algorithm for this problem");
    } catch (...) {
      release();
      throw;
    }
  }
  cublaslt_core(const cublaslt_core&) = delete;
  cublaslt_core& operator=(const cublaslt_core&) = delete;
  ~cublaslt_core() { release(); }

  int num_algos() const { return nresults_; }
  // Which of the heuristic's candidates run() uses (0 = the library's first choice).
  bool select(int index) {
    if (index < 0 || index >= nresults_) return false;
    chosen_ = index;
    return true;
  }

  // alpha/beta: host pointers, float (int32 for s8 inputs).  c_mem may be null when beta == 0.
  cublasStatus_t run(const void* a_mem, const void* b_mem, const void* c_mem, void* d_mem,
                     const void* alpha, const void* beta, cudaStream_t stream) {
    const bool no_c = c_mem == nullptr;
    return cublasLtMatmul(handle_, op_, alpha, b_mem, la_, a_mem, lb_, beta, no_c ? d_mem : c_mem,
                          no_c ? ld_ : lc_, d_mem, ld_, &results_[chosen_].algo, workspace_,
                          workspace_bytes_, stream);
  }

 private:
  static cudaDataType_t cuda_type(int dt) {
    switch (dt) {
      case 0: return CUDA_R_16F;
      case 1: return CUDA_R_16BF;
      case 2: return CUDA_R_32F;
      case 3: return CUDA_R_8I;
      case 5: return CUDA_R_8F_E4M3;
      case 6: return CUDA_R_8F_E5M2;
      default: return CUDA_R_32I;
    }
  }
  static void check(cublasStatus_t s, const char* what) {
    if (s != CUBLAS_STATUS_SUCCESS)
      throw std::runtime_error(std::string("cuBLASLt comparator: ") + what + " failed with status " +
                               std::to_string(static_cast<int>(s)));
  }
  void release() {
    if (pref_) cublasLtMatmulPreferenceDestroy(pref_);
    if (la_) cublasLtMatrixLayoutDestroy(la_);
    if (lb_) cublasLtMatrixLayoutDestroy(lb_);
    if (lc_) cublasLtMatrixLayoutDestroy(lc_);
    if (ld_) cublasLtMatrixLayoutDestroy(ld_);
    if (op_) cublasLtMatmulDescDestroy(op_);
    if (handle_) cublasLtDestroy(handle_);
    if (workspace_) cudaFree(workspace_);
    pref_ = nullptr;
    la_ = lb_ = lc_ = ld_ = nullptr;
    op_ = nullptr;
    handle_ = nullptr;
    workspace_ = nullptr;
  }

  cublasLtHandle_t handle_ = nullptr;
  cublasLtMatmulDesc_t op_ = nullptr;
  cublasLtMatrixLayout_t la_ = nullptr, lb_ = nullptr, lc_ = nullptr, ld_ = nullptr;
  cublasLtMatmulPreference_t pref_ = nullptr;
  cublasLtMatmulHeuristicResult_t results_[16];
  int nresults_ = 0;
  int chosen_ = 0;
  void* workspace_ = nullptr;
  std::size_t workspace_bytes_ = 0;
  int in_type_;
};

namespace detail {
template <typename T>
constexpr int lt_dtype_of() {
  if constexpr (std::is_same_v<T, __half>) return 0;
  else if constexpr (std::is_same_v<T, __nv_bfloat16>) return 1;
  else if constexpr (std::is_same_v<T, float>) return 2;
  else if constexpr (std::is_same_v<T, std::int8_t>) return 3;
  else if constexpr (std::is_same_v<T, std::int32_t>) return 4;
  else if constexpr (std::is_same_v<T, __nv_fp8_e4m3>) return 5;
  else if constexpr (std::is_same_v<T, __nv_fp8_e5m2>) return 6;
  else static_assert(sizeof(T) == 0, "unsupported element type");
}
template <typename T>
inline float lt_scalar_to_float(T v) {
  if constexpr (std::is_same_v<T, __half>) return __half2float(v);
  else if constexpr (std::is_same_v<T, __nv_bfloat16>) return __bfloat162float(v);
  else return static_cast<float>(v);
}
}  // namespace detail

// Functor with the reference's constructor and call operator (nvidia/utils/benchmark.cuh:54-57).
template <typename TIn, typename TOut, typename LayoutA = RowMajor, typename LayoutB = RowMajor>
struct cublasLt_gemm {
  static constexpr bool a_col_major = std::is_same_v<LayoutA, ColMajor>;
  static constexpr bool b_col_major = std::is_same_v<LayoutB, ColMajor>;

  cublasLt_gemm(std::size_t m, std::size_t n, std::size_t k, const cudaDeviceProp&)
      : core_(detail::lt_dtype_of<TIn>(), detail::lt_dtype_of<TOut>(), std::is_same_v<LayoutA, ColMajor>,
              std::is_same_v<LayoutB, ColMajor>, static_cast<std::int64_t>(m), static_cast<std::int64_t>(n),
              static_cast<std::int64_t>(k), 0, 0, 0, 0, std::size_t(64) << 20) {}

  void operator()(const TIn* a, const TIn* b, const TOut* c, TOut* d, const TOut alpha, const TOut beta,
                  cudaStream_t stream) {
    cublasStatus_t s;
    if constexpr (std::is_same_v<TIn, std::int8_t>) {
      const std::int32_t al = static_cast<std::int32_t>(alpha), be = static_cast<std::int32_t>(beta);
      s = core_.run(a, b, c, d, &al, &be, stream);
    } else {
      const float al = detail::lt_scalar_to_float(alpha), be = detail::lt_scalar_to_float(beta);
      s = core_.run(a, b, c, d, &al, &be, stream);
    }
    if (s != CUBLAS_STATUS_SUCCESS)
      throw std::runtime_error("cublasLtMatmul failed with status " + std::to_string(static_cast<int>(s)));
  }

  cublaslt_core& core() { return core_; }

 private:
  cublaslt_core core_;
};

}  // namespace nvidia::kernel_functors
#endif
