// cuBLASLt comparator behind a small C ABI (bench and tests only; the product
// library libgemmzoo.so does not link cuBLAS).
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
#include <cublasLt.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdio>
#include <cstring>
#include <new>

#define GZC_API extern "C" __attribute__((visibility("default")))

namespace {
enum { DT_F16 = 0, DT_BF16 = 1, DT_F32 = 2, DT_S8 = 3, DT_S32 = 4 };

cudaDataType_t cuda_type(int dt) {
  switch (dt) {
    case DT_F16: return CUDA_R_16F;
    case DT_BF16: return CUDA_R_16BF;
    case DT_F32: return CUDA_R_32F;
    case DT_S8: return CUDA_R_8I;
    default: return CUDA_R_32I;
  }
}

struct Cmp {
  cublasLtHandle_t handle = nullptr;
  cublasLtMatmulDesc_t op = nullptr;
  cublasLtMatrixLayout_t la = nullptr, lb = nullptr, lc = nullptr, ld = nullptr;
  cublasLtMatmulPreference_t pref = nullptr;
  cublasLtMatmulHeuristicResult_t results[16];
  int nresults = 0;
  int chosen = 0;
  void* workspace = nullptr;
  size_t workspace_bytes = 0;
  int in_type = 0;
};

void destroy(Cmp* c) {
  if (!c) return;
  if (c->pref) cublasLtMatmulPreferenceDestroy(c->pref);
  if (c->la) cublasLtMatrixLayoutDestroy(c->la);
  if (c->lb) cublasLtMatrixLayoutDestroy(c->lb);
  if (c->lc) cublasLtMatrixLayoutDestroy(c->lc);
  if (c->ld) cublasLtMatrixLayoutDestroy(c->ld);
  if (c->op) cublasLtMatmulDescDestroy(c->op);
  if (c->handle) cublasLtDestroy(c->handle);
  if (c->workspace) cudaFree(c->workspace);
  delete c;
}
}  // namespace

// Returns 0 on success, else a negative code (-1 unsupported, -2 library error,
// -3 no algorithm).  *num_algos receives how many candidates the heuristic gave.
GZC_API int gzc_create(void** out, int in_type, int out_type, int a_col_major, int b_col_major,
                       int64_t m, int64_t n, int64_t k, int64_t lda, int64_t ldb, int64_t ldc,
                       int64_t ldd, size_t workspace_bytes, int* num_algos) {
  if (!out) return -1;
  *out = nullptr;
  Cmp* c = new (std::nothrow) Cmp();
  if (!c) return -2;
  c->in_type = in_type;
  cublasComputeType_t compute;
  cudaDataType_t scale;
  if (in_type == DT_S8) {
    compute = CUBLAS_COMPUTE_32I;
    scale = CUDA_R_32I;
  } else if (in_type == DT_F32) {
    compute = CUBLAS_COMPUTE_32F_FAST_TF32;
    scale = CUDA_R_32F;
  } else {
    compute = CUBLAS_COMPUTE_32F;
    scale = CUDA_R_32F;
  }
#define LT(call)                                                          \
  do {                                                                    \
    cublasStatus_t s_ = (call);                                           \
    if (s_ != CUBLAS_STATUS_SUCCESS) {                                    \
      std::fprintf(stderr, "cublasLt: %s -> %d\n", #call, (int)s_);       \
      destroy(c);                                                         \
      return -2;                                                          \
    }                                                                     \
  } while (0)
  LT(cublasLtCreate(&c->handle));
  LT(cublasLtMatmulDescCreate(&c->op, compute, scale));
  const cublasOperation_t op_first = b_col_major ? CUBLAS_OP_T : CUBLAS_OP_N;   // B memory
  const cublasOperation_t op_second = a_col_major ? CUBLAS_OP_T : CUBLAS_OP_N;  // A memory
  LT(cublasLtMatmulDescSetAttribute(c->op, CUBLASLT_MATMUL_DESC_TRANSA, &op_first, sizeof(op_first)));
  LT(cublasLtMatmulDescSetAttribute(c->op, CUBLASLT_MATMUL_DESC_TRANSB, &op_second, sizeof(op_second)));
  const cudaDataType_t tin = cuda_type(in_type), tout = cuda_type(out_type);
  if (b_col_major) LT(cublasLtMatrixLayoutCreate(&c->la, tin, k, n, ldb));
  else LT(cublasLtMatrixLayoutCreate(&c->la, tin, n, k, ldb));
  if (a_col_major) LT(cublasLtMatrixLayoutCreate(&c->lb, tin, m, k, lda));
  else LT(cublasLtMatrixLayoutCreate(&c->lb, tin, k, m, lda));
  LT(cublasLtMatrixLayoutCreate(&c->lc, tout, n, m, ldc));
  LT(cublasLtMatrixLayoutCreate(&c->ld, tout, n, m, ldd));
  if (workspace_bytes) {
    if (cudaMalloc(&c->workspace, workspace_bytes) != cudaSuccess) {
      destroy(c);
      return -2;
    }
    c->workspace_bytes = workspace_bytes;
  }
  LT(cublasLtMatmulPreferenceCreate(&c->pref));
  LT(cublasLtMatmulPreferenceSetAttribute(c->pref, CUBLASLT_MATMUL_PREF_MAX_WORKSPACE_BYTES,
                                          &c->workspace_bytes, sizeof(c->workspace_bytes)));
  cublasStatus_t hs = cublasLtMatmulAlgoGetHeuristic(c->handle, c->op, c->la, c->lb, c->lc, c->ld,
                                                     c->pref, 16, c->results, &c->nresults);
  if (hs != CUBLAS_STATUS_SUCCESS || c->nresults == 0) {
    destroy(c);
    return -3;
  }
#undef LT
  if (num_algos) *num_algos = c->nresults;
  *out = c;
  return 0;
}

// Choose which of the heuristic's candidates gzc_run uses (0 = the library's first choice).
GZC_API int gzc_select(void* h, int index) {
  Cmp* c = static_cast<Cmp*>(h);
  if (!c || index < 0 || index >= c->nresults) return -1;
  c->chosen = index;
  return 0;
}

// alpha/beta: host pointers, float (int32 for s8 inputs).  c_mem may equal d_mem.
GZC_API int gzc_run(void* h, const void* a_mem, const void* b_mem, const void* c_mem, void* d_mem,
                    const void* alpha, const void* beta, void* stream) {
  Cmp* c = static_cast<Cmp*>(h);
  if (!c) return -1;
  const void* cm = c_mem ? c_mem : d_mem;
  cublasStatus_t s = cublasLtMatmul(c->handle, c->op, alpha, b_mem, c->la, a_mem, c->lb, beta, cm, c->lc,
                                    d_mem, c->ld, &c->results[c->chosen].algo, c->workspace,
                                    c->workspace_bytes, static_cast<cudaStream_t>(stream));
  return s == CUBLAS_STATUS_SUCCESS ? 0 : -2 - (int)s * 100;
}

GZC_API int gzc_destroy(void* h) {
  destroy(static_cast<Cmp*>(h));
  return 0;
}
