// C ABI over the cuBLASLt comparator core (nvidia/kernel_functors/cublaslt_gemm.cuh),
// for the Python test driver and bench.py.  Bench and tests only: the product
// library libgemmzoo.so does not link cuBLAS.
#include <cstdint>
#include <cstdio>
#include <exception>

#include "kernel_functors/cublaslt_gemm.cuh"

#define GZC_API extern "C" __attribute__((visibility("default")))
using nvidia::kernel_functors::cublaslt_core;

// Returns 0 on success, -2 on a library error, -3 if cuBLASLt offers no algorithm.
// *num_algos receives how many candidates the heuristic gave.
GZC_API int gzc_create(void** out, int in_type, int out_type, int a_col_major, int b_col_major,
                       int64_t m, int64_t n, int64_t k, int64_t lda, int64_t ldb, int64_t ldc,
                       int64_t ldd, size_t workspace_bytes, int* num_algos) {
  if (!out) return -1;
  *out = nullptr;
  try {
    cublaslt_core* c = new cublaslt_core(in_type, out_type, a_col_major != 0, b_col_major != 0, m, n, k,
                                         lda, ldb, ldc, ldd, workspace_bytes);
    if (num_algos) *num_algos = c->num_algos();
    *out = c;
    return 0;
  } catch (const std::exception& e) {
    std::fprintf(stderr, "%s\n", e.what());
    return std::string(e.what()).find("no algorithm") != std::string::npos ? -3 : -2;
  }
}

GZC_API int gzc_select(void* h, int index) {
  return (h && static_cast<cublaslt_core*>(h)->select(index)) ? 0 : -1;
}

// alpha/beta: host pointers, float (int32 for s8 inputs).
GZC_API int gzc_run(void* h, const void* a_mem, const void* b_mem, const void* c_mem, void* d_mem,
                    const void* alpha, const void* beta, void* stream) {
  if (!h) return -1;
  const cublasStatus_t s = static_cast<cublaslt_core*>(h)->run(a_mem, b_mem, c_mem, d_mem, alpha, beta,
                                                               static_cast<cudaStream_t>(stream));
  return s == CUBLAS_STATUS_SUCCESS ? 0 : -100 - static_cast<int>(s);
}

GZC_API int gzc_destroy(void* h) {
  delete static_cast<cublaslt_core*>(h);
  return 0;
}
