// Error convention of the harness: print and exit, as the reference's
// checkCudaError does (nvidia/defines.hpp:6-14).  The library underneath never
// exits; it returns gz_status codes, which checkGzStatus turns into exceptions.
#ifndef GZ_NVIDIA_DEFINES_HPP
#define GZ_NVIDIA_DEFINES_HPP

#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <stdexcept>
#include <string>

#include "gemmzoo/gemm.h"

#define checkCudaError(call)                                                                    \
  do {                                                                                          \
    cudaError_t gz_err_ = (call);                                                               \
    if (gz_err_ != cudaSuccess) {                                                               \
      std::printf("CUDA error at %s %d: %s\n", __FILE__, __LINE__, cudaGetErrorString(gz_err_)); \
      std::exit(EXIT_FAILURE);                                                                  \
    }                                                                                           \
  } while (0)

inline void checkGzStatus(gz_status st, const char* where) {
  if (st == GZ_OK) return;
  std::string msg = std::string(where) + ": " + gz_status_string(st);
  if (st == GZ_ERR_CUDA) msg += std::string(" (") + gz_last_cuda_error() + ")";
  throw std::runtime_error(msg);
}

#endif
