#include "kernel_inst.cuh"
GZ_DEFINE_KERNEL_TABLE(kernels_s8_bf16, I8, __nv_bfloat16, false)
