#include "kernel_inst.cuh"
GZ_DEFINE_KERNEL_TABLE(kernels_bf16_bf16, F16, __nv_bfloat16, true)
