#include "kernel_inst.cuh"
GZ_DEFINE_KERNEL_TABLE(kernels_f8_bf16, F8, __nv_bfloat16, false)
