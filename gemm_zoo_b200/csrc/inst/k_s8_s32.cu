#include "kernel_inst.cuh"
GZ_DEFINE_KERNEL_TABLE(kernels_s8_s32, I8, int32_t, false)
