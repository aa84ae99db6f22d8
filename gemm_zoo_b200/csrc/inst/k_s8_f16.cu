#include "kernel_inst.cuh"
GZ_DEFINE_KERNEL_TABLE(kernels_s8_f16, I8, __half, false)
