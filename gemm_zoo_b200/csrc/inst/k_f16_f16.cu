#include "kernel_inst.cuh"
GZ_DEFINE_KERNEL_TABLE(kernels_f16_f16, F16, __half, false)
