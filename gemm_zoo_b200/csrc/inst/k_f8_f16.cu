#include "kernel_inst.cuh"
GZ_DEFINE_KERNEL_TABLE(kernels_f8_f16, F8, __half, false)
