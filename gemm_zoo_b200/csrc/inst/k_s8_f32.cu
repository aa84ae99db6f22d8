#include "kernel_inst.cuh"
GZ_DEFINE_KERNEL_TABLE(kernels_s8_f32, I8, float, false)
