#include "kernel_inst.cuh"
GZ_DEFINE_KERNEL_TABLE(kernels_16_f32, F16, float, false)
