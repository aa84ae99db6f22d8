#include "kernel_inst.cuh"
GZ_DEFINE_KERNEL_TABLE(kernels_f8_f32, F8, float, false)
