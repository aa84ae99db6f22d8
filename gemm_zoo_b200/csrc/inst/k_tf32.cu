#include "kernel_inst.cuh"
GZ_DEFINE_KERNEL_TABLE(kernels_tf32, TF32, float, false)
