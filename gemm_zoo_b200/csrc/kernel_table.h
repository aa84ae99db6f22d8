// Launch table of the tcgen05 GEMM kernel.  Every (operand kind, output type) pair is instantiated
// in a translation unit of its own (csrc/inst/*.cu) so that the library builds in parallel; the
// host layer (gemm_api.cu) sees only these function pointers.
#ifndef GZ_KERNEL_TABLE_H
#define GZ_KERNEL_TABLE_H

#include <cuda.h>
#include <cuda_runtime.h>

#include "gemmzoo/gemm.h"

namespace gz {

struct GemmParams;

using LaunchFn = cudaError_t (*)(const CUtensorMap&, const CUtensorMap&, const CUtensorMap&,
                                 const GemmParams&, int grid, cudaStream_t);
using AttrFn = cudaError_t (*)();

struct KernelEntry {
  LaunchFn launch;
  AttrFn attr;           // opt-in to the kernel's dynamic shared-memory size (once per device)
  LaunchFn launch_prof;  // same kernel with stall counters compiled in (null where not built)
  AttrFn attr_prof;
};

// config: a gz_config naming a tensor-core tile shape.  All-null entry = not instantiated.
KernelEntry kernels_f16_f16(int config);    // fp16 x fp16 -> fp16
KernelEntry kernels_bf16_bf16(int config);  // bf16 x bf16 -> bf16 (stall-counter variants built)
KernelEntry kernels_16_f32(int config);     // fp16 or bf16 -> fp32
KernelEntry kernels_tf32(int config);       // fp32 storage, tf32 multiply -> fp32
KernelEntry kernels_s8_s32(int config);
KernelEntry kernels_s8_f16(int config);
KernelEntry kernels_s8_bf16(int config);
KernelEntry kernels_s8_f32(int config);
KernelEntry kernels_f8_f16(int config);     // e4m3 / e5m2 (the element format is in the instruction descriptor)
KernelEntry kernels_f8_bf16(int config);
KernelEntry kernels_f8_f32(int config);

}  // namespace gz
#endif
