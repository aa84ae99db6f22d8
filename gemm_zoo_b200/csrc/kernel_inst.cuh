// Instantiates sm100_gemm_kernel for every tile shape of one (operand kind, output type) pair and
// returns the launchers.  Included by the one-line translation units in csrc/inst/.
#ifndef GZ_KERNEL_INST_CUH
#define GZ_KERNEL_INST_CUH

#include <cstring>

#include "kernel_table.h"
#include "sm100_gemm.cuh"

namespace gz {
namespace inst {

template <class Cfg, bool PROF = false>
cudaError_t set_attr() {
  return cudaFuncSetAttribute(sm100_gemm_kernel<Cfg, PROF>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                              Cfg::SMEM_BYTES);
}

template <class Cfg, bool PROF = false>
cudaError_t launch(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& td, const GemmParams& p,
                   int grid, cudaStream_t stream) {
  cudaLaunchConfig_t cfg;
  std::memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(grid, 1, 1);
  cfg.blockDim = dim3(Cfg::THREADS, 1, 1);
  cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  unsigned na = 0;
  // Programmatic dependent launch: this grid may be scheduled while the previous kernel of the
  // stream is still running; it sets itself up (barriers, tensor memory, descriptor prefetch) and
  // then waits in the kernel (griddepcontrol.wait) before it touches global memory.
  attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[na].val.programmaticStreamSerializationAllowed = 1;
  ++na;
  if (Cfg::CTAS > 1) {
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = Cfg::CTAS;
    attr[na].val.clusterDim.y = 1;
    attr[na].val.clusterDim.z = 1;
    ++na;
  }
  cfg.attrs = attr;
  cfg.numAttrs = na;
  return cudaLaunchKernelEx(&cfg, sm100_gemm_kernel<Cfg, PROF>, ta, tb, td, p);
}

template <class C, bool WITH_PROF>
KernelEntry make_entry() {
  if constexpr (WITH_PROF) return {launch<C>, set_attr<C>, launch<C, true>, set_attr<C, true>};
  else return {launch<C>, set_attr<C>, nullptr, nullptr};
}

// Tile shapes: (columns, CTAs per tile, pipeline stages[, swapped operands[, row blocks per CTA]]).
// Stall counters (WITH_PROF) are compiled for one tile of each family.
template <ptx::Kind KIND, typename TOut, bool WITH_PROF = false>
KernelEntry entry_for_shape(int config) {
  switch (config) {
    case GZ_CFG_2CTA_N256: return make_entry<GemmCfg<KIND, TOut, 256, 2, 6>, WITH_PROF>();
    case GZ_CFG_1CTA_N256: return make_entry<GemmCfg<KIND, TOut, 256, 1, 4>, false>();
    case GZ_CFG_2CTA_N128: return make_entry<GemmCfg<KIND, TOut, 128, 2, 8>, false>();
    case GZ_CFG_1CTA_N128: return make_entry<GemmCfg<KIND, TOut, 128, 1, 6>, false>();
    case GZ_CFG_1CTA_N64: return make_entry<GemmCfg<KIND, TOut, 64, 1, 8>, WITH_PROF>();
    case GZ_CFG_SWAP_M16: return make_entry<GemmCfg<KIND, TOut, 16, 1, 12, true>, WITH_PROF>();
    case GZ_CFG_SWAP_M32: return make_entry<GemmCfg<KIND, TOut, 32, 1, 11, true>, false>();
    case GZ_CFG_SWAP_M64: return make_entry<GemmCfg<KIND, TOut, 64, 1, 9, true>, false>();
    case GZ_CFG_SWAP_M128: return make_entry<GemmCfg<KIND, TOut, 128, 1, 6, true>, false>();
    case GZ_CFG_2CTA_M512_N256: return make_entry<GemmCfg<KIND, TOut, 256, 2, 4, false, 2>, WITH_PROF>();
  }
  return {nullptr, nullptr, nullptr, nullptr};
}

}  // namespace inst
}  // namespace gz

#define GZ_DEFINE_KERNEL_TABLE(NAME, KIND, TOUT, WITH_PROF) \
  gz::KernelEntry gz::NAME(int config) { return gz::inst::entry_for_shape<gz::ptx::Kind::KIND, TOUT, WITH_PROF>(config); }

#endif
