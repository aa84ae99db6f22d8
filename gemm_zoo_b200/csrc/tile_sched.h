// Tile order of the persistent GEMM kernel, shared by host and device code.
//
// Replaces the Hilbert-curve rasteriser of the reference
// (nvidia/kernels/hilbert.cuh:20-36), which is a bijection only on square
// power-of-two tile grids.  Here tiles are visited in groups of `group_m`
// tile-rows: inside a group the tile-row index runs fastest, then the
// tile-column.  CTAs that run concurrently therefore touch a roughly square
// patch of the output, so the A row-panels and B column-panels they stream are
// shared through L2.  Valid for every tiles_m, tiles_n >= 1.
#ifndef GZ_TILE_SCHED_H
#define GZ_TILE_SCHED_H

#include <stdint.h>

#if defined(__CUDACC__)
#define GZ_HD __host__ __device__ __forceinline__
#else
#define GZ_HD inline
#endif

namespace gz {

struct TileGrid {
  uint32_t tiles_m;
  uint32_t tiles_n;
  uint32_t group_m;    // >= 1
  uint32_t num_tiles;  // tiles_m * tiles_n
};

GZ_HD void tile_coords(const TileGrid& g, uint32_t t, uint32_t& tm, uint32_t& tn) {
  const uint32_t per_group = g.group_m * g.tiles_n;
  const uint32_t grp = t / per_group;
  const uint32_t first_m = grp * g.group_m;
  const uint32_t rem_m = g.tiles_m - first_m;
  const uint32_t rows = rem_m < g.group_m ? rem_m : g.group_m;  // last group may be short
  const uint32_t in = t - grp * per_group;
  tm = first_m + in % rows;
  tn = in / rows;
}

}  // namespace gz
#endif
