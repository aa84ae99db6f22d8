// C ABI of the library (see include/gemmzoo/gemm.h): descriptor validation,
// plan creation (configuration choice, shared-memory opt-in, launch geometry),
// per-call tensor-map encoding and launch, host-operand convenience path,
// device status read-back, seeded fills and the column partition helper.
//
// The plan does what the constructor of a reference functor does
// (nvidia/kernel_functors/bf16_mma_gemm.cuh:17-49) and gz_gemm_run does what its
// operator() does (:51-63): one asynchronous launch, no host synchronisation.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <atomic>
#include <mutex>
#include <new>
#include <string>
#include <vector>

#include "gemmzoo/gemm.h"
#include "kernel_table.h"
#include "placement.cuh"
#include "rng.h"
#include "simt_gemm.cuh"
#include "sm100_gemm.cuh"
#include "tile_sched.h"

namespace {

thread_local std::string g_last_cuda_error;

bool cuda_ok(cudaError_t e, const char* what) {
  if (e == cudaSuccess) return true;
  g_last_cuda_error = std::string(what) + ": " + cudaGetErrorString(e);
  (void)cudaGetLastError();
  return false;
}

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) ==
            cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
    (void)cudaGetLastError();
  });
  return fn;
}

// Makes `device` current for the calling thread and puts the previous device back on scope exit:
// no entry point of the library leaves the caller's current device changed.
class DeviceGuard {
 public:
  explicit DeviceGuard(int device) {
    ok_ = cudaGetDevice(&prev_) == cudaSuccess;
    if (ok_ && prev_ != device) {
      ok_ = cuda_ok(cudaSetDevice(device), "cudaSetDevice");
      changed_ = ok_;
    }
  }
  ~DeviceGuard() {
    if (changed_) (void)cudaSetDevice(prev_);
  }
  DeviceGuard(const DeviceGuard&) = delete;
  DeviceGuard& operator=(const DeviceGuard&) = delete;
  bool ok() const { return ok_; }

 private:
  int prev_ = 0;
  bool ok_ = false, changed_ = false;
};

int dtype_size(int dt) {
  switch (dt) {
    case GZ_DT_F16:
    case GZ_DT_BF16: return 2;
    case GZ_DT_F32:
    case GZ_DT_S32: return 4;
    case GZ_DT_S8:
    case GZ_DT_E4M3:
    case GZ_DT_E5M2: return 1;
  }
  return 0;
}

bool is_fp8(int dt) { return dt == GZ_DT_E4M3 || dt == GZ_DT_E5M2; }

bool pair_supported(int in, int out) {
  return (in == GZ_DT_F16 && (out == GZ_DT_F16 || out == GZ_DT_F32)) ||
         (in == GZ_DT_BF16 && (out == GZ_DT_BF16 || out == GZ_DT_F32)) ||
         (in == GZ_DT_F32 && out == GZ_DT_F32) || (in == GZ_DT_S8 && out == GZ_DT_S32) ||
         // int32 accumulation, float epilogue (dequantising GEMM)
         (in == GZ_DT_S8 && (out == GZ_DT_F16 || out == GZ_DT_BF16 || out == GZ_DT_F32)) ||
         (is_fp8(in) && (out == GZ_DT_F16 || out == GZ_DT_BF16 || out == GZ_DT_F32));
}

struct CfgShape {
  int config, ctas, bn, stages;
  bool swap;  // operand roles exchanged: the 128-row side walks N, the bn side walks M
  int mb;     // 128-row blocks of the wide operand per CTA
  int tile_wide() const { return 128 * ctas * mb; }  // tile extent along the 128-row side
};
const CfgShape kShapes[] = {
    {GZ_CFG_2CTA_N256, 2, 256, 6, false, 1}, {GZ_CFG_1CTA_N256, 1, 256, 4, false, 1},
    {GZ_CFG_2CTA_N128, 2, 128, 8, false, 1}, {GZ_CFG_1CTA_N128, 1, 128, 6, false, 1},
    {GZ_CFG_1CTA_N64, 1, 64, 8, false, 1},   {GZ_CFG_SWAP_M16, 1, 16, 12, true, 1},
    {GZ_CFG_SWAP_M32, 1, 32, 11, true, 1},   {GZ_CFG_SWAP_M64, 1, 64, 9, true, 1},
    {GZ_CFG_SWAP_M128, 1, 128, 6, true, 1},  {GZ_CFG_2CTA_M512_N256, 2, 256, 4, false, 2},
};
const CfgShape* shape_of(int config) {
  for (const auto& s : kShapes)
    if (s.config == config) return &s;
  return nullptr;
}

int64_t cdiv(int64_t a, int64_t b) { return (a + b - 1) / b; }

// Normalised view of a descriptor.
struct Problem {
  gz_gemm_desc d;
  int in_size, out_size;
  bool a_mn_major, b_mn_major;  // A column-major / B row-major
  bool tma_ld_ok;               // leading dimensions satisfy TMA's 16-byte stride rule
};

gz_status normalise(const gz_gemm_desc* desc, Problem* pr) {
  if (!desc) return GZ_ERR_INVALID_ARG;
  if (desc->struct_size != sizeof(gz_gemm_desc)) return GZ_ERR_INVALID_ARG;
  gz_gemm_desc d = *desc;
  if (d.m <= 0 || d.n <= 0 || d.k <= 0) return GZ_ERR_INVALID_ARG;
  if (d.layout_a != GZ_ROW_MAJOR && d.layout_a != GZ_COL_MAJOR) return GZ_ERR_INVALID_ARG;
  if (d.layout_b != GZ_ROW_MAJOR && d.layout_b != GZ_COL_MAJOR) return GZ_ERR_INVALID_ARG;
  if (dtype_size(d.in_type) == 0 || dtype_size(d.out_type) == 0) return GZ_ERR_INVALID_ARG;
  if (d.device < 0) return GZ_ERR_INVALID_ARG;
  if ((d.flags & GZ_FLAG_EPILOGUE_DIRECT) && (d.flags & GZ_FLAG_EPILOGUE_TMA))
    return GZ_ERR_INVALID_ARG;
  if ((d.flags & GZ_FLAG_NO_SPLIT_K) && (d.flags & GZ_FLAG_SPLIT_K)) return GZ_ERR_INVALID_ARG;
  if (d.flags & ~(GZ_FLAG_EPILOGUE_DIRECT | GZ_FLAG_EPILOGUE_TMA | GZ_FLAG_NO_SPLIT_K | GZ_FLAG_SPLIT_K |
                  GZ_FLAG_BROADCAST_A | GZ_FLAG_BROADCAST_B | GZ_FLAG_NO_DIE_ORDER | GZ_FLAG_TEST_WITHHOLD_ACC_READY))
    return GZ_ERR_INVALID_ARG;
  if (d.batch == 0) d.batch = 1;
  if (d.batch < 0 || d.batch > 65535 || d.stride_a < 0 || d.stride_b < 0 || d.stride_c < 0 || d.stride_d < 0)
    return GZ_ERR_INVALID_ARG;
  if (!pair_supported(d.in_type, d.out_type)) return GZ_ERR_UNSUPPORTED;
  if (d.config != GZ_CFG_AUTO && d.config != GZ_CFG_SIMT && !shape_of(d.config))
    return GZ_ERR_INVALID_ARG;
  const int64_t min_lda = d.layout_a == GZ_ROW_MAJOR ? d.k : d.m;
  const int64_t min_ldb = d.layout_b == GZ_ROW_MAJOR ? d.n : d.k;
  if (d.lda == 0) d.lda = min_lda;
  if (d.ldb == 0) d.ldb = min_ldb;
  if (d.ldc == 0) d.ldc = d.n;
  if (d.ldd == 0) d.ldd = d.n;
  if (d.lda < min_lda || d.ldb < min_ldb || d.ldc < d.n || d.ldd < d.n) return GZ_ERR_INVALID_ARG;
  // Tile coordinates and TMA coordinates are 32-bit.
  const int64_t lim = (int64_t(1) << 31) - 1024;
  if (d.m > lim || d.n > lim || d.k > lim) return GZ_ERR_TOO_LARGE;
  // at most 2^49 tiles of the smallest shape per problem, so the product with the batch (< 2^16)
  // is taken in two steps
  const int64_t tiles_min = cdiv(d.m, 128) * cdiv(d.n, 64);
  if (tiles_min > (int64_t(1) << 31) - 1 || tiles_min * d.batch > (int64_t(1) << 31) - 1) return GZ_ERR_TOO_LARGE;
  // A matrix must be addressable: rows x leading dimension (and that times the batch) within 2^60 elements.
  const int64_t addr_lim = int64_t(1) << 60;
  auto span = [&](int64_t rows, int64_t ld, int64_t* out) {
    return !__builtin_mul_overflow(rows, ld, out) && *out <= addr_lim / d.batch;
  };
  int64_t span_a, span_b, span_c, span_d;
  if (!span(d.layout_a == GZ_ROW_MAJOR ? d.m : d.k, d.lda, &span_a) ||
      !span(d.layout_b == GZ_ROW_MAJOR ? d.k : d.n, d.ldb, &span_b) || !span(d.m, d.ldc, &span_c) ||
      !span(d.m, d.ldd, &span_d) || d.stride_a > addr_lim / d.batch || d.stride_b > addr_lim / d.batch ||
      d.stride_c > addr_lim / d.batch || d.stride_d > addr_lim / d.batch)
    return GZ_ERR_TOO_LARGE;
  // Batch strides: packed by default; a broadcast operand has none.
  if (d.stride_a == 0) d.stride_a = span_a;
  if (d.stride_b == 0) d.stride_b = span_b;
  if (d.stride_c == 0) d.stride_c = span_c;
  if (d.stride_d == 0) d.stride_d = span_d;
  if (d.flags & GZ_FLAG_BROADCAST_A) d.stride_a = 0;
  if (d.flags & GZ_FLAG_BROADCAST_B) d.stride_b = 0;
  if (d.wait_limit_ns == 0) d.wait_limit_ns = 2000000000ull;
  pr->d = d;
  pr->in_size = dtype_size(d.in_type);
  pr->out_size = dtype_size(d.out_type);
  pr->a_mn_major = d.layout_a == GZ_COL_MAJOR;
  pr->b_mn_major = d.layout_b == GZ_ROW_MAJOR;
  pr->tma_ld_ok = (d.lda * pr->in_size) % 16 == 0 && (d.ldb * pr->in_size) % 16 == 0 &&
                  (d.lda * (int64_t)pr->in_size) < (int64_t(1) << 40) &&
                  (d.ldb * (int64_t)pr->in_size) < (int64_t(1) << 40) &&
                  // the batch dimension of a tensor map is a stride like any other
                  (d.batch == 1 || ((d.stride_a * pr->in_size) % 16 == 0 && (d.stride_b * pr->in_size) % 16 == 0 &&
                                    (d.stride_a * (int64_t)pr->in_size) < (int64_t(1) << 40) &&
                                    (d.stride_b * (int64_t)pr->in_size) < (int64_t(1) << 40)));
  return GZ_OK;
}

// An M/N-contiguous operand is fetched in 128-byte chunks of its tile edge, so the
// edge (in elements) must hold at least one chunk: 128 for s8, 64 for 16-bit, 32 for fp32.
bool shape_fits(const Problem& pr, const CfgShape& s) {
  const int chunk = 128 / pr.in_size;
  // Which matrix rides the 128-row side and which the bn side of the MMA.
  const bool wide_mn_major = s.swap ? pr.b_mn_major : pr.a_mn_major;
  const bool narrow_mn_major = s.swap ? pr.a_mn_major : pr.b_mn_major;
  if (narrow_mn_major && (s.bn / s.ctas) % chunk != 0) return false;
  if (wide_mn_major && 128 % chunk != 0) return false;
  if (s.swap && pr.d.m > s.bn) return false;  // swapped tiles cover all of M with one tile
  return true;
}

// Split-K is implemented by the swapped (skinny) tiles only.  It pays when whole tiles would
// occupy at most half of the SMs (with more than that streaming, HBM is already saturated) and
// there are enough K blocks to share out (each CTA gets at least four).
bool wants_split_k(const Problem& pr, const CfgShape& s, int sm_count) {
  if (!s.swap || (pr.d.flags & GZ_FLAG_NO_SPLIT_K)) return false;
  const int64_t k_blocks = cdiv(pr.d.k, 128 / pr.in_size);
  const int64_t tiles = cdiv(pr.d.n, 128) * cdiv(pr.d.m, s.bn) * pr.d.batch;
  const int64_t total = tiles * k_blocks;
  if (total < 2) return false;
  if (pr.d.flags & GZ_FLAG_SPLIT_K) return true;
  // Wide partial tiles are costly to park and add up; left to the caller's explicit request.
  return s.bn <= 64 && tiles * 2 <= sm_count && total >= 16;
}

// Tail splitting for whole-tile schedules: if the last wave would fill at most half (a quarter) of
// the SMs, its tiles are cut into 2 (4) column strips so that the wave is short instead of sparse.
// Returns the number of strips per tail tile (1 = none) and sets *first to the first tail tile.
int tail_parts_for(const Problem& pr, const CfgShape& s, int64_t tiles, int64_t units, int64_t* first) {
  *first = tiles;
  if (s.swap || units <= 0 || tiles <= units) return 1;  // a single (partial) wave is not split
  const int64_t rem = tiles % units;
  if (rem == 0) return 1;
  const int chunk = 128 / pr.in_size;
  int parts = 1;
  for (int f = 2; f <= 4; f *= 2) {
    const int strip = s.bn / f;                      // columns per strip
    if (strip < 64 || rem * f > units) break;
    if (pr.b_mn_major && (strip / s.ctas) % chunk != 0) break;  // N-contiguous B is fetched in 128-byte chunks
    if ((strip / s.ctas) % 8 != 0) break;
    // with eight epilogue warps each stores whole 128-byte boxes of its half of the strip
    if (s.bn >= 128 && (strip / 2) % (128 / pr.out_size) != 0) break;
    parts = f;
  }
  if (parts > 1) *first = tiles - rem;
  return parts;
}

// CTAs a split-K launch uses: each gets at least four K blocks, and a tile is shared by few enough
// CTAs that the partial sums its finisher must add stay around 256 KB.
int64_t split_k_grid(const CfgShape& s, int64_t tiles, int64_t k_blocks, int64_t units) {
  const int64_t total = tiles * k_blocks;
  const int64_t slot_bytes = (int64_t)s.bn * 128 * 4;
  int64_t share = (256 * 1024) / slot_bytes;  // CTAs per tile
  if (share < 2) share = 2;
  int64_t grid = cdiv(total, 4);
  if (grid > tiles * share) grid = tiles * share;
  if (grid > units) grid = units;
  if (grid < 1) grid = 1;
  return grid;
}

// Pick the tile shape with the least estimated time.  Per 128-byte K block a CTA is held up by
// the slowest of: the MMAs (a 128 x bn x 32-byte MMA takes bn/2 cycles, four per block), the
// L2 -> shared-memory fill of its stage (about 64 bytes per cycle per SM), and the issue cost of
// the block (about 250 cycles).  On top of that, every byte moved costs power, and a large GEMM
// runs at the part's power limit, where power is paid for in clock frequency: 35 % of the fill
// time is added for it (fitted to measurements of the 256- and 512-row tiles at 8192^3 and
// 16384^3).  Tiles with two row blocks per CTA expose part of their epilogue once per tile.
// Whole tiles are dealt to the SMs in waves; with split-K the K blocks of all tiles are spread
// evenly.
int choose_config(const Problem& pr, int sm_count) {
  if (!pr.tma_ld_ok) return GZ_CFG_SIMT;
  double best = 0;
  int best_cfg = GZ_CFG_SIMT;
  const int64_t k_blocks = cdiv(pr.d.k, 128 / pr.in_size);
  for (const auto& s : kShapes) {
    if (!shape_fits(pr, s)) continue;
    const int64_t wide = s.swap ? pr.d.n : pr.d.m, narrow = s.swap ? pr.d.m : pr.d.n;
    const int64_t tiles = cdiv(wide, s.tile_wide()) * cdiv(narrow, s.bn) * pr.d.batch;
    const int64_t units = sm_count / s.ctas;
    if (units <= 0) continue;
    const double mma = 4.0 * (s.bn / 2.0) * s.mb;
    const double fill = (128.0 * s.mb + double(s.bn) / s.ctas) * 128.0 / 64.0;
    const double issue = 250.0;
    double per_block = mma > fill ? mma : fill;
    if (issue > per_block) per_block = issue;
    per_block += 0.35 * fill;
    // Clocks per tile during which the tensor pipe waits for the epilogue: only the accumulator
    // hand-over when a warp's share of both accumulators fits its registers (16-bit outputs),
    // most of the output stores otherwise.
    const double per_tile = s.mb == 2 ? (pr.out_size == 2 ? 3500.0 : 6000.0) : 0.0;
    double blocks_per_cta;
    if (wants_split_k(pr, s, sm_count)) {
      const int64_t total = tiles * k_blocks;
      const int64_t ctas = split_k_grid(s, tiles, k_blocks, units);
      // plus parking one partial tile and, for the finisher, adding the others (64 bytes per cycle)
      const double share = double(ctas) / double(tiles) + 1.0;
      blocks_per_cta = double(cdiv(total, ctas)) + share * (s.bn * 128.0 * 4.0 / 64.0) / per_block;
    } else {
      int64_t first;
      const int parts = tail_parts_for(pr, s, tiles, units, &first);
      const double waves = parts > 1 ? double(first / units) + 1.0 / parts : double(cdiv(tiles, units));
      blocks_per_cta = waves * (double(k_blocks) + per_tile / per_block);
    }
    // Once per CTA: set-up and teardown (a CTA pair also synchronises as a cluster and allocates
    // tensor memory jointly) and the last tile's epilogue, which nothing hides.  These decide
    // between shapes when a CTA has only a handful of K blocks to do; the pair's figure is fitted
    // to short-K problems (1024 x 4096 x 1024, 1536^3), where one-CTA tiles measure 3-5 % faster.
    const double fixed = (s.ctas == 2 ? 7000.0 : 800.0) + 1500.0 + 8.0 * s.bn;
    const double cost = blocks_per_cta * per_block + fixed;
    if (best == 0 || cost < best) {
      best = cost;
      best_cfg = s.config;
    }
  }
  return best_cfg;
}

void fill_info(const Problem& pr, int config, int sm_count, gz_plan_info* info) {
  std::memset(info, 0, sizeof(*info));
  info->config = config;
  info->sm_count = sm_count;
  info->lda = pr.d.lda;
  info->ldb = pr.d.ldb;
  info->ldc = pr.d.ldc;
  info->ldd = pr.d.ldd;
  if (config == GZ_CFG_SIMT) {
    info->tile_m = 64;
    info->tile_n = 64;
    info->tile_k = 16;
    info->stages = 1;
    info->ctas_per_tile = 1;
    info->tiles = cdiv(pr.d.m, 64) * cdiv(pr.d.n, 64) * pr.d.batch;
    info->grid = (int32_t)info->tiles;
    info->smem_bytes = 0;
    return;
  }
  const CfgShape* s = shape_of(config);
  info->tile_m = s->swap ? s->bn : s->tile_wide();
  info->tile_n = s->swap ? 128 : s->bn;
  info->tile_k = 128 / pr.in_size;
  info->stages = s->stages;
  info->ctas_per_tile = s->ctas;
  info->tiles = cdiv(pr.d.m, info->tile_m) * cdiv(pr.d.n, info->tile_n) * pr.d.batch;
  const int64_t units = sm_count / s->ctas;
  info->grid = (int32_t)((info->tiles < units ? info->tiles : units) * s->ctas);
  // Mirrors GemmCfg::SMEM_BYTES: alignment slack, the operand ring, epilogue staging, barriers.
  const int staging = s->swap ? 0 : (s->bn >= 128 ? 8 : 4) * 4096;
  info->smem_bytes = 1024 + s->stages * (128 * s->mb * 128 + (s->bn / s->ctas) * 128) + staging + 256;
  // Output rows go through shared memory and TMA stores when D's row pitch allows it; the swapped
  // (skinny) tiles hold the transposed tile and always store straight from registers.
  const bool d_tma_ok = (pr.d.ldd * pr.out_size) % 16 == 0 &&
                        (pr.d.batch == 1 || ((pr.d.stride_d * pr.out_size) % 16 == 0 &&
                                             pr.d.stride_d * (int64_t)pr.out_size < (int64_t(1) << 40)));
  info->epilogue_tma = (!s->swap && d_tma_ok && !(pr.d.flags & GZ_FLAG_EPILOGUE_DIRECT)) ? 1 : 0;
  if (wants_split_k(pr, *s, sm_count)) {
    const int64_t k_blocks = cdiv(pr.d.k, info->tile_k);
    const int64_t total = info->tiles * k_blocks;
    const int64_t grid = split_k_grid(*s, info->tiles, k_blocks, units);
    const int64_t shortest = total / grid;  // K blocks in the shortest range
    const int64_t contrib = (k_blocks - 1) / shortest + 2;
    info->split_k = 1;
    info->grid = (int32_t)grid;
    info->workspace_bytes = info->tiles * contrib * (int64_t)s->bn * 128 * 4 + info->tiles * 4;
    info->reserved = (int32_t)contrib;
  }
}

using gz::KernelEntry;
using gz::LaunchFn;

// The kernels themselves are instantiated in csrc/inst/*.cu, one translation unit per pair of types.
KernelEntry entry_for(int in, int out, int config) {
  if (in == GZ_DT_F16 && out == GZ_DT_F16) return gz::kernels_f16_f16(config);
  if (in == GZ_DT_BF16 && out == GZ_DT_BF16) return gz::kernels_bf16_bf16(config);
  if ((in == GZ_DT_F16 || in == GZ_DT_BF16) && out == GZ_DT_F32) return gz::kernels_16_f32(config);
  if (in == GZ_DT_F32) return gz::kernels_tf32(config);
  if (in == GZ_DT_S8 && out == GZ_DT_S32) return gz::kernels_s8_s32(config);
  if (in == GZ_DT_S8 && out == GZ_DT_F16) return gz::kernels_s8_f16(config);
  if (in == GZ_DT_S8 && out == GZ_DT_BF16) return gz::kernels_s8_bf16(config);
  if (in == GZ_DT_S8 && out == GZ_DT_F32) return gz::kernels_s8_f32(config);
  if (is_fp8(in) && out == GZ_DT_F16) return gz::kernels_f8_f16(config);
  if (is_fp8(in) && out == GZ_DT_BF16) return gz::kernels_f8_bf16(config);
  if (is_fp8(in) && out == GZ_DT_F32) return gz::kernels_f8_f32(config);
  return {nullptr, nullptr, nullptr, nullptr};
}

template <typename TIn, typename TOut>
cudaError_t launch_simt(const gz::SimtParams& sp, cudaStream_t stream) {
  dim3 grid((unsigned)cdiv(sp.n, 64), (unsigned)cdiv(sp.m, 64), (unsigned)(sp.batch > 0 ? sp.batch : 1));
  gz::simt_gemm_kernel<TIn, TOut><<<grid, 256, 0, stream>>>(sp);
  return cudaGetLastError();
}

cudaError_t launch_simt_any(int in, int out, const gz::SimtParams& sp, cudaStream_t stream) {
  if (in == GZ_DT_F16 && out == GZ_DT_F16) return launch_simt<__half, __half>(sp, stream);
  if (in == GZ_DT_F16 && out == GZ_DT_F32) return launch_simt<__half, float>(sp, stream);
  if (in == GZ_DT_BF16 && out == GZ_DT_BF16)
    return launch_simt<__nv_bfloat16, __nv_bfloat16>(sp, stream);
  if (in == GZ_DT_BF16 && out == GZ_DT_F32) return launch_simt<__nv_bfloat16, float>(sp, stream);
  if (in == GZ_DT_F32) return launch_simt<float, float>(sp, stream);
  if (in == GZ_DT_S8 && out == GZ_DT_S32) return launch_simt<int8_t, int32_t>(sp, stream);
  if (in == GZ_DT_S8 && out == GZ_DT_F16) return launch_simt<int8_t, __half>(sp, stream);
  if (in == GZ_DT_S8 && out == GZ_DT_BF16) return launch_simt<int8_t, __nv_bfloat16>(sp, stream);
  if (in == GZ_DT_S8 && out == GZ_DT_F32) return launch_simt<int8_t, float>(sp, stream);
  if (in == GZ_DT_E4M3 && out == GZ_DT_F16) return launch_simt<__nv_fp8_e4m3, __half>(sp, stream);
  if (in == GZ_DT_E4M3 && out == GZ_DT_BF16) return launch_simt<__nv_fp8_e4m3, __nv_bfloat16>(sp, stream);
  if (in == GZ_DT_E4M3 && out == GZ_DT_F32) return launch_simt<__nv_fp8_e4m3, float>(sp, stream);
  if (in == GZ_DT_E5M2 && out == GZ_DT_F16) return launch_simt<__nv_fp8_e5m2, __half>(sp, stream);
  if (in == GZ_DT_E5M2 && out == GZ_DT_BF16) return launch_simt<__nv_fp8_e5m2, __nv_bfloat16>(sp, stream);
  if (in == GZ_DT_E5M2 && out == GZ_DT_F32) return launch_simt<__nv_fp8_e5m2, float>(sp, stream);
  return cudaErrorInvalidValue;
}

CUtensorMapDataType tmap_type(int dt) {
  switch (dt) {
    case GZ_DT_F16: return CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    case GZ_DT_BF16: return CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    case GZ_DT_F32: return CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
    case GZ_DT_S32: return CU_TENSOR_MAP_DATA_TYPE_INT32;
    default: return CU_TENSOR_MAP_DATA_TYPE_UINT8;
  }
}

// Tensor map of a batch of matrices: dim0 (contiguous) x dim1 with row pitch `pitch_bytes`, times
// `batch` matrices `batch_stride_bytes` apart (a single matrix is a batch of one), 128-byte
// swizzle, boxes of box0 x box1 x 1.
bool encode_2d(CUtensorMap* tm, int dt, const void* base, uint64_t dim0, uint64_t dim1,
               uint64_t pitch_bytes, uint32_t box0, uint32_t box1, bool promote,
               bool swizzle_32b_atom = false, uint64_t batch = 1, uint64_t batch_stride_bytes = 0) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) {
    g_last_cuda_error = "cuTensorMapEncodeTiled entry point not available";
    return false;
  }
  if (batch <= 1 || batch_stride_bytes == 0) {  // one matrix (or one shared by the whole batch)
    batch = 1;
    batch_stride_bytes = pitch_bytes * dim1;
  }
  cuuint64_t dims[3] = {dim0, dim1, batch};
  cuuint64_t strides[2] = {pitch_bytes, batch_stride_bytes};
  cuuint32_t box[3] = {box0, box1, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(tm, tmap_type(dt), 3, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle_32b_atom ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                  promote ? CU_TENSOR_MAP_L2_PROMOTION_L2_256B : CU_TENSOR_MAP_L2_PROMOTION_NONE,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    char buf[96];
    std::snprintf(buf, sizeof(buf), "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    g_last_cuda_error = buf;
    return false;
  }
  return true;
}

// Placement of each device, measured at most once per process (see placement.cuh).
gz::DevicePlacement g_placement[64];
bool g_placement_done[64] = {};
std::mutex g_placement_mu;

const gz::DevicePlacement* placement_of(int device, int sm_count) {
  if (device < 0 || device >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(g_placement_mu);
  if (!g_placement_done[device]) {
    // The device is current (plan creation).  The probe times L2 hits, so a measurement taken while
    // the clocks ramp up from idle can be too noisy to classify: try a few times before giving up
    // (giving up only switches the die-aware order off).
    for (int attempt = 0; attempt < 4; ++attempt) {
      g_placement[device] = gz::measure_placement(sm_count);
      if (g_placement[device].known) break;
    }
    g_placement_done[device] = true;
  }
  return &g_placement[device];
}

// The die-aware order pays where a launch fills the whole machine for several waves of tiles: then
// what the two dies read in a wave is large against the L2, and keeping their tiles apart saves
// die-to-die traffic.  Skinny (swapped) problems stream their weight matrix once and gain nothing.
bool wants_die_order(const Problem& pr, const CfgShape& s, int sm_count, int64_t all_tiles) {
  if (s.swap || (pr.d.flags & GZ_FLAG_NO_DIE_ORDER)) return false;
  const int64_t units = sm_count / s.ctas;
  return units * s.ctas == sm_count && all_tiles >= 3 * units;
}

}  // namespace

// Encoded tensor maps of one set of operand pointers.  A tensor map embeds the base address, and
// callers such as the reference's harness rotate their operand buffers every call
// (nvidia/utils/benchmark.cuh:80-83), so a plan keeps the last few sets instead of encoding three
// maps per launch.  Extents, strides and boxes are constants of the plan.
struct TensorMapSet {
  const void* a = nullptr;
  const void* b = nullptr;
  const void* d = nullptr;  // null when the launch does not store through TMA
  uint64_t stamp = 0;       // 0 = empty; otherwise the plan's clock at the last use
  CUtensorMap ta, tb, td;
};

struct gz_plan {
  Problem pr;
  gz_plan_info info;
  KernelEntry entry;
  gz::GemmParams base;  // everything that does not depend on the operand pointers
  // Die-aware tile order: ticket counters, one set of four words per launch in flight (see
  // GemmParams::die_tickets); launches take the sets in turn.
  static constexpr int kDieTicketSets = 32;
  uint32_t* die_tickets = nullptr;
  std::atomic<uint32_t> launch_seq{0};
  static constexpr int kTensorMapSets = 8;
  TensorMapSet tmaps[kTensorMapSets];
  uint64_t tmap_clock = 0;
  std::mutex tmap_mu;
  uint32_t* status_dev;
  void* workspace;  // split-K partial sums followed by the per-tile arrival counters
  // device staging for gz_gemm_run_host
  void *ha, *hb, *hc, *hd;
  size_t ha_bytes, hb_bytes, hcd_bytes;
  // gz_gemm_run_host pipeline: column blocks of B/C/D travel on two copy streams while the
  // caller's stream computes (PCIe is full duplex, so uploads, GEMMs and downloads overlap).
  static constexpr int kMaxBlocks = 16;
  cudaStream_t copy_in = nullptr, copy_out = nullptr;
  cudaEvent_t ev_start = nullptr, ev_out = nullptr;
  cudaEvent_t ev_in[kMaxBlocks] = {}, ev_gemm[kMaxBlocks] = {};
  gz_plan* block_plan = nullptr;  // plan for one full column block
  gz_plan* tail_plan = nullptr;   // plan for the last, narrower block (if any)
  int64_t block_cols = 0;
  int blocks = 0;
  bool pipe_ready = false;
  std::mutex mu;
};

namespace {

void build_operand(gz::OperandDesc* od, bool mn_major, int rows, int in_size) {
  const int bk = 128 / in_size;  // K elements per 128 bytes
  od->mn_major = mn_major ? 1u : 0u;
  const uint32_t sbo = 1024u >> 4;  // 8 rows of 128 bytes between core-matrix groups
  if (!mn_major) {
    // K contiguous: one box of `rows` x 128 bytes; a K step moves 32 bytes inside the swizzle atom.
    od->boxes = 1;
    od->box_mn = rows;
    od->box_bytes = rows * 128;
    od->desc_lo = 1u << 16;  // leading byte offset is unused for swizzled K-major operands
    od->k_step16 = 32u >> 4;
  } else {
    // M/N contiguous: boxes of (128 bytes of M/N) x (bk rows of K), one per 128-byte chunk of the
    // tile edge; an MMA K step moves whole 8-row groups.
    const int mn_per_box = 128 / in_size;
    od->boxes = rows / mn_per_box;
    od->box_mn = mn_per_box;
    od->box_bytes = bk * 128;
    od->desc_lo = ((od->box_bytes >> 4) & 0x3FFFu) << 16;  // distance between M/N chunks
    const int umma_k = 32 / in_size;
    od->k_step16 = (uint32_t)(umma_k * 128) >> 4;
    if (in_size == 4) {
      // 32-bit elements with M/N contiguous exist only in the "128-byte swizzle,
      // 32-byte atom" layout: 32-byte chunks are permuted over groups of 4 K-rows
      // (TMA: SWIZZLE_128B_ATOM_32B), and the descriptor strides over 4-row groups.
      od->desc_hi = (512u >> 4) | (1u << 14) | (1u << 29);
      return;
    }
  }
  od->desc_hi = sbo | (1u << 14) /* descriptor version for sm_100 */ | (2u << 29) /* 128B swizzle */;
}

uint32_t build_idesc(const Problem& pr, const CfgShape& s) {
  uint32_t fmt_ab, fmt_c;
  switch (pr.d.in_type) {
    case GZ_DT_F16: fmt_ab = 0; fmt_c = 1; break;
    case GZ_DT_BF16: fmt_ab = 1; fmt_c = 1; break;
    case GZ_DT_F32: fmt_ab = 2; fmt_c = 1; break;  // tf32 operands, f32 accumulate
    case GZ_DT_E4M3: fmt_ab = 0; fmt_c = 1; break;
    case GZ_DT_E5M2: fmt_ab = 1; fmt_c = 1; break;
    default: fmt_ab = 1; fmt_c = 2; break;         // signed 8-bit operands, s32 accumulate
  }
  uint32_t idesc = 0;
  idesc |= fmt_c << 4;
  idesc |= fmt_ab << 7;
  idesc |= fmt_ab << 10;
  idesc |= ((s.swap ? pr.b_mn_major : pr.a_mn_major) ? 1u : 0u) << 15;
  idesc |= ((s.swap ? pr.a_mn_major : pr.b_mn_major) ? 1u : 0u) << 16;
  idesc |= (uint32_t)(s.bn >> 3) << 17;
  idesc |= (uint32_t)((128 * s.ctas) >> 4) << 24;
  return idesc;
}

gz_status read_scalars(const Problem& pr, const void* alpha, const void* beta, float* af, float* bf,
                       int32_t* ai, int32_t* bi) {
  if (!alpha || !beta) return GZ_ERR_INVALID_ARG;
  *af = *bf = 0.f;
  *ai = *bi = 0;
  if (pr.d.out_type == GZ_DT_S32) {
    *ai = *static_cast<const int32_t*>(alpha);
    *bi = *static_cast<const int32_t*>(beta);
  } else {
    *af = *static_cast<const float*>(alpha);
    *bf = *static_cast<const float*>(beta);
  }
  return GZ_OK;
}

}  // namespace

extern "C" {

GZ_API int32_t gz_version(void) { return 100; }

GZ_API const char* gz_status_string(gz_status s) {
  switch (s) {
    case GZ_OK: return "ok";
    case GZ_ERR_INVALID_ARG: return "invalid argument";
    case GZ_ERR_UNSUPPORTED: return "unsupported data type combination or configuration";
    case GZ_ERR_MISALIGNED:
      return "operand violates an alignment rule (element alignment, or 16-byte leading dimension for "
             "an explicitly requested tensor-core configuration)";
    case GZ_ERR_CUDA: return "CUDA call failed";
    case GZ_ERR_DEVICE_TIMEOUT: return "a bounded wait inside the kernel expired";
    case GZ_ERR_NO_DEVICE: return "no CUDA device of compute capability 10.x";
    case GZ_ERR_TOO_LARGE: return "extent too large";
    case GZ_ERR_OUT_OF_MEMORY: return "out of memory";
    case GZ_ERR_DEBUG_CHECK: return "debug build: an epilogue store failed its bounds check and was skipped";
  }
  return "unknown status";
}

GZ_API const char* gz_last_cuda_error(void) { return g_last_cuda_error.c_str(); }

GZ_API void gz_tile_coords(uint32_t tiles_m, uint32_t tiles_n, uint32_t group_m, uint32_t t,
                           uint32_t* tile_m, uint32_t* tile_n) {
  gz::TileGrid g{tiles_m, tiles_n, group_m ? group_m : 1u, tiles_m * tiles_n};
  uint32_t tm = 0, tn = 0;
  gz::tile_coords(g, t, tm, tn);
  if (tile_m) *tile_m = tm;
  if (tile_n) *tile_n = tn;
}

GZ_API gz_status gz_partition_columns(int64_t n, int32_t parts, int32_t p, int64_t align,
                                      int64_t* begin, int64_t* end) {
  if (n <= 0 || parts <= 0 || p < 0 || p >= parts || align <= 0 || !begin || !end)
    return GZ_ERR_INVALID_ARG;
  // Distribute whole `align`-column blocks; the first (blocks % parts) parts get one more.
  const int64_t blocks = cdiv(n, align);
  const int64_t q = blocks / parts, r = blocks % parts;
  const int64_t b0 = p * q + (p < r ? p : r);
  const int64_t b1 = b0 + q + (p < r ? 1 : 0);
  int64_t lo = b0 * align, hi = b1 * align;
  if (lo > n) lo = n;
  if (hi > n) hi = n;
  *begin = lo;
  *end = hi;
  return GZ_OK;
}

GZ_API gz_status gz_gemm_desc_validate(const gz_gemm_desc* desc, int sm_count, gz_plan_info* info) {
  Problem pr;
  gz_status st = normalise(desc, &pr);
  if (st != GZ_OK) return st;
  if (sm_count <= 0) sm_count = 148;
  int config = pr.d.config;
  if (config == GZ_CFG_AUTO) config = choose_config(pr, sm_count);
  if (config != GZ_CFG_SIMT && !pr.tma_ld_ok) return GZ_ERR_MISALIGNED;
  if (config != GZ_CFG_SIMT && !shape_fits(pr, *shape_of(config))) return GZ_ERR_UNSUPPORTED;
  if (info) fill_info(pr, config, sm_count, info);
  return GZ_OK;
}

GZ_API gz_status gz_gemm_plan_create(gz_plan** out, const gz_gemm_desc* desc) {
  if (!out) return GZ_ERR_INVALID_ARG;
  *out = nullptr;
  Problem pr;
  gz_status st = normalise(desc, &pr);
  if (st != GZ_OK) return st;

  int ndev = 0;
  if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0) {
    (void)cudaGetLastError();
    return GZ_ERR_NO_DEVICE;
  }
  if (pr.d.device >= ndev) return GZ_ERR_INVALID_ARG;
  cudaDeviceProp prop;
  if (!cuda_ok(cudaGetDeviceProperties(&prop, pr.d.device), "cudaGetDeviceProperties"))
    return GZ_ERR_CUDA;
  if (prop.major != 10) return GZ_ERR_NO_DEVICE;
  DeviceGuard guard(pr.d.device);
  if (!guard.ok()) return GZ_ERR_CUDA;

  const int sm_count = prop.multiProcessorCount;
  int config = pr.d.config;
  if (config == GZ_CFG_AUTO) config = choose_config(pr, sm_count);
  if (config != GZ_CFG_SIMT && !pr.tma_ld_ok) return GZ_ERR_MISALIGNED;
  if (config != GZ_CFG_SIMT && !shape_fits(pr, *shape_of(config))) return GZ_ERR_UNSUPPORTED;

  gz_plan* pl = new (std::nothrow) gz_plan();
  if (!pl) return GZ_ERR_OUT_OF_MEMORY;
  pl->pr = pr;
  pl->status_dev = nullptr;
  pl->workspace = nullptr;
  pl->ha = pl->hb = pl->hc = pl->hd = nullptr;
  pl->ha_bytes = pl->hb_bytes = pl->hcd_bytes = 0;
  fill_info(pr, config, sm_count, &pl->info);
  std::memset(&pl->base, 0, sizeof(pl->base));
  pl->entry = {nullptr, nullptr, nullptr, nullptr};

  if (!cuda_ok(cudaMalloc(&pl->status_dev, 4 * sizeof(uint32_t)), "cudaMalloc(status)") ||
      !cuda_ok(cudaMemset(pl->status_dev, 0, 4 * sizeof(uint32_t)), "cudaMemset(status)")) {
    if (pl->status_dev) cudaFree(pl->status_dev);
    delete pl;
    return GZ_ERR_CUDA;
  }

  if (config != GZ_CFG_SIMT) {
    const CfgShape& s = *shape_of(config);
    pl->entry = entry_for(pr.d.in_type, pr.d.out_type, config);
    if (!pl->entry.launch) {
      cudaFree(pl->status_dev);
      delete pl;
      return GZ_ERR_UNSUPPORTED;
    }
    if (!cuda_ok(pl->entry.attr(), "cudaFuncSetAttribute(max dynamic shared memory)")) {
      cudaFree(pl->status_dev);
      delete pl;
      return GZ_ERR_CUDA;
    }
    gz::GemmParams& p = pl->base;
    // Operand "a" of the kernel is whatever rides the 128-row side of the MMA.
    build_operand(&p.a, s.swap ? pr.b_mn_major : pr.a_mn_major, 128 * s.mb, pr.in_size);
    build_operand(&p.b, s.swap ? pr.a_mn_major : pr.b_mn_major, s.bn / s.ctas, pr.in_size);
    const uint32_t tile_m = (uint32_t)s.tile_wide();
    const int64_t wide = s.swap ? pr.d.n : pr.d.m, narrow = s.swap ? pr.d.m : pr.d.n;
    p.grid.tiles_m = (uint32_t)cdiv(wide, tile_m);
    p.grid.tiles_n = (uint32_t)cdiv(narrow, s.bn);
    // Rows of tiles that run concurrently should span about as many output rows as columns.
    uint32_t gm = 2048u / tile_m;
    p.grid.group_m = gm < 1 ? 1 : gm;
    p.grid.num_tiles = p.grid.tiles_m * p.grid.tiles_n;  // per problem of the batch
    const int64_t all_tiles = (int64_t)p.grid.num_tiles * pr.d.batch;
    {
      int64_t first;
      const int parts = tail_parts_for(pr, s, all_tiles, sm_count / s.ctas, &first);
      p.tail_first = (uint32_t)first;
      p.tail_parts = (uint32_t)parts;
      p.virt_tiles = (uint32_t)(first + (all_tiles - first) * parts);
    }
    p.stride_c = pr.d.stride_c;
    p.stride_d = pr.d.stride_d;
    // Operand "a" of the kernel is A, or B for the swapped tiles.
    p.a.broadcast = ((s.swap ? pr.d.stride_b : pr.d.stride_a) == 0) ? 1u : 0u;
    p.b.broadcast = ((s.swap ? pr.d.stride_a : pr.d.stride_b) == 0) ? 1u : 0u;
    p.m = (uint32_t)wide;
    p.n = (uint32_t)narrow;
    p.k = (uint32_t)pr.d.k;
    p.bk = 128u / pr.in_size;
    p.k_blocks = (uint32_t)cdiv(pr.d.k, p.bk);
    p.idesc = build_idesc(pr, s);
    {
      CfgShape strip = s;
      strip.bn = s.bn / (int)p.tail_parts;
      p.idesc_tail = build_idesc(pr, strip);
    }
    p.epilogue_tma = pl->info.epilogue_tma;
    p.test_flags = (pr.d.flags & 0x80000000u) ? 1u : 0u;
    // Skinny problems stream the weight matrix once: spread the tiles' K positions over the HBM channels.
    if (pr.d.m <= 128) p.tune |= gz::TUNE_K_STAGGER;
    p.ldc = pr.d.ldc;
    p.ldd = pr.d.ldd;
    p.status = pl->status_dev;
    p.wait_limit_ns = pr.d.wait_limit_ns;
    if (wants_die_order(pr, s, sm_count, all_tiles)) {
      const gz::DevicePlacement* place = placement_of(pr.d.device, sm_count);
      if (place && place->known) {
        const size_t bytes = gz_plan::kDieTicketSets * 4 * sizeof(uint32_t);
        if (!cuda_ok(cudaMalloc(&pl->die_tickets, bytes), "cudaMalloc(die tickets)") ||
            !cuda_ok(cudaMemset(pl->die_tickets, 0, bytes), "cudaMemset(die tickets)")) {
          if (pl->die_tickets) cudaFree(pl->die_tickets);
          cudaFree(pl->status_dev);
          delete pl;
          return GZ_ERR_OUT_OF_MEMORY;
        }
        std::memcpy(p.die_of_sm, place->die_of_sm, sizeof(p.die_of_sm));
        pl->info.die_order = 1;
      }
    }
    if (pl->info.split_k) {
      const size_t ws_bytes = (size_t)pl->info.workspace_bytes;
      const size_t counter_bytes = (size_t)all_tiles * 4;
      if (!cuda_ok(cudaMalloc(&pl->workspace, ws_bytes), "cudaMalloc(split-K workspace)") ||
          !cuda_ok(cudaMemset(pl->workspace, 0, ws_bytes), "cudaMemset(split-K workspace)")) {
        if (pl->workspace) cudaFree(pl->workspace);
        cudaFree(pl->status_dev);
        delete pl;
        return GZ_ERR_OUT_OF_MEMORY;
      }
      p.split_k = 1;
      p.max_contrib = (uint32_t)pl->info.reserved;
      p.total_kb = (unsigned long long)all_tiles * p.k_blocks;
      p.ws = static_cast<float*>(pl->workspace);
      p.counters = reinterpret_cast<int*>(static_cast<char*>(pl->workspace) + (ws_bytes - counter_bytes));
    }
  }
  *out = pl;
  return GZ_OK;
}

GZ_API gz_status gz_gemm_plan_destroy(gz_plan* pl) {
  if (!pl) return GZ_ERR_INVALID_ARG;
  DeviceGuard guard(pl->pr.d.device);
  if (pl->status_dev) cudaFree(pl->status_dev);
  if (pl->die_tickets) cudaFree(pl->die_tickets);
  if (pl->workspace) cudaFree(pl->workspace);
  if (pl->ha) cudaFree(pl->ha);
  if (pl->hb) cudaFree(pl->hb);
  if (pl->hc) cudaFree(pl->hc);
  if (pl->hd) cudaFree(pl->hd);
  if (pl->block_plan) gz_gemm_plan_destroy(pl->block_plan);
  if (pl->tail_plan) gz_gemm_plan_destroy(pl->tail_plan);
  if (pl->copy_in) cudaStreamDestroy(pl->copy_in);
  if (pl->copy_out) cudaStreamDestroy(pl->copy_out);
  if (pl->ev_start) cudaEventDestroy(pl->ev_start);
  if (pl->ev_out) cudaEventDestroy(pl->ev_out);
  for (int i = 0; i < gz_plan::kMaxBlocks; ++i) {
    if (pl->ev_in[i]) cudaEventDestroy(pl->ev_in[i]);
    if (pl->ev_gemm[i]) cudaEventDestroy(pl->ev_gemm[i]);
  }
  delete pl;
  return GZ_OK;
}

GZ_API gz_status gz_gemm_plan_set_profile(gz_plan* pl, void* device_words) {
  if (!pl) return GZ_ERR_INVALID_ARG;
  if (device_words) {
    if (!pl->entry.launch_prof) return GZ_ERR_UNSUPPORTED;
    DeviceGuard guard(pl->pr.d.device);
    if (!guard.ok() || !cuda_ok(pl->entry.attr_prof(), "cudaFuncSetAttribute(max dynamic shared memory)"))
      return GZ_ERR_CUDA;
  }
  pl->base.prof = static_cast<unsigned long long*>(device_words);
  return GZ_OK;
}

GZ_API gz_status gz_classify_dies(const uint32_t* clocks, int32_t sms, int32_t lines, uint8_t* die_of_sm,
                                  int32_t sms_on_die[2]) {
  if (!clocks || !die_of_sm || !sms_on_die || sms <= 0 || sms > 160 || lines <= 0) return GZ_ERR_INVALID_ARG;
  std::vector<uint32_t> v(clocks, clocks + static_cast<size_t>(sms) * lines);
  int counts[2] = {0, 0};
  uint8_t dies[160] = {};
  const bool ok = gz::classify_dies(v, sms, lines, dies, counts);
  if (!ok) return GZ_ERR_UNSUPPORTED;
  std::memcpy(die_of_sm, dies, static_cast<size_t>(sms));
  sms_on_die[0] = counts[0];
  sms_on_die[1] = counts[1];
  return GZ_OK;
}

GZ_API gz_status gz_device_placement(int32_t device, uint8_t* die_of_sm, int32_t sms_on_die[2]) {
  if (!die_of_sm || !sms_on_die) return GZ_ERR_INVALID_ARG;
  int ndev = 0;
  if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0) {
    (void)cudaGetLastError();
    return GZ_ERR_NO_DEVICE;
  }
  if (device < 0 || device >= ndev || device >= 64) return GZ_ERR_INVALID_ARG;
  int sms = 0;
  if (!cuda_ok(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device), "device attribute")) return GZ_ERR_CUDA;
  DeviceGuard guard(device);
  if (!guard.ok()) return GZ_ERR_CUDA;
  const gz::DevicePlacement* place = placement_of(device, sms);
  if (!place || !place->known) return GZ_ERR_UNSUPPORTED;
  std::memcpy(die_of_sm, place->die_of_sm, static_cast<size_t>(sms));
  sms_on_die[0] = place->sms_on_die[0];
  sms_on_die[1] = place->sms_on_die[1];
  return GZ_OK;
}

GZ_API gz_status gz_gemm_plan_info(const gz_plan* pl, gz_plan_info* info) {
  if (!pl || !info) return GZ_ERR_INVALID_ARG;
  *info = pl->info;
  return GZ_OK;
}

}  // extern "C"

namespace {

// Where a launch writes its output when not to one matrix: column block o of width `cols` goes to
// ptrs[o] (row pitch ld elements).  Used by the K-sharded GEMM, whose pointers are peer memory.
struct ScatterSpec {
  uint32_t cols;
  int parts;
  int64_t ld;
  void* ptrs[8];
  // completion signal raised by the launch's last CTA (see GemmParams::signal_count); 0 = none
  int signal_count = 0;
  uint32_t signal_value = 0;
  uint32_t* signal_ptrs[8] = {};
  uint32_t* signal_counter = nullptr;
};

gz_status run_impl(gz_plan* pl, const void* a, const void* b, const void* c, void* d, const void* alpha,
                   const void* beta, void* stream_v, const ScatterSpec* sc, const gz_epilogue* ep = nullptr) {
  if (!pl || !a || !b || !d) return GZ_ERR_INVALID_ARG;
  const Problem& pr = pl->pr;
  uint32_t epi_flags = 0;
  if (ep) {
    if (ep->struct_size != sizeof(gz_epilogue) || ep->activation < GZ_ACT_NONE || ep->activation > GZ_ACT_SILU)
      return GZ_ERR_INVALID_ARG;
    epi_flags = (ep->bias ? 1u : 0u) | (ep->row_scale ? 2u : 0u) | (ep->col_scale ? 4u : 0u) |
                (ep->activation != GZ_ACT_NONE ? 8u : 0u);
    if (epi_flags != 0 && pr.d.out_type == GZ_DT_S32) return GZ_ERR_UNSUPPORTED;
    auto bad = [](const float* q) { return q && reinterpret_cast<uintptr_t>(q) % 4 != 0; };
    if (bad(ep->bias) || bad(ep->row_scale) || bad(ep->col_scale)) return GZ_ERR_MISALIGNED;
  }
  if (sc) {
    if (pl->info.config == GZ_CFG_SIMT || pr.out_size != 4 || pr.d.batch != 1 || sc->cols == 0 || sc->cols % 32 != 0 ||
        sc->parts < 1 || sc->parts > 8 || (int64_t)sc->cols * sc->parts < pr.d.n || sc->ld < sc->cols)
      return GZ_ERR_UNSUPPORTED;
  }
  float af, bf;
  int32_t ai, bi;
  gz_status st = read_scalars(pr, alpha, beta, &af, &bf, &ai, &bi);
  if (st != GZ_OK) return st;
  const bool beta_zero = (pr.d.out_type == GZ_DT_S32) ? (bi == 0) : (bf == 0.0f);
  if (!beta_zero && !c) return GZ_ERR_INVALID_ARG;
  auto misaligned = [](const void* p, int sz) { return (reinterpret_cast<uintptr_t>(p) % sz) != 0; };
  if (misaligned(a, pr.in_size) || misaligned(b, pr.in_size) || misaligned(d, pr.out_size) ||
      (c && misaligned(c, pr.out_size)))
    return GZ_ERR_MISALIGNED;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  DeviceGuard guard(pr.d.device);
  if (!guard.ok()) return GZ_ERR_CUDA;

  const bool tma_ptr_ok = (reinterpret_cast<uintptr_t>(a) % 16 == 0) &&
                          (reinterpret_cast<uintptr_t>(b) % 16 == 0);
  if (sc && !tma_ptr_ok) return GZ_ERR_MISALIGNED;
  if (pl->info.config == GZ_CFG_SIMT || !tma_ptr_ok) {
    gz::SimtParams sp;
    sp.a = a;
    sp.b = b;
    sp.c = beta_zero ? nullptr : c;
    sp.d = d;
    sp.m = pr.d.m;
    sp.n = pr.d.n;
    sp.k = pr.d.k;
    sp.a_sm = pr.a_mn_major ? 1 : pr.d.lda;
    sp.a_sk = pr.a_mn_major ? pr.d.lda : 1;
    sp.b_sk = pr.b_mn_major ? pr.d.ldb : 1;
    sp.b_sn = pr.b_mn_major ? 1 : pr.d.ldb;
    sp.ldc = pr.d.ldc;
    sp.ldd = pr.d.ldd;
    sp.batch = pr.d.batch;
    sp.stride_a = pr.d.stride_a;
    sp.stride_b = pr.d.stride_b;
    sp.stride_c = pr.d.stride_c;
    sp.stride_d = pr.d.stride_d;
    sp.alpha_f = af;
    sp.beta_f = bf;
    sp.alpha_i = ai;
    sp.beta_i = bi;
    sp.epi_flags = epi_flags;
    sp.act = epi_flags ? (uint32_t)ep->activation : 0u;
    sp.bias = epi_flags ? ep->bias : nullptr;
    sp.row_scale = epi_flags ? ep->row_scale : nullptr;
    sp.col_scale = epi_flags ? ep->col_scale : nullptr;
    if (!cuda_ok(launch_simt_any(pr.d.in_type, pr.d.out_type, sp, stream), "simt launch"))
      return GZ_ERR_CUDA;
    return GZ_OK;
  }

  const CfgShape& s = *shape_of(pl->info.config);
  gz::GemmParams p = pl->base;
  p.alpha_f = af;
  p.beta_f = bf;
  p.alpha_i = ai;
  p.beta_i = bi;
  p.c = beta_zero ? nullptr : c;
  p.d = d;
  p.c_vec_ok = (c && reinterpret_cast<uintptr_t>(c) % 16 == 0 && (pr.d.ldc * pr.out_size) % 16 == 0) ? 1u : 0u;
  p.d_vec_ok = (reinterpret_cast<uintptr_t>(d) % 16 == 0 && (pr.d.ldd * pr.out_size) % 16 == 0) ? 1u : 0u;
  if (p.epilogue_tma && reinterpret_cast<uintptr_t>(d) % 16 != 0) p.epilogue_tma = 0;
  if (epi_flags) {
    p.epi_flags = epi_flags;
    p.act = (uint32_t)ep->activation;
    // The swapped (skinny) tiles walk N along the 128-row side; the kernel indexes the vectors by
    // output row and column, so nothing is exchanged here.
    p.bias = ep->bias;
    p.row_scale = ep->row_scale;
    p.col_scale = ep->col_scale;
  }
  if (sc) {
    p.epilogue_tma = 0;
    p.scatter_cols = sc->cols;
    p.ldd = sc->ld;
    bool vec = (sc->ld * pr.out_size) % 16 == 0;
    for (int i = 0; i < 8; ++i) {
      p.scatter_ptrs[i] = i < sc->parts ? sc->ptrs[i] : nullptr;
      if (i < sc->parts && reinterpret_cast<uintptr_t>(sc->ptrs[i]) % 16 != 0) vec = false;
    }
    p.d_vec_ok = vec ? 1u : 0u;
    if (sc->signal_count > 0 && sc->signal_counter) {
      p.signal_count = (uint32_t)sc->signal_count;
      p.signal_value = sc->signal_value;
      p.signal_counter = sc->signal_counter;
      for (int i = 0; i < 8; ++i) p.signal_ptrs[i] = i < sc->signal_count ? sc->signal_ptrs[i] : nullptr;
    }
  }

  if (pl->die_tickets)
    p.die_tickets = pl->die_tickets + 4u * (pl->launch_seq.fetch_add(1u, std::memory_order_relaxed) % gz_plan::kDieTicketSets);
  CUtensorMap ta, tb, td;
  const void* const d_key = p.epilogue_tma ? d : nullptr;
  bool cached = false;
  {
    std::lock_guard<std::mutex> lock(pl->tmap_mu);
    for (TensorMapSet& e : pl->tmaps) {
      if (e.stamp != 0 && e.a == a && e.b == b && e.d == d_key) {
        ta = e.ta;
        tb = e.tb;
        td = e.td;
        e.stamp = ++pl->tmap_clock;
        cached = true;
        break;
      }
    }
  }
  const LaunchFn fn = p.prof ? pl->entry.launch_prof : pl->entry.launch;
  if (cached) {
    if (!cuda_ok(fn(ta, tb, td, p, pl->info.grid, stream), "kernel launch")) return GZ_ERR_CUDA;
    return GZ_OK;
  }
  const uint32_t bk = 128u / pr.in_size;
  // Tensor map of one input matrix: `rows` is its M (or N) extent, `od` the kernel operand it feeds.
  auto encode_input = [&](CUtensorMap* tm, const void* base, bool mn_major, int64_t rows, int64_t ld,
                          const gz::OperandDesc& od, int64_t batch_stride) {
    if (!mn_major)
      return encode_2d(tm, pr.d.in_type, base, (uint64_t)pr.d.k, (uint64_t)rows, (uint64_t)ld * pr.in_size,
                       bk, od.box_mn, true, false, (uint64_t)pr.d.batch, (uint64_t)batch_stride * pr.in_size);
    return encode_2d(tm, pr.d.in_type, base, (uint64_t)rows, (uint64_t)pr.d.k, (uint64_t)ld * pr.in_size,
                     od.box_mn, bk, true, pr.in_size == 4, (uint64_t)pr.d.batch,
                     (uint64_t)batch_stride * pr.in_size);
  };
  bool ok;
  if (!s.swap) {
    ok = encode_input(&ta, a, pr.a_mn_major, pr.d.m, pr.d.lda, p.a, pr.d.stride_a) &&
         encode_input(&tb, b, pr.b_mn_major, pr.d.n, pr.d.ldb, p.b, pr.d.stride_b);
  } else {
    ok = encode_input(&ta, b, pr.b_mn_major, pr.d.n, pr.d.ldb, p.a, pr.d.stride_b) &&
         encode_input(&tb, a, pr.a_mn_major, pr.d.m, pr.d.lda, p.b, pr.d.stride_a);
  }
  if (!ok) return GZ_ERR_CUDA;
  if (p.epilogue_tma) {
    ok = encode_2d(&td, pr.d.out_type, d, (uint64_t)pr.d.n, (uint64_t)pr.d.m,
                   (uint64_t)pr.d.ldd * pr.out_size, 128u / pr.out_size, 32, false, false,
                   (uint64_t)pr.d.batch, (uint64_t)pr.d.stride_d * pr.out_size);
    if (!ok) return GZ_ERR_CUDA;
  } else {
    td = ta;  // unused by the kernel in this mode
  }
  {
    std::lock_guard<std::mutex> lock(pl->tmap_mu);
    TensorMapSet* victim = &pl->tmaps[0];
    for (TensorMapSet& e : pl->tmaps)
      if (e.stamp < victim->stamp) victim = &e;  // an empty slot, else the least recently used
    victim->a = a;
    victim->b = b;
    victim->d = d_key;
    victim->ta = ta;
    victim->tb = tb;
    victim->td = td;
    victim->stamp = ++pl->tmap_clock;
  }
  if (!cuda_ok(fn(ta, tb, td, p, pl->info.grid, stream), "kernel launch"))
    return GZ_ERR_CUDA;
  return GZ_OK;
}

}  // namespace

extern "C" {

GZ_API gz_status gz_gemm_run(gz_plan* pl, const void* a, const void* b, const void* c, void* d,
                             const void* alpha, const void* beta, void* stream_v) {
  return run_impl(pl, a, b, c, d, alpha, beta, stream_v, nullptr);
}

GZ_API gz_status gz_gemm_run_ex(gz_plan* pl, const void* a, const void* b, const void* c, void* d,
                                const void* alpha, const void* beta, const gz_epilogue* ep, void* stream_v) {
  return run_impl(pl, a, b, c, d, alpha, beta, stream_v, nullptr, ep);
}

}  // extern "C"

namespace {

// a_on_device: A is a device pointer on the plan's GPU and already valid in stream order (the
// replicated operand of a column-partitioned run, gathered GPU to GPU); only B, C and D cross PCIe.
gz_status run_host_impl(gz_plan* pl, const void* a, const void* b, const void* c, void* d, const void* alpha,
                        const void* beta, void* stream_v, bool a_on_device) {
  if (!pl || !a || !b || !d) return GZ_ERR_INVALID_ARG;
  const Problem& pr = pl->pr;
  float af, bf;
  int32_t ai, bi;
  gz_status st = read_scalars(pr, alpha, beta, &af, &bf, &ai, &bi);
  if (st != GZ_OK) return st;
  const bool beta_zero = (pr.d.out_type == GZ_DT_S32) ? (bi == 0) : (bf == 0.0f);
  if (!beta_zero && !c) return GZ_ERR_INVALID_ARG;
  if (pr.d.batch != 1) return GZ_ERR_UNSUPPORTED;  // the host-operand pipeline moves one problem
  DeviceGuard guard(pr.d.device);
  if (!guard.ok()) return GZ_ERR_CUDA;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);

  const size_t a_rows = pr.a_mn_major ? pr.d.k : pr.d.m;
  const size_t b_rows = pr.b_mn_major ? pr.d.k : pr.d.n;
  const size_t a_bytes = a_rows * pr.d.lda * pr.in_size;
  const size_t b_bytes = b_rows * pr.d.ldb * pr.in_size;
  const size_t c_bytes = (size_t)pr.d.m * pr.d.ldc * pr.out_size;
  const size_t d_bytes = (size_t)pr.d.m * pr.d.ldd * pr.out_size;
  {
    std::lock_guard<std::mutex> lock(pl->mu);
    if (!pl->hb) {
      const size_t cd = c_bytes > d_bytes ? c_bytes : d_bytes;
      if ((!a_on_device && !cuda_ok(cudaMalloc(&pl->ha, a_bytes), "cudaMalloc(A staging)")) ||
          !cuda_ok(cudaMalloc(&pl->hb, b_bytes), "cudaMalloc(B staging)") ||
          !cuda_ok(cudaMalloc(&pl->hc, cd), "cudaMalloc(C staging)") ||
          !cuda_ok(cudaMalloc(&pl->hd, cd), "cudaMalloc(D staging)"))
        return GZ_ERR_OUT_OF_MEMORY;
    }
  }
  // Small problems: one upload, one launch, one download on the caller's stream.
  const bool pipelined = (a_bytes + b_bytes + d_bytes >= (size_t(32) << 20)) && pr.d.n >= 2048;
  if (!a_on_device && !pl->ha) {  // a plan first used with a resident A, now with a host A
    std::lock_guard<std::mutex> lock(pl->mu);
    if (!pl->ha && !cuda_ok(cudaMalloc(&pl->ha, a_bytes), "cudaMalloc(A staging)")) return GZ_ERR_OUT_OF_MEMORY;
  }
  const void* a_dev = a_on_device ? a : pl->ha;
  if (!pipelined) {
    if ((!a_on_device && !cuda_ok(cudaMemcpyAsync(pl->ha, a, a_bytes, cudaMemcpyHostToDevice, stream), "H2D A")) ||
        !cuda_ok(cudaMemcpyAsync(pl->hb, b, b_bytes, cudaMemcpyHostToDevice, stream), "H2D B"))
      return GZ_ERR_CUDA;
    if (!beta_zero &&
        !cuda_ok(cudaMemcpyAsync(pl->hc, c, c_bytes, cudaMemcpyHostToDevice, stream), "H2D C"))
      return GZ_ERR_CUDA;
    st = gz_gemm_run(pl, a_dev, pl->hb, beta_zero ? nullptr : pl->hc, pl->hd, alpha, beta, stream_v);
    if (st != GZ_OK) return st;
    if (!cuda_ok(cudaMemcpyAsync(d, pl->hd, d_bytes, cudaMemcpyDeviceToHost, stream), "D2H D") ||
        !cuda_ok(cudaStreamSynchronize(stream), "cudaStreamSynchronize"))
      return GZ_ERR_CUDA;
    return GZ_OK;
  }

  // Large problems: A goes up first, then B (and C) in column blocks; block j is multiplied on the
  // caller's stream as soon as it has landed, and its block of D goes down while later blocks are
  // still going up.
  {
    std::lock_guard<std::mutex> lock(pl->mu);
    if (!pl->pipe_ready) {
      // About 16 blocks, 256-column granularity: what nothing can overlap is the last block's GEMM
      // and download, so the blocks are as small as the event budget (kMaxBlocks) allows.
      int64_t cols = cdiv(cdiv(pr.d.n, gz_plan::kMaxBlocks), 256) * 256;
      if (cols < 256) cols = 256;
      int blocks = (int)cdiv(pr.d.n, cols);
      if (blocks > gz_plan::kMaxBlocks) {
        cols = cdiv(cdiv(pr.d.n, gz_plan::kMaxBlocks), 256) * 256;
        blocks = (int)cdiv(pr.d.n, cols);
      }
      gz_gemm_desc bd = pr.d;
      bd.flags &= ~GZ_FLAG_TEST_WITHHOLD_ACC_READY;
      bd.config = GZ_CFG_AUTO;
      bd.n = cols < pr.d.n ? cols : pr.d.n;
      if ((st = gz_gemm_plan_create(&pl->block_plan, &bd)) != GZ_OK) return st;
      const int64_t tail = pr.d.n - (int64_t)(blocks - 1) * cols;
      if (blocks > 1 && tail != cols) {
        bd.n = tail;
        if ((st = gz_gemm_plan_create(&pl->tail_plan, &bd)) != GZ_OK) return st;
      }
      bool ok = cuda_ok(cudaStreamCreateWithFlags(&pl->copy_in, cudaStreamNonBlocking), "cudaStreamCreate") &&
                cuda_ok(cudaStreamCreateWithFlags(&pl->copy_out, cudaStreamNonBlocking), "cudaStreamCreate") &&
                cuda_ok(cudaEventCreateWithFlags(&pl->ev_start, cudaEventDisableTiming), "cudaEventCreate") &&
                cuda_ok(cudaEventCreateWithFlags(&pl->ev_out, cudaEventDisableTiming), "cudaEventCreate");
      for (int i = 0; ok && i < blocks; ++i)
        ok = cuda_ok(cudaEventCreateWithFlags(&pl->ev_in[i], cudaEventDisableTiming), "cudaEventCreate") &&
             cuda_ok(cudaEventCreateWithFlags(&pl->ev_gemm[i], cudaEventDisableTiming), "cudaEventCreate");
      if (!ok) return GZ_ERR_CUDA;
      pl->block_cols = cols;
      pl->blocks = blocks;
      pl->pipe_ready = true;
    }
  }
  const int64_t cols = pl->block_cols;
  const size_t isz = pr.in_size, osz = pr.out_size;
  // The uploads start where the caller's stream stands.  With a resident A that is after whatever
  // the caller queued to make A valid (its own slice's upload and the gather): the slice gets the
  // host-to-device direction of the link to itself first, because nothing can be multiplied before
  // A is complete, and the blocks of B follow.
  bool ok = cuda_ok(cudaEventRecord(pl->ev_start, stream), "cudaEventRecord") &&
            cuda_ok(cudaStreamWaitEvent(pl->copy_in, pl->ev_start, 0), "cudaStreamWaitEvent") &&
            cuda_ok(cudaStreamWaitEvent(pl->copy_out, pl->ev_start, 0), "cudaStreamWaitEvent") &&
            (a_on_device || cuda_ok(cudaMemcpyAsync(pl->ha, a, a_bytes, cudaMemcpyHostToDevice, pl->copy_in), "H2D A"));
  for (int j = 0; ok && j < pl->blocks; ++j) {
    const int64_t n0 = (int64_t)j * cols;
    const int64_t nj = (n0 + cols <= pr.d.n) ? cols : pr.d.n - n0;
    if (!pr.b_mn_major) {  // column-major B: a column block is contiguous
      const size_t off = (size_t)n0 * pr.d.ldb * isz;
      ok = cuda_ok(cudaMemcpyAsync(static_cast<char*>(pl->hb) + off, static_cast<const char*>(b) + off,
                                   (size_t)nj * pr.d.ldb * isz, cudaMemcpyHostToDevice, pl->copy_in), "H2D B block");
    } else {               // row-major B: k rows of nj columns
      const size_t off = (size_t)n0 * isz, pitch = (size_t)pr.d.ldb * isz;
      ok = cuda_ok(cudaMemcpy2DAsync(static_cast<char*>(pl->hb) + off, pitch, static_cast<const char*>(b) + off,
                                     pitch, (size_t)nj * isz, (size_t)pr.d.k, cudaMemcpyHostToDevice, pl->copy_in),
                   "H2D B block");
    }
    if (ok && !beta_zero) {
      const size_t off = (size_t)n0 * osz, pitch = (size_t)pr.d.ldc * osz;
      ok = cuda_ok(cudaMemcpy2DAsync(static_cast<char*>(pl->hc) + off, pitch, static_cast<const char*>(c) + off,
                                     pitch, (size_t)nj * osz, (size_t)pr.d.m, cudaMemcpyHostToDevice, pl->copy_in),
                   "H2D C block");
    }
    ok = ok && cuda_ok(cudaEventRecord(pl->ev_in[j], pl->copy_in), "cudaEventRecord");
  }
  if (!ok) return GZ_ERR_CUDA;
  for (int j = 0; j < pl->blocks; ++j) {
    const int64_t n0 = (int64_t)j * cols;
    const int64_t nj = (n0 + cols <= pr.d.n) ? cols : pr.d.n - n0;
    gz_plan* sub = (nj == cols || !pl->tail_plan) ? pl->block_plan : pl->tail_plan;
    const char* bj = static_cast<const char*>(pl->hb) + (pr.b_mn_major ? (size_t)n0 * isz : (size_t)n0 * pr.d.ldb * isz);
    const char* cj = static_cast<const char*>(pl->hc) + (size_t)n0 * osz;
    char* dj = static_cast<char*>(pl->hd) + (size_t)n0 * osz;
    if (!cuda_ok(cudaStreamWaitEvent(stream, pl->ev_in[j], 0), "cudaStreamWaitEvent")) return GZ_ERR_CUDA;
    st = gz_gemm_run(sub, a_dev, bj, beta_zero ? nullptr : cj, dj, alpha, beta, stream_v);
    if (st != GZ_OK) return st;
    const size_t pitch_h = (size_t)pr.d.ldd * osz;
    if (!cuda_ok(cudaEventRecord(pl->ev_gemm[j], stream), "cudaEventRecord") ||
        !cuda_ok(cudaStreamWaitEvent(pl->copy_out, pl->ev_gemm[j], 0), "cudaStreamWaitEvent") ||
        !cuda_ok(cudaMemcpy2DAsync(static_cast<char*>(d) + (size_t)n0 * osz, pitch_h, dj, pitch_h, (size_t)nj * osz,
                                   (size_t)pr.d.m, cudaMemcpyDeviceToHost, pl->copy_out), "D2H D block"))
      return GZ_ERR_CUDA;
  }
  if (!cuda_ok(cudaEventRecord(pl->ev_out, pl->copy_out), "cudaEventRecord") ||
      !cuda_ok(cudaStreamWaitEvent(stream, pl->ev_out, 0), "cudaStreamWaitEvent") ||
      !cuda_ok(cudaStreamSynchronize(stream), "cudaStreamSynchronize"))
    return GZ_ERR_CUDA;
  return GZ_OK;
}

}  // namespace

extern "C" {

GZ_API gz_status gz_gemm_run_host(gz_plan* pl, const void* a, const void* b, const void* c, void* d,
                                  const void* alpha, const void* beta, void* stream_v) {
  return run_host_impl(pl, a, b, c, d, alpha, beta, stream_v, false);
}

GZ_API gz_status gz_gemm_run_host_ex(gz_plan* pl, const void* a, const void* b, const void* c, void* d,
                                     const void* alpha, const void* beta, void* stream_v, uint32_t host_flags) {
  if (host_flags & ~GZ_HOST_A_ON_DEVICE) return GZ_ERR_INVALID_ARG;
  return run_host_impl(pl, a, b, c, d, alpha, beta, stream_v, (host_flags & GZ_HOST_A_ON_DEVICE) != 0);
}

GZ_API gz_status gz_last_device_status(gz_plan* pl, void* stream_v, uint32_t detail[4]) {
  if (!pl) return GZ_ERR_INVALID_ARG;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  DeviceGuard guard(pl->pr.d.device);
  if (!guard.ok()) return GZ_ERR_CUDA;
  uint32_t h[4] = {0, 0, 0, 0};
  if (!cuda_ok(cudaStreamSynchronize(stream), "cudaStreamSynchronize") ||
      !cuda_ok(cudaMemcpy(h, pl->status_dev, sizeof(h), cudaMemcpyDeviceToHost), "read status"))
    return GZ_ERR_CUDA;
  if (detail) std::memcpy(detail, h, sizeof(h));
  if (h[0] != 0) {
    (void)cudaMemset(pl->status_dev, 0, sizeof(h));
    // A split-K launch that gave up may have left arrival counters of unfinished tiles non-zero
    // (only a tile's last arriver resets its counter); the next launch must find them at zero.
    if (pl->base.split_k && pl->base.counters) {
      const size_t counter_bytes = (size_t)pl->base.grid.num_tiles * (size_t)pl->pr.d.batch * 4;
      (void)cudaMemset(pl->base.counters, 0, counter_bytes);
    }
    return h[0] == gz::STORE_OUT_OF_BOUNDS ? GZ_ERR_DEBUG_CHECK : GZ_ERR_DEVICE_TIMEOUT;
  }
  return GZ_OK;
}

}  // extern "C"

// ------------------------------------------------------------------ fills
namespace {

template <typename T>
__device__ __forceinline__ T fill_cast(float v);
template <>
__device__ __forceinline__ float fill_cast<float>(float v) { return v; }
template <>
__device__ __forceinline__ __half fill_cast<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 fill_cast<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}
template <>
__device__ __forceinline__ __nv_fp8_e4m3 fill_cast<__nv_fp8_e4m3>(float v) { return __nv_fp8_e4m3(v); }
template <>
__device__ __forceinline__ __nv_fp8_e5m2 fill_cast<__nv_fp8_e5m2>(float v) { return __nv_fp8_e5m2(v); }
template <>
__device__ __forceinline__ int8_t fill_cast<int8_t>(float v) {
  return static_cast<int8_t>(fmaxf(-128.f, fminf(127.f, rintf(v))));
}
template <>
__device__ __forceinline__ int32_t fill_cast<int32_t>(float v) {
  return static_cast<int32_t>(rintf(v));
}

template <typename T>
__global__ void fill_kernel(T* ptr, int64_t count, uint64_t seed, uint32_t stream_id, int dist,
                            float scale) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < count;
       i += stride) {
    const uint64_t bits = gz::rng_bits(seed, stream_id, static_cast<uint64_t>(i));
    float v;
    if (dist == 0) {
      v = gz::rng_uniform_pm1(bits) * scale;
    } else if (dist == 1) {
      // Box-Muller on two 24-bit uniforms taken from the same 64 random bits.
      const float u1 = (static_cast<float>(static_cast<uint32_t>(bits >> 40)) + 1.0f) * (1.0f / 16777216.0f);
      const float u2 = static_cast<float>(static_cast<uint32_t>(bits >> 16) & 0xFFFFFFu) * (1.0f / 16777216.0f);
      v = sqrtf(-2.0f * logf(u1)) * cospif(2.0f * u2) * scale;
    } else {
      if (std::is_same<T, int8_t>::value) v = static_cast<float>(gz::rng_int8(bits));
      else {
        const int32_t span = 2 * static_cast<int32_t>(scale) + 1;
        v = static_cast<float>(static_cast<int32_t>((bits >> 33) % static_cast<uint64_t>(span)) -
                               static_cast<int32_t>(scale));
      }
    }
    ptr[i] = fill_cast<T>(v);
  }
}

}  // namespace

extern "C" GZ_API gz_status gz_fill(void* ptr, int32_t dtype, int64_t count, uint64_t seed,
                                    uint32_t stream_id, int32_t dist, float scale, void* stream_v) {
  if (!ptr || count < 0 || dist < 0 || dist > 2 || dtype_size(dtype) == 0) return GZ_ERR_INVALID_ARG;
  if (count == 0) return GZ_OK;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  // The kernel runs on the GPU that owns the buffer, whatever the caller's current device.
  cudaPointerAttributes attr;
  if (!cuda_ok(cudaPointerGetAttributes(&attr, ptr), "cudaPointerGetAttributes")) return GZ_ERR_CUDA;
  if (attr.type != cudaMemoryTypeDevice && attr.type != cudaMemoryTypeManaged) return GZ_ERR_INVALID_ARG;
  DeviceGuard guard(attr.device);
  if (!guard.ok()) return GZ_ERR_CUDA;
  const int block = 256;
  int64_t want = cdiv(count, block);
  const int grid = (int)(want < 148 * 16 ? want : 148 * 16);
  switch (dtype) {
    case GZ_DT_F16:
      fill_kernel<__half><<<grid, block, 0, stream>>>((__half*)ptr, count, seed, stream_id, dist, scale);
      break;
    case GZ_DT_BF16:
      fill_kernel<__nv_bfloat16><<<grid, block, 0, stream>>>((__nv_bfloat16*)ptr, count, seed, stream_id, dist, scale);
      break;
    case GZ_DT_F32:
      fill_kernel<float><<<grid, block, 0, stream>>>((float*)ptr, count, seed, stream_id, dist, scale);
      break;
    case GZ_DT_S8:
      fill_kernel<int8_t><<<grid, block, 0, stream>>>((int8_t*)ptr, count, seed, stream_id, dist, scale);
      break;
    case GZ_DT_S32:
      fill_kernel<int32_t><<<grid, block, 0, stream>>>((int32_t*)ptr, count, seed, stream_id, dist, scale);
      break;
    case GZ_DT_E4M3:
      fill_kernel<__nv_fp8_e4m3><<<grid, block, 0, stream>>>((__nv_fp8_e4m3*)ptr, count, seed, stream_id, dist, scale);
      break;
    case GZ_DT_E5M2:
      fill_kernel<__nv_fp8_e5m2><<<grid, block, 0, stream>>>((__nv_fp8_e5m2*)ptr, count, seed, stream_id, dist, scale);
      break;
  }
  if (!cuda_ok(cudaGetLastError(), "fill launch")) return GZ_ERR_CUDA;
  return GZ_OK;
}

// ------------------------------------------------------------------ no-allocation entry point
//
// Some hosts hand all device memory to their own allocator at start-up and forbid any later
// cudaMalloc: it could fail against their budget, and it synchronises the device in the middle of
// a latency-critical loop.  Such a host cannot use gz_gemm_plan_create (which allocates the plan's
// status words and split-K workspace).  For it, the skinny split-K GEMM is offered once more with
// its scratch memory in a fixed array that is part of the library image: every GPU that loads the
// library holds GZ_STATIC_SCRATCH_BYTES of it until the process exits.
namespace {

static __device__ __align__(256) unsigned char g_static_scratch[GZ_STATIC_SCRATCH_BYTES];

struct StaticScratchDevice {
  void* ptr = nullptr;  // device address of g_static_scratch on this device
  int sm_count = 0;
  bool ready = false;
};
constexpr int kMaxDevices = 64;
StaticScratchDevice g_static_dev[kMaxDevices];
std::mutex g_static_mu;

// Once per device, with that device current: the array's name is only a host-side handle, the
// kernel needs the address cudaGetSymbolAddress reports for the current device.
gz_status static_scratch_setup(int device, StaticScratchDevice** out) {
  if (device < 0 || device >= kMaxDevices) return GZ_ERR_INVALID_ARG;
  std::lock_guard<std::mutex> lock(g_static_mu);
  StaticScratchDevice& sd = g_static_dev[device];
  if (!sd.ready) {
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0) {
      (void)cudaGetLastError();
      return GZ_ERR_NO_DEVICE;
    }
    if (device >= ndev) return GZ_ERR_INVALID_ARG;
    int major = 0, sms = 0;
    if (!cuda_ok(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device), "device attribute") ||
        !cuda_ok(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device), "device attribute"))
      return GZ_ERR_CUDA;
    if (major != 10) return GZ_ERR_NO_DEVICE;
    DeviceGuard guard(device);  // the symbol's address is taken with its device current
    if (!guard.ok()) return GZ_ERR_CUDA;
    void* ptr = nullptr;
    if (!cuda_ok(cudaGetSymbolAddress(&ptr, g_static_scratch), "cudaGetSymbolAddress(static scratch)") || !ptr)
      return GZ_ERR_CUDA;
    sd.ptr = ptr;
    sd.sm_count = sms;
    sd.ready = true;
  }
  *out = &sd;
  return GZ_OK;
}

}  // namespace

extern "C" GZ_API gz_status gz_gemm_skinny_static(const gz_gemm_desc* desc, const void* a, const void* b,
                                                  const void* c, void* d, const void* alpha,
                                                  const void* beta, void* stream_v) {
  if (!desc || !a || !b || !d) return GZ_ERR_INVALID_ARG;
  gz_gemm_desc dd = *desc;
  if (dd.struct_size != sizeof(gz_gemm_desc)) return GZ_ERR_INVALID_ARG;
  dd.flags = (dd.flags & ~GZ_FLAG_NO_SPLIT_K) | GZ_FLAG_SPLIT_K | GZ_FLAG_EPILOGUE_DIRECT;
  dd.flags &= ~GZ_FLAG_EPILOGUE_TMA;
  Problem pr;
  gz_status st = normalise(&dd, &pr);
  if (st != GZ_OK) return st;
  if (pr.d.m > 128) return GZ_ERR_UNSUPPORTED;  // only the skinny (swapped-operand) kernel uses scratch
  if (!pr.tma_ld_ok) return GZ_ERR_MISALIGNED;
  auto misaligned = [](const void* p, int sz) { return (reinterpret_cast<uintptr_t>(p) % sz) != 0; };
  if (misaligned(a, 16) || misaligned(b, 16) || misaligned(d, pr.out_size) || (c && misaligned(c, pr.out_size)))
    return GZ_ERR_MISALIGNED;
  float af, bf;
  int32_t ai, bi;
  st = read_scalars(pr, alpha, beta, &af, &bf, &ai, &bi);
  if (st != GZ_OK) return st;
  const bool beta_zero = (pr.d.out_type == GZ_DT_S32) ? (bi == 0) : (bf == 0.0f);
  if (!beta_zero && !c) return GZ_ERR_INVALID_ARG;

  if (pr.d.batch != 1) return GZ_ERR_UNSUPPORTED;
  StaticScratchDevice* sd = nullptr;
  st = static_scratch_setup(pr.d.device, &sd);
  if (st != GZ_OK) return st;
  DeviceGuard guard(pr.d.device);
  if (!guard.ok()) return GZ_ERR_CUDA;

  int config = pr.d.config;
  if (config == GZ_CFG_AUTO)
    config = pr.d.m <= 16 ? GZ_CFG_SWAP_M16 : pr.d.m <= 32 ? GZ_CFG_SWAP_M32 : pr.d.m <= 64 ? GZ_CFG_SWAP_M64
                                                                                            : GZ_CFG_SWAP_M128;
  const CfgShape* sp = shape_of(config);
  if (!sp || !sp->swap) return GZ_ERR_UNSUPPORTED;
  const CfgShape& s = *sp;
  if (!shape_fits(pr, s)) return GZ_ERR_UNSUPPORTED;
  gz_plan_info info;
  fill_info(pr, config, sd->sm_count, &info);
  if (!info.split_k) return GZ_ERR_UNSUPPORTED;  // a single K block in total: nothing to share
  constexpr size_t kStatusBytes = 256;
  if ((size_t)info.workspace_bytes + kStatusBytes > (size_t)GZ_STATIC_SCRATCH_BYTES) {
    char buf[160];
    std::snprintf(buf, sizeof(buf), "static scratch too small: this problem needs %lld bytes, the library holds %u",
                  (long long)info.workspace_bytes + (long long)kStatusBytes, (unsigned)GZ_STATIC_SCRATCH_BYTES);
    g_last_cuda_error = buf;
    return GZ_ERR_TOO_LARGE;
  }
  const KernelEntry entry = entry_for(pr.d.in_type, pr.d.out_type, config);
  if (!entry.launch) return GZ_ERR_UNSUPPORTED;
  if (!cuda_ok(entry.attr(), "cudaFuncSetAttribute(max dynamic shared memory)")) return GZ_ERR_CUDA;

  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  unsigned char* base = static_cast<unsigned char*>(sd->ptr);
  const size_t ws_bytes = (size_t)info.workspace_bytes;
  gz::GemmParams p;
  std::memset(&p, 0, sizeof(p));
  build_operand(&p.a, pr.b_mn_major, 128, pr.in_size);
  build_operand(&p.b, pr.a_mn_major, s.bn, pr.in_size);
  p.grid.tiles_m = (uint32_t)cdiv(pr.d.n, 128);
  p.grid.tiles_n = (uint32_t)cdiv(pr.d.m, s.bn);
  p.grid.group_m = 16;
  p.grid.num_tiles = p.grid.tiles_m * p.grid.tiles_n;
  p.tail_first = p.grid.num_tiles;
  p.tail_parts = 1;
  p.virt_tiles = p.grid.num_tiles;
  p.m = (uint32_t)pr.d.n;
  p.n = (uint32_t)pr.d.m;
  p.k = (uint32_t)pr.d.k;
  p.bk = 128u / pr.in_size;
  p.k_blocks = (uint32_t)cdiv(pr.d.k, p.bk);
  p.idesc = build_idesc(pr, s);
  p.epilogue_tma = 0;
  p.ldc = pr.d.ldc;
  p.ldd = pr.d.ldd;
  p.tune = gz::TUNE_K_STAGGER;  // as gz_gemm_plan_create does for skinny problems (same summation order)
  p.test_flags = (pr.d.flags & GZ_FLAG_TEST_WITHHOLD_ACC_READY) ? 1u : 0u;
  p.wait_limit_ns = pr.d.wait_limit_ns;
  p.alpha_f = af;
  p.beta_f = bf;
  p.alpha_i = ai;
  p.beta_i = bi;
  p.c = beta_zero ? nullptr : c;
  p.d = d;
  p.split_k = 1;
  p.max_contrib = (uint32_t)info.reserved;
  p.total_kb = (unsigned long long)p.grid.num_tiles * p.k_blocks;
  const size_t counter_bytes = (size_t)p.grid.num_tiles * 4;
  p.ws = reinterpret_cast<float*>(base);
  p.counters = reinterpret_cast<int*>(base + (ws_bytes - counter_bytes));
  p.status = reinterpret_cast<uint32_t*>(base + (GZ_STATIC_SCRATCH_BYTES - kStatusBytes));
  // The array keeps whatever the last call left in it.  The partial sums are always written before
  // they are read; the arrival counters must start at zero (a launch that gave up on a bounded wait
  // may have left some behind).  The status words are NOT cleared here: they start at zero when the
  // library image is loaded, keep the first failure until gz_static_last_device_status reads (and
  // clears) them, so a timeout cannot be lost under the next call.
  if (!cuda_ok(cudaMemsetAsync(p.counters, 0, counter_bytes, stream), "clear arrival counters"))
    return GZ_ERR_CUDA;

  CUtensorMap ta, tb;
  const uint32_t bk = p.bk;
  auto encode_input = [&](CUtensorMap* tm, const void* ptr, bool mn_major, int64_t rows, int64_t ld,
                          const gz::OperandDesc& od) {
    if (!mn_major)
      return encode_2d(tm, pr.d.in_type, ptr, (uint64_t)pr.d.k, (uint64_t)rows, (uint64_t)ld * pr.in_size, bk,
                       od.box_mn, true);
    return encode_2d(tm, pr.d.in_type, ptr, (uint64_t)rows, (uint64_t)pr.d.k, (uint64_t)ld * pr.in_size,
                     od.box_mn, bk, true, pr.in_size == 4);
  };
  if (!encode_input(&ta, b, pr.b_mn_major, pr.d.n, pr.d.ldb, p.a) ||
      !encode_input(&tb, a, pr.a_mn_major, pr.d.m, pr.d.lda, p.b))
    return GZ_ERR_CUDA;
  if (!cuda_ok(entry.launch(ta, tb, ta, p, info.grid, stream), "kernel launch")) return GZ_ERR_CUDA;
  return GZ_OK;
}

extern "C" GZ_API gz_status gz_static_last_device_status(int32_t device, void* stream_v, uint32_t detail[4]) {
  StaticScratchDevice* sd = nullptr;
  gz_status st = static_scratch_setup(device, &sd);
  if (st != GZ_OK) return st;
  DeviceGuard guard(device);
  if (!guard.ok()) return GZ_ERR_CUDA;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  constexpr size_t kStatusBytes = 256;
  unsigned char* words = static_cast<unsigned char*>(sd->ptr) + (GZ_STATIC_SCRATCH_BYTES - kStatusBytes);
  uint32_t h[4] = {0, 0, 0, 0};
  if (!cuda_ok(cudaStreamSynchronize(stream), "cudaStreamSynchronize") ||
      !cuda_ok(cudaMemcpy(h, words, sizeof(h), cudaMemcpyDeviceToHost), "read status"))
    return GZ_ERR_CUDA;
  if (detail) std::memcpy(detail, h, sizeof(h));
  if (h[0] != 0) {
    (void)cudaMemset(words, 0, sizeof(h));
    return h[0] == gz::STORE_OUT_OF_BOUNDS ? GZ_ERR_DEBUG_CHECK : GZ_ERR_DEVICE_TIMEOUT;
  }
  return GZ_OK;
}

// ------------------------------------------------------------------ K-sharded GEMM (multi-GPU)
#include "ksharded.cuh"
