// Persistent, warp-specialised tcgen05 GEMM for sm_100a:
//   D = alpha * A * B + beta * C
//
// This kernel takes the place of the three mma.sync kernels of the reference
// (nvidia/kernels/sm_80/bf16_mma_gemm.cuh:16-265, fp16_mma_gemm.cuh:14-305,
// tf32_mma_gemm.cuh:15-260) and of the s8 contract of
// intel/kernels/xe_gemm_s8_s8_s32_m8k16.hpp:17-77.  Same outer shape as those
// (persistent CTAs, multi-stage operand ring, fused alpha/beta epilogue,
// next tile's loads overlapping this tile's epilogue), different machinery:
//
//   warps 0, 6  one lane of each issues TMA tile loads (128-byte-swizzled boxes;
//               warp 0 the A tile, warp 6 the B tile) into a STAGES-deep
//               shared-memory ring; completion is counted in bytes on the
//               stage's "full" mbarrier.
//   warp 1      allocates TMEM; one lane (of the leader CTA when two CTAs share
//               a tile) issues tcgen05.mma from shared-memory descriptors into
//               one of two TMEM accumulators and commits each stage back to its
//               "empty" mbarrier.
//   warps 2..5  (and 7..10 when MB == 2)
//               epilogue: tcgen05.ld the finished accumulator (each warp owns
//               the 32 TMEM lanes of its warp_id % 4 quadrant), apply
//               alpha/beta in fp32 (int32 for s8), cast, and either stage rows
//               in swizzled shared memory for a TMA store or store directly.
//
// With one 128-row block of A per CTA (MB == 1) the second accumulator lets the
// epilogue of tile i run under the main loop of tile i+1.  With two blocks per
// CTA (MB == 2: a CTA pair covers 512 x 256 outputs) the two accumulators are
// the two row blocks of one tile: every B stage feeds twice as many MMAs, so a
// quarter less data moves from L2 to shared memory per flop.  That pays once the
// part runs at its power limit, where data movement is paid for in clock
// frequency.  The price is that the tensor pipe idles from the end of a tile
// until accumulator 0 is free again, so that hand-over is kept short: eight
// epilogue warps (two per TMEM lane quadrant, half of the columns each) copy
// their share to registers and give the accumulator back before storing
// anything, and the MMA warp starts the next tile with row block 0 alone on
// the first stages while accumulator 1 is still being copied.
// No cluster-multicast load is used anywhere: with CTAS == 2 each CTA of the
// pair loads its own rows of A and its own half of the B tile.
//
// Every wait on an mbarrier is bounded (Params::wait_limit_ns).  When a wait
// expires the waiter records a code in Params::status, raises a CTA-wide abort
// flag that all roles poll, and every role falls through to the common
// teardown, which still frees TMEM.
#ifndef GZ_SM100_GEMM_CUH
#define GZ_SM100_GEMM_CUH

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <type_traits>

#include "ptx.cuh"
#include "tile_sched.h"

namespace gz {

// How one operand tile is fetched by TMA and described to tcgen05.mma.
struct OperandDesc {
  uint32_t boxes;      // TMA boxes per stage per CTA
  uint32_t box_bytes;  // bytes one box deposits in shared memory
  uint32_t box_mn;     // extent of one box along the M (or N) dimension, in elements
  uint32_t mn_major;   // 0: K contiguous in memory (coords {k, mn}); 1: M/N contiguous ({mn, k})
  uint32_t desc_lo;    // shared-memory descriptor bits 16..31 (leading byte offset >> 4) << 16
  uint32_t desc_hi;    // bits 32..63: stride byte offset >> 4, version 1, 128B swizzle
  uint32_t k_step16;   // descriptor start-address advance (bytes >> 4) per MMA K step
  uint32_t broadcast;  // batched problems: 1 = every problem of the batch reads the same matrix
};

// Codes written to status[0] when a bounded wait expires.
enum WaitCode : uint32_t {
  WAIT_OK = 0,
  WAIT_PRODUCER_EMPTY = 1,
  WAIT_MMA_FULL = 2,
  WAIT_MMA_TMEM_EMPTY = 3,
  WAIT_EPILOGUE_TMEM_FULL = 4,
  WAIT_MMA_DRAIN = 5
};
// Written to status[0] by a debug build (GZ_BOUNDS_CHECK) when an epilogue store would have left
// the output matrix; status[1] = block, status[2] = row, status[3] = column of the refused store.
constexpr uint32_t STORE_OUT_OF_BOUNDS = 32;

struct GemmParams {
  OperandDesc a, b;
  TileGrid grid;
  uint32_t m, n, k;
  uint32_t k_blocks;  // ceil(k / elements per 128 bytes)
  uint32_t bk;        // K elements per stage
  uint32_t idesc;     // tcgen05 instruction descriptor
  uint32_t epilogue_tma;
  uint32_t c_vec_ok, d_vec_ok;  // 16-byte vector access to C / D rows is legal
  uint32_t test_flags;          // bit 0: MMA warp withholds the accumulator-ready signal
  float alpha_f, beta_f;
  int32_t alpha_i, beta_i;
  int64_t ldc, ldd;
  // Batched problems: tile indices run over batch * grid.num_tiles; problem i of the batch uses
  // coordinate i of the tensor maps' third dimension and C + i * stride_c, D + i * stride_d.
  int64_t stride_c, stride_d;  // elements
  const void* c;
  void* d;
  uint32_t* status;  // 4 words in global memory
  uint64_t wait_limit_ns;
  // Tail splitting (whole-tile mode only): tiles [tail_first, num_tiles) — the ones that would form a
  // last, mostly empty wave — are each cut into tail_parts column strips of BN / tail_parts columns,
  // so that the last wave is short instead of sparse.  virt_tiles counts whole tiles plus strips.
  uint32_t tail_first, tail_parts, virt_tiles;
  uint32_t idesc_tail;  // instruction descriptor with N = BN / tail_parts
  // Split-K work distribution (0 = whole tiles, dealt round-robin).  When set, the K blocks of all
  // tiles form one line that is cut into equal contiguous ranges, one per CTA; a tile whose K range
  // is shared by several CTAs is finished by whichever of them arrives last (see the epilogue).
  uint32_t split_k;
  uint32_t max_contrib;          // workspace slots per tile
  unsigned long long total_kb;   // num_tiles * k_blocks
  float* ws;                     // [num_tiles][max_contrib][BN/4][128] float4 partial accumulators (fp32 or int32 bits)
  int* counters;                 // [num_tiles], zero between launches
  // Scattered output (0 = off): output columns [o * scatter_cols, (o + 1) * scatter_cols) are written
  // to the matrix at scatter_ptrs[o] (row pitch ldd, column index relative to the block) instead
  // of d.  The pointers may be peer-GPU memory: a K-sharded GEMM pushes each column block of its
  // partial sums straight to the GPU that owns the block.  Direct-store epilogue only.
  uint32_t scatter_cols;
  void* scatter_ptrs[8];
  // Completion signal (signal_count == 0: off).  The CTA that leaves the kernel last, after every
  // CTA's output stores have been fenced system-wide, writes signal_value to signal_ptrs[0 ..
  // signal_count): the K-sharded GEMM tells every owner "my partial sums are in your memory" from
  // inside the GEMM instead of from a second launch.  signal_counter: one word, zero between launches.
  uint32_t signal_count, signal_value;
  uint32_t* signal_ptrs[8];
  uint32_t* signal_counter;
  // Optional epilogue terms (floating-point outputs only), applied in fp32:
  //   D = act(alpha * row_scale[i] * col_scale[j] * acc + beta * C + bias[j])
  // epi_flags != 0 says that at least one of them is present (bit 0 bias, 1 row_scale,
  // 2 col_scale, 3 activation); the kernel then takes its slice-by-slice epilogue (the terms,
  // above all the activations, are too much code to unroll over a warp's whole share).
  uint32_t epi_flags;
  uint32_t act;  // 0 none, 1 relu, 2 gelu (erf), 3 gelu (tanh), 4 silu
  const float* bias;
  const float* row_scale;
  const float* col_scale;
  // Scheduling switches set by the plan (see TUNE_* below).
  uint32_t tune;
  // Die-aware tile order (die_tickets == null: off).  A B200 is two dies, each with its own half
  // of the L2; a line that the SMs of both dies read crosses the die-to-die link.  With the order
  // on, the CTA pairs of one die take neighbouring tiles of each wave: a pair looks up the die of
  // its SM (die_of_sm, measured once per device by the plan), draws a ticket from that die's
  // counter, and numbers itself from the bottom (die 0) or from the top (die 1) of [0, pairs).  Every
  // pair draws exactly one ticket, so the numbers are a permutation wherever the hardware placed
  // the CTAs: placement decides locality, never results.  The last pair to leave clears the
  // counters.  die_tickets: 4 words (arrived on die 0, arrived on die 1, left, unused), zero
  // between launches; two launches that overlap on the GPU must not share them.
  uint32_t* die_tickets;
  uint8_t die_of_sm[160];
  // Optional stall counters and timeline, PROF_WORDS = 24 words per CTA (null = off):
  //  [0] A producer: clocks waiting for a free stage   [1] A producer: total clocks
  //  [2] MMA: clocks waiting for operand data          [3] MMA: clocks waiting for a free accumulator
  //  [4] MMA: total clocks                             [5] epilogue warp 2: clocks waiting for an accumulator
  //  [6] epilogue warp 2: total clocks                 [7] MMA: elapsed nanoseconds (globaltimer)
  //  [8] A producer: clocks issuing copies               [9] MMA: clocks issuing MMAs and commits
  //  [10] B producer: clocks waiting for a free stage   [11] B producer: clocks issuing copies
  //  [12] epilogue warp 2: clocks parking split-K partial sums (two-row-block tiles: clocks copying
  //       accumulators to registers)
  //  [13] MMA: clocks waiting for the second accumulator of a two-row-block tile (part of [3])
  //  [14] clocks from kernel entry to the end of set-up   [15] clocks from kernel entry to exit
  // Words 16..23 are a timeline in nanoseconds of the global timer (comparable between the CTAs of
  // one launch and between consecutive launches):
  //  [16] kernel entry                      [17] set-up done and dependencies of the launch satisfied
  //  [18] MMA: first operand stage landed   [19] MMA: last MMA of the CTA's last tile issued
  //  [20] epilogue warp 2: last accumulator ready   [21] its last output stores issued
  //  [22] shared memory of those stores read out (TMA-store epilogue; else = [21])   [23] kernel exit
  // Only kernels instantiated with PROF = true write them; the buffer holds PROF_WORDS words per CTA.
  unsigned long long* prof;
};

constexpr uint32_t PROF_WORDS = 24;

enum : uint32_t {
  // Tiles start their K range at different K blocks and wrap around.  Set by the plan for skinny
  // (weight-streaming) problems: all CTAs walking K in step read addresses that differ only by
  // multiples of the row pitch, which loads the HBM channels unevenly (measured: 24.5 -> 23.4 us at
  // M = 16, 26.5 -> 24.7 us at M = 128, N = 14336, K = 4096).  The order in which a tile's K blocks
  // are summed then depends on the tile index, which is why it is not used where results are
  // expected to be bitwise independent of the tile shape.
  TUNE_K_STAGGER = 2u,
};

// SWAP_: the roles of the operands are exchanged.  The 128-row side of the MMA (TMEM lanes) walks N
// and carries B; the narrow side (BN = 16..128 TMEM columns) carries the few rows of A.  Used for
// skinny problems (M <= 128), where a 128-row A tile would be mostly padding: every byte a stage
// loads is then a useful byte of B, which is what such HBM-bound shapes need.  The accumulator
// holds the transpose of the output tile; the epilogue stores it straight to global memory.
template <ptx::Kind KIND_, typename TOut_, int BN_, int CTAS_, int STAGES_, bool SWAP_ = false, int MB_ = 1>
struct GemmCfg {
  static constexpr ptx::Kind KIND = KIND_;
  static constexpr bool SWAP = SWAP_;
  using TOut = TOut_;
  static constexpr int BN = BN_;        // tile columns (= MMA N)
  static constexpr int CTAS = CTAS_;    // CTAs sharing one tile (1 or 2)
  static constexpr int STAGES = STAGES_;
  static constexpr int MB = MB_;                 // 128-row blocks of A per CTA (1 or 2)
  static constexpr int BM = 128 * MB;            // tile rows per CTA
  static constexpr int BN_CTA = BN / CTAS;       // B rows (tile columns) each CTA loads
  static constexpr int A_BYTES = BM * 128;       // one stage of A: BM rows x 128 bytes
  static constexpr int B_BYTES = BN_CTA * 128;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  // Epilogue warps: one per TMEM lane quadrant, or two (each taking half of the tile's columns)
  // where a half is at least one 128-byte box wide for every output type.
  static constexpr int EPI_WARPS = (!SWAP && BN >= 128) ? 8 : 4;
  static constexpr int STAGING_WARP_BYTES = SWAP ? 0 : 4096;  // one 32-row x 128-byte box per warp
  static constexpr int STAGING_BYTES = EPI_WARPS * STAGING_WARP_BYTES;
  static constexpr int BAR_BYTES = 256;
  static constexpr int TMEM_COLS = 2 * BN;  // two accumulators (MB == 2: one per row block)
  static constexpr int THREADS = 96 + 32 * EPI_WARPS;  // 2 producer warps, 1 MMA warp, 4 or 8 epilogue warps
  static constexpr int SMEM_BYTES = 1024 + STAGES * STAGE_BYTES + STAGING_BYTES + BAR_BYTES;
  static_assert(BN % 16 == 0 && BN >= 16 && BN <= 256, "tile N");
  static_assert(!SWAP || (CTAS == 1 && BN <= 128), "swapped tiles are single-CTA and narrow");
  static_assert(MB == 1 || (MB == 2 && !SWAP), "one or two row blocks per CTA");
  static_assert(TMEM_COLS == 32 || TMEM_COLS == 64 || TMEM_COLS == 128 || TMEM_COLS == 256 || TMEM_COLS == 512,
                "TMEM allocation must be a power of two");
  static_assert(8 * (2 * STAGES + 5) + 16 <= BAR_BYTES, "barrier area");
  static_assert(STAGE_BYTES % 1024 == 0, "stage must keep 1024-byte alignment");
};

namespace detail {

struct Abort {
  uint32_t* flag;  // CTA-shared
  uint32_t* status;
  uint64_t limit_ns;
};

__device__ __forceinline__ bool aborted(const Abort& ab) {
  return *reinterpret_cast<volatile uint32_t*>(ab.flag) != 0;
}

static __device__ __noinline__ void record_timeout(const Abort& ab, uint32_t code, uint32_t tile,
                                            uint32_t kb) {
  if (atomicCAS(ab.status, 0u, code) == 0u) {
    ab.status[1] = blockIdx.x;
    ab.status[2] = tile;
    ab.status[3] = kb;
    __threadfence();
  }
  *reinterpret_cast<volatile uint32_t*>(ab.flag) = 1u;
}

// Wait for `bar` to complete the phase of parity `parity`, for at most
// ab.limit_ns.  Returns false if the CTA is aborting.
template <bool CLUSTER_ACQUIRE = false>
__device__ __forceinline__ bool wait(uint32_t bar, uint32_t parity, const Abort& ab, uint32_t code,
                                     uint32_t tile, uint32_t kb) {
  auto poll = [&]() {
    if constexpr (CLUSTER_ACQUIRE) return ptx::mbar_try_wait_cluster(bar, parity);
    else return ptx::mbar_try_wait(bar, parity);
  };
  if (poll()) return true;
  // Slow path.  The timer is read only every 256 failed polls (each poll may
  // itself sleep for a hardware-defined slice), so the common short wait costs
  // nothing but polls; the limit counts from the first timer read.
  uint64_t t0 = 0;
  uint32_t spins = 0;
  for (;;) {
    if (poll()) return true;
    if ((++spins & 255u) == 0u) {
      if (aborted(ab)) return false;
      const uint64_t now = ptx::globaltimer_ns();
      if (t0 == 0) {
        t0 = now;
      } else if (now - t0 > ab.limit_ns) {
        record_timeout(ab, code, tile, kb);
        return false;
      }
    }
  }
}

// The sequence of (tile, K-block range) pieces one CTA (or CTA pair) works through.  Every role
// of the CTA constructs the same iterator and so sees the same sequence.
struct WorkIter {
  uint32_t k_blocks, virt_tiles, tail_first, tail_parts, bn, step, next_tile;
  uint32_t col_off, cols;  // column strip of the tile the current piece covers
  unsigned long long cur, end;
  bool split;
  __device__ __forceinline__ WorkIter(const GemmParams& p, uint32_t cluster, uint32_t num_clusters,
                                      uint32_t tile_cols)
      : k_blocks(p.k_blocks), virt_tiles(p.virt_tiles), tail_first(p.tail_first),
        tail_parts(p.tail_parts), bn(tile_cols), step(num_clusters), next_tile(cluster), col_off(0),
        cols(tile_cols), cur(0), end(0), split(p.split_k != 0u) {
    if (split) {
      cur = static_cast<unsigned long long>(cluster) * p.total_kb / num_clusters;
      end = static_cast<unsigned long long>(cluster + 1u) * p.total_kb / num_clusters;
    }
  }
  __device__ __forceinline__ bool next(uint32_t& tile, uint32_t& kb_lo, uint32_t& kb_hi) {
    if (!split) {
      if (next_tile >= virt_tiles) return false;
      if (next_tile < tail_first) {
        tile = next_tile;
        col_off = 0;
        cols = bn;
      } else {
        const uint32_t sub = next_tile - tail_first;
        tile = tail_first + sub / tail_parts;
        cols = bn / tail_parts;
        col_off = (sub % tail_parts) * cols;
      }
      kb_lo = 0;
      kb_hi = k_blocks;
      next_tile += step;
      return true;
    }
    if (cur >= end) return false;
    tile = static_cast<uint32_t>(cur / k_blocks);
    kb_lo = static_cast<uint32_t>(cur - static_cast<unsigned long long>(tile) * k_blocks);
    const unsigned long long left = end - cur;
    kb_hi = (left < k_blocks - kb_lo) ? kb_lo + static_cast<uint32_t>(left) : k_blocks;
    cur += kb_hi - kb_lo;
    return true;
  }
};

// Index of the CTA whose contiguous range contains K-block unit `u` (inverse of the cut above).
__device__ __forceinline__ uint32_t split_owner(unsigned long long u, unsigned long long total,
                                                uint32_t parts) {
  return static_cast<uint32_t>(((u + 1ull) * parts + total - 1ull) / total - 1ull);
}

template <typename TOut>
struct OutTraits;
template <>
struct OutTraits<float> {
  static constexpr bool INT = false;
  __device__ static float to_f(float v) { return v; }
};
template <>
struct OutTraits<__half> {
  static constexpr bool INT = false;
  __device__ static float to_f(__half v) { return __half2float(v); }
};
template <>
struct OutTraits<__nv_bfloat16> {
  static constexpr bool INT = false;
  __device__ static float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
};
template <>
struct OutTraits<int32_t> {
  static constexpr bool INT = true;
};

// Pack two fp32 values into one 32-bit word of two 16-bit outputs (low = first).
template <typename TOut>
__device__ __forceinline__ uint32_t pack2(float lo, float hi);
template <>
__device__ __forceinline__ uint32_t pack2<__half>(float lo, float hi) {
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}
template <>
__device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

// The two 16-bit values of one 32-bit word (low = first) as fp32.
template <typename TOut>
__device__ __forceinline__ float2 unpack2(uint32_t w);
template <>
__device__ __forceinline__ float2 unpack2<__half>(uint32_t w) {
  return __half22float2(*reinterpret_cast<const __half2*>(&w));
}
template <>
__device__ __forceinline__ float2 unpack2<__nv_bfloat16>(uint32_t w) {
  return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xFFFF0000u));
}

// An accumulator word as fp32: int32 accumulators (kind::i8) are converted, the rest reinterpreted.
template <bool ACC_INT>
__device__ __forceinline__ float acc_as_float(uint32_t v) {
  if constexpr (ACC_INT) return static_cast<float>(static_cast<int32_t>(v));
  else return __uint_as_float(v);
}

// erf to about 2e-7 absolute (Abramowitz & Stegun 7.1.26: 1 - (a1 t + ... + a5 t^5) exp(-z^2),
// t = 1 / (1 + p z), |error| <= 1.5e-7 before rounding) in a dozen instructions.  GELU multiplies it
// by x / 2, and erf is exactly +-1 in fp32 beyond |z| = 4, so the activation stays well inside fp32
// accuracy; the library erff costs about three times as many instructions, and this runs once per
// output element in the epilogue of the last tile, which nothing overlaps.
// 1 / x to within an ulp or two in one instruction (the correctly rounded reciprocal costs six).
__device__ __forceinline__ float rcp_approx(float x) {
  float r;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}

__device__ __forceinline__ float erf_fast(float z) {
  const float az = fabsf(z);
  // The correctly rounded reciprocal on purpose: with rcp_approx here the epilogue of a tile is
  // 40 % shorter, but the main loop that runs beside it loses 7 % (measured at bf16 2048x14336x4096
  // with bias + GELU: MMA issue 215 -> 271 clocks per K block, 1.069x the plain GEMM instead of
  // 1.045x); the tanh form and SiLU below do not show that and use the approximation.
  const float t = __frcp_rn(fmaf(0.3275911f, az, 1.0f));
  float poly = fmaf(1.061405429f, t, -1.453152027f);
  poly = fmaf(poly, t, 1.421413741f);
  poly = fmaf(poly, t, -0.284496736f);
  poly = fmaf(poly, t, 0.254829592f);
  const float e = __expf(-az * az);
  return copysignf(fmaf(-poly * t, e, 1.0f), z);
}

__device__ __forceinline__ float activate(float x, uint32_t act) {
  switch (act) {
    case 1: return fmaxf(x, 0.0f);
    case 2: return 0.5f * x * (1.0f + erf_fast(x * 0.70710678118654752f));
    case 3: {
      // 0.5 x (1 + tanh u) with tanh u = 1 - 2 / (e^(2u) + 1), i.e. x (1 - 1 / (e^(2u) + 1)): one
      // exponential and one reciprocal instead of the library tanhf, to about 2e-7 absolute.
      const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
      return x - x * rcp_approx(__expf(2.0f * u) + 1.0f);
    }
    case 4: return x * rcp_approx(1.0f + __expf(-x));
    default: return x;
  }
}

// The optional terms around one element: epi_scale() takes alpha * acc, epi_finish() takes
// alpha * rs * cs * acc + beta * c.
__device__ __forceinline__ float epi_scale(const GemmParams& p, float f, uint32_t row, uint32_t col) {
  if (p.row_scale) f *= __ldg(p.row_scale + row);
  if (p.col_scale) f *= __ldg(p.col_scale + col);
  return f;
}
__device__ __forceinline__ float epi_finish(const GemmParams& p, float f, uint32_t col) {
  if (p.bias) f += __ldg(p.bias + col);
  return activate(f, p.act);
}

// Debug builds (compiled with -DGZ_BOUNDS_CHECK) check every plain global store of the epilogue
// before it is made: the coordinates must lie inside the output matrix (rows x cols of this
// problem of the batch).  A store that fails the check is recorded and skipped, never made; TMA
// stores need no check, the hardware clips them to the tensor map.  Release builds compile the
// check away.
#if defined(GZ_BOUNDS_CHECK)
static __device__ __noinline__ bool store_in_bounds(const GemmParams& p, uint32_t row, uint32_t col, uint32_t ncols,
                                                    uint32_t rows, uint32_t cols) {
  if (row < rows && col < cols && ncols <= cols - col) return true;
  if (atomicCAS(p.status, 0u, STORE_OUT_OF_BOUNDS) == 0u) {
    p.status[1] = blockIdx.x;
    p.status[2] = row;
    p.status[3] = col;
    __threadfence();
  }
  return false;
}
#define GZ_STORE_OK(p, row, col, ncols, rows, cols) detail::store_in_bounds(p, row, col, ncols, rows, cols)
#else
#define GZ_STORE_OK(p, row, col, ncols, rows, cols) true
#endif

// alpha * acc + beta * c for one 32-column slice of one row.
//   v[32]     in:  raw accumulator words;  out: packed output words (32 * sizeof(TOut) / 4 used)
//   crow      pointer to C(row, col0) (only dereferenced when beta != 0 and row_ok)
//   ncols     valid columns in this slice (1..32)
//   row, col0 output coordinates of the slice (for the optional per-row / per-column terms)
template <typename TOut, bool ACC_INT>
__device__ __forceinline__ void epilogue_math(uint32_t (&v)[32], const GemmParams& p,
                                              const TOut* crow, bool row_ok, uint32_t ncols,
                                              uint32_t row, uint32_t col0) {
  using Tr = OutTraits<TOut>;
  if constexpr (Tr::INT) {
    const uint32_t alpha = static_cast<uint32_t>(p.alpha_i);
    const uint32_t beta = static_cast<uint32_t>(p.beta_i);
    if (beta != 0u && row_ok) {
      if (ncols == 32 && p.c_vec_ok) {
        const uint4* c4 = reinterpret_cast<const uint4*>(crow);
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          const uint4 cv = c4[q];
          v[4 * q + 0] = alpha * v[4 * q + 0] + beta * cv.x;
          v[4 * q + 1] = alpha * v[4 * q + 1] + beta * cv.y;
          v[4 * q + 2] = alpha * v[4 * q + 2] + beta * cv.z;
          v[4 * q + 3] = alpha * v[4 * q + 3] + beta * cv.w;
        }
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const uint32_t cv = (static_cast<uint32_t>(i) < ncols) ? static_cast<uint32_t>(crow[i]) : 0u;
          v[i] = alpha * v[i] + beta * cv;
        }
      }
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = alpha * v[i];
    }
  } else {
    const float alpha = p.alpha_f;
    const float beta = p.beta_f;
    float f[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) f[i] = alpha * acc_as_float<ACC_INT>(v[i]);
    // Optional terms.  The per-column vectors are fetched once per slice (lane l takes column
    // col0 + l) and handed round by shuffles, which the whole warp executes.
    const bool epi = p.epi_flags != 0u;
    const uint32_t lane = ptx::lane_id();
    const bool col_ok = lane < ncols;
    if (epi) {
      const float rs = (p.row_scale && row_ok) ? __ldg(p.row_scale + row) : 1.0f;
      const float my_cs = (p.col_scale && col_ok) ? __ldg(p.col_scale + col0 + lane) : 1.0f;
      if (p.row_scale) {
#pragma unroll
        for (int i = 0; i < 32; ++i) f[i] *= rs;
      }
      if (p.col_scale) {
#pragma unroll
        for (int i = 0; i < 32; ++i) f[i] *= __shfl_sync(0xFFFFFFFFu, my_cs, i);
      }
    }
    if (beta != 0.0f && row_ok) {
      if (ncols == 32 && p.c_vec_ok) {
        constexpr int PER16 = 16 / sizeof(TOut);  // elements per 16-byte load
        const uint4* c4 = reinterpret_cast<const uint4*>(crow);
#pragma unroll
        for (int q = 0; q < 32 / PER16; ++q) {
          const uint4 cv = c4[q];
          const TOut* ce = reinterpret_cast<const TOut*>(&cv);
#pragma unroll
          for (int e = 0; e < PER16; ++e)
            f[q * PER16 + e] = fmaf(beta, Tr::to_f(ce[e]), f[q * PER16 + e]);
        }
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if (static_cast<uint32_t>(i) < ncols) f[i] = fmaf(beta, Tr::to_f(crow[i]), f[i]);
      }
    }
    if (epi) {
      if (p.bias) {
        const float my_bias = col_ok ? __ldg(p.bias + col0 + lane) : 0.0f;
#pragma unroll
        for (int i = 0; i < 32; ++i) f[i] += __shfl_sync(0xFFFFFFFFu, my_bias, i);
      }
      // one activation's code per pass over the slice, not five per element
      switch (p.act) {
        case 1:
#pragma unroll
          for (int i = 0; i < 32; ++i) f[i] = activate(f[i], 1);
          break;
        case 2:
#pragma unroll
          for (int i = 0; i < 32; ++i) f[i] = activate(f[i], 2);
          break;
        case 3:
#pragma unroll
          for (int i = 0; i < 32; ++i) f[i] = activate(f[i], 3);
          break;
        case 4:
#pragma unroll
          for (int i = 0; i < 32; ++i) f[i] = activate(f[i], 4);
          break;
        default: break;
      }
    }
    if constexpr (sizeof(TOut) == 4) {
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(f[i]);
    } else {
#pragma unroll
      for (int i = 0; i < 16; ++i) v[i] = pack2<TOut>(f[2 * i], f[2 * i + 1]);
    }
  }
}

// alpha * acc (+ beta * *c) for a single element (the swapped-operand epilogue).
template <typename TOut, bool HAS_BETA, bool ACC_INT>
__device__ __forceinline__ TOut epilogue_scalar(uint32_t acc, const GemmParams& p, const TOut* c, uint32_t row,
                                                uint32_t col) {
  using Tr = OutTraits<TOut>;
  if constexpr (Tr::INT) {
    uint32_t v = static_cast<uint32_t>(p.alpha_i) * acc;
    if constexpr (HAS_BETA) v += static_cast<uint32_t>(p.beta_i) * static_cast<uint32_t>(*c);
    return static_cast<int32_t>(v);
  } else {
    float f = p.alpha_f * acc_as_float<ACC_INT>(acc);
    if (p.epi_flags != 0u) f = epi_scale(p, f, row, col);
    if constexpr (HAS_BETA) f = fmaf(p.beta_f, Tr::to_f(*c), f);
    if (p.epi_flags != 0u) f = epi_finish(p, f, col);
    if constexpr (sizeof(TOut) == 4) return f;
    else if constexpr (std::is_same<TOut, __half>::value) return __float2half_rn(f);
    else return __float2bfloat16_rn(f);
  }
}

// The plain output path of a swapped tile (no C term, no epilogue vectors, floating-point output):
// accumulator lane = output column, accumulator column = output row; row i of the tile goes to
// dp + i * ldd.  Deliberately NOT inlined: the epilogue runs once per tile, long after anything
// else the warp executed, so it runs at the speed instructions can be fetched; the caller runs
// this once with store = false while it waits for its first accumulator (the loads read whatever
// tensor memory holds and nothing is stored), which leaves the code in the instruction caches.
template <typename TOut, int BN, bool ACC_INT>
__device__ __noinline__ void swapped_store_plain(uint32_t taddr, TOut* dp, long long ldd, uint32_t rows, float alpha,
                                                 bool store) {
#pragma unroll
  for (int sl = 0; sl < BN / 16; ++sl) {
    if (static_cast<uint32_t>(sl * 16) >= rows) break;
    uint32_t v[16];
    ptx::tmem_ld_32x16(taddr + sl * 16u, v);
    ptx::tmem_wait_ld();
    const uint32_t cnt = (rows - sl * 16u < 16u) ? (rows - sl * 16u) : 16u;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      if (static_cast<uint32_t>(i) >= cnt) break;  // uniform
      const float f = alpha * acc_as_float<ACC_INT>(v[i]);
      if (store) {
        TOut* const q = dp + static_cast<long long>(sl * 16 + i) * ldd;
        if constexpr (sizeof(TOut) == 4) *q = f;
        else if constexpr (std::is_same<TOut, __half>::value) *q = __float2half_rn(f);
        else *q = __float2bfloat16_rn(f);
      }
    }
  }
}

// Store one packed 32-column slice of one row straight to global memory.
template <typename TOut>
__device__ __forceinline__ void store_direct(const uint32_t (&v)[32], TOut* drow, uint32_t ncols,
                                             bool vec_ok) {
  constexpr int WORDS = 32 * sizeof(TOut) / 4;
  if (ncols == 32 && vec_ok) {
    uint4* d4 = reinterpret_cast<uint4*>(drow);
#pragma unroll
    for (int q = 0; q < WORDS / 4; ++q)
      d4[q] = make_uint4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
  } else {
    if constexpr (sizeof(TOut) == 4) {
      uint32_t* d32 = reinterpret_cast<uint32_t*>(drow);
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (static_cast<uint32_t>(i) < ncols) d32[i] = v[i];
    } else {
      uint16_t* d16 = reinterpret_cast<uint16_t*>(drow);
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (static_cast<uint32_t>(i) < ncols)
          d16[i] = static_cast<uint16_t>(v[i >> 1] >> (16 * (i & 1)));
    }
  }
}


// Address of output element (row, col); col must not be split from its 32-aligned neighbours by a
// scatter boundary (scatter_cols is a multiple of 32).
template <typename TOut>
__device__ __forceinline__ TOut* out_ptr(const GemmParams& p, uint32_t row, uint32_t col, uint32_t batch = 0) {
  if (p.scatter_cols == 0u)
    return static_cast<TOut*>(p.d) + static_cast<int64_t>(batch) * p.stride_d + static_cast<int64_t>(row) * p.ldd + col;
  const uint32_t owner = col / p.scatter_cols;
  return static_cast<TOut*>(p.scatter_ptrs[owner]) + static_cast<int64_t>(row) * p.ldd +
         (col - owner * p.scatter_cols);
}

// Write a staged 32-row x 128-byte box (rows 128-byte-swizzled, as a TMA store would read it) to
// the output with plain stores: per instruction eight lanes cover one row's 128 bytes, so every
// store instruction writes four whole 128-byte lines.  This is the store path when D cannot be
// described to TMA and when the output is scattered to peer GPUs, where 16-byte fragments of
// 32 different rows per instruction would waste the link.
template <typename TOut>
__device__ __forceinline__ void store_staged_box(const GemmParams& p, uint32_t stg, uint32_t lane, uint32_t row0,
                                                 uint32_t box_col, uint32_t batch) {
  constexpr uint32_t PER16 = 16 / sizeof(TOut);
  const uint32_t j = lane & 7u;
#pragma unroll
  for (uint32_t i = 0; i < 8; ++i) {
    const uint32_t r = i * 4u + (lane >> 3);
    uint4 v;
    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "r"(stg + r * 128u + ((j ^ (r & 7u)) << 4))
                 : "memory");
    if (row0 + r < p.m && GZ_STORE_OK(p, row0 + r, box_col + j * PER16, PER16, p.m, p.n))
      *reinterpret_cast<uint4*>(out_ptr<TOut>(p, row0 + r, box_col + j * PER16, batch)) = v;
  }
}

// alpha * acc (+ beta * c) for one full 32-column slice of one row, in place and without a second
// register array: on return x[0 .. 32 * sizeof(TOut) / 4) holds the packed outputs.  `crow` points
// at C(row, col0), 16-byte aligned; it is read only when HAS_BETA.
// The four scalars of the epilogue, for code that must not drag the whole parameter block along.
struct EpiScalars {
  float alpha_f, beta_f;
  int32_t alpha_i, beta_i;
};

template <typename TOut, bool HAS_BETA, bool ACC_INT, class P>
__device__ __forceinline__ void scale_slice_in_place(uint32_t (&x)[32], const P& p, const TOut* crow) {
  using Tr = OutTraits<TOut>;
  const uint4* c4 = reinterpret_cast<const uint4*>(crow);
  if constexpr (Tr::INT) {
    const uint32_t alpha = static_cast<uint32_t>(p.alpha_i);
    const uint32_t beta = static_cast<uint32_t>(p.beta_i);
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      uint4 cv = make_uint4(0u, 0u, 0u, 0u);
      if constexpr (HAS_BETA) cv = c4[q];
      x[4 * q + 0] = alpha * x[4 * q + 0] + beta * cv.x;
      x[4 * q + 1] = alpha * x[4 * q + 1] + beta * cv.y;
      x[4 * q + 2] = alpha * x[4 * q + 2] + beta * cv.z;
      x[4 * q + 3] = alpha * x[4 * q + 3] + beta * cv.w;
    }
  } else if constexpr (sizeof(TOut) == 4) {
    const float alpha = p.alpha_f, beta = p.beta_f;
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      float f0 = alpha * acc_as_float<ACC_INT>(x[4 * q + 0]), f1 = alpha * acc_as_float<ACC_INT>(x[4 * q + 1]);
      float f2 = alpha * acc_as_float<ACC_INT>(x[4 * q + 2]), f3 = alpha * acc_as_float<ACC_INT>(x[4 * q + 3]);
      if constexpr (HAS_BETA) {
        const uint4 cv = c4[q];
        f0 = fmaf(beta, __uint_as_float(cv.x), f0);
        f1 = fmaf(beta, __uint_as_float(cv.y), f1);
        f2 = fmaf(beta, __uint_as_float(cv.z), f2);
        f3 = fmaf(beta, __uint_as_float(cv.w), f3);
      }
      x[4 * q + 0] = __float_as_uint(f0);
      x[4 * q + 1] = __float_as_uint(f1);
      x[4 * q + 2] = __float_as_uint(f2);
      x[4 * q + 3] = __float_as_uint(f3);
    }
  } else {
    // Eight inputs (words 8q .. 8q+7) become four packed words (4q .. 4q+3): every word is read
    // before the slot it shares is written.
    const float alpha = p.alpha_f, beta = p.beta_f;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      uint4 cv = make_uint4(0u, 0u, 0u, 0u);
      if constexpr (HAS_BETA) cv = c4[q];
      const uint32_t cw[4] = {cv.x, cv.y, cv.z, cv.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float lo = alpha * acc_as_float<ACC_INT>(x[8 * q + 2 * e]);
        float hi = alpha * acc_as_float<ACC_INT>(x[8 * q + 2 * e + 1]);
        if constexpr (HAS_BETA) {
          const float2 cf = unpack2<TOut>(cw[e]);
          lo = fmaf(beta, cf.x, lo);
          hi = fmaf(beta, cf.y, hi);
        }
        x[4 * q + e] = pack2<TOut>(lo, hi);
      }
    }
  }
}

// The plain epilogue of one warp's share of a tile (no C term, no epilogue vectors, whole share
// inside the matrix, TMA store): copy NSL 32-column slices of the accumulator to registers, hand
// the accumulator back (arrive on `empty_bar`), then scale, pack, stage and store box by box.
// Not inlined, for the reason given at swapped_store_plain: a CTA with a single tile executes its
// epilogue exactly once, cold, with nothing to overlap it; the caller runs this once with
// live = false (no arrival, no store; it reads whatever tensor memory holds and writes only the
// warp's own staging box) before it waits for its first accumulator.
template <typename TOut, bool ACC_INT, int NSL, int CTAS>
__device__ __noinline__ void plain_tile_epilogue(uint32_t taddr, uint32_t stg, const void* tmap_d, int32_t col_w,
                                                 int32_t row0, int32_t bidx, EpiScalars sc, uint32_t empty_bar,
                                                 bool live) {
  constexpr int BOX_COLS = 128 / sizeof(TOut);
  constexpr int SLICES = BOX_COLS / 32;
  constexpr int WORDS = 32 * sizeof(TOut) / 4;
  const uint32_t lane = threadIdx.x & 31u;
  uint32_t v[NSL][32];
#pragma unroll
  for (int sl = 0; sl < NSL; ++sl) ptx::tmem_ld_32x32(taddr + sl * 32u, v[sl]);
  ptx::tmem_wait_ld();
  ptx::tc_fence_before_sync();
  __syncwarp();
  if (live && lane == 0) {
    if constexpr (CTAS == 2) ptx::mbar_arrive_cluster(empty_bar);
    else ptx::mbar_arrive(empty_bar);
  }
#pragma unroll
  for (int box = 0; box < NSL / SLICES; ++box) {
    // One staging box per warp: the store issued from it must have read it out.
    if (lane == 0) ptx::bulk_wait_group_read<0>();
    __syncwarp();
#pragma unroll
    for (int sl = 0; sl < SLICES; ++sl) {
      uint32_t(&x)[32] = v[box * SLICES + sl];
      scale_slice_in_place<TOut, false, ACC_INT>(x, sc, static_cast<const TOut*>(nullptr));
#pragma unroll
      for (int q = 0; q < WORDS / 4; ++q) {
        const uint32_t j = static_cast<uint32_t>(sl * (WORDS / 4) + q);
        const uint32_t addr = stg + lane * 128u + ((j ^ (lane & 7u)) << 4);
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(x[4 * q]), "r"(x[4 * q + 1]),
                     "r"(x[4 * q + 2]), "r"(x[4 * q + 3])
                     : "memory");
      }
    }
    ptx::fence_proxy_async_smem();
    __syncwarp();
    if (live && lane == 0) {
      ptx::tma_store_3d(tmap_d, stg, col_w + box * BOX_COLS, row0, bidx);
      ptx::bulk_commit_group();
    }
  }
}

}  // namespace detail

template <class Cfg, bool PROF = false>
__global__ void __launch_bounds__(Cfg::THREADS, 1)
sm100_gemm_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                  const __grid_constant__ CUtensorMap tm_d, const GemmParams p) {
  using TOut = typename Cfg::TOut;
  constexpr bool ACC_INT = Cfg::KIND == ptx::Kind::I8;  // int32 accumulators
  constexpr int CTAS = Cfg::CTAS;
  constexpr int STAGES = Cfg::STAGES;
  constexpr int BN = Cfg::BN;

  const long long kernel_t0 = PROF ? clock64() : 0;
  const uint64_t tl_entry = PROF ? ptx::globaltimer_ns() : 0;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = ptx::smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;  // 128B-swizzle atoms need 1024-byte alignment
  uint8_t* const smem = smem_raw + (base - raw_addr);

  const uint32_t staging_base = base + STAGES * Cfg::STAGE_BYTES;
  const uint32_t bars = staging_base + Cfg::STAGING_BYTES;
  uint8_t* const bars_ptr = smem + STAGES * Cfg::STAGE_BYTES + Cfg::STAGING_BYTES;
  auto full_bar = [&](uint32_t s) { return bars + 8u * s; };
  auto empty_bar = [&](uint32_t s) { return bars + 8u * (STAGES + s); };
  auto tmem_full_bar = [&](uint32_t b) { return bars + 8u * (2 * STAGES + b); };
  auto tmem_empty_bar = [&](uint32_t b) { return bars + 8u * (2 * STAGES + 2 + b); };
  const uint32_t drain_bar = bars + 8u * (2 * STAGES + 4);
  uint32_t* const tmem_slot = reinterpret_cast<uint32_t*>(bars_ptr + 8 * (2 * STAGES + 5));
  uint32_t* const abort_flag = tmem_slot + 1;
  uint32_t* const split_flag = tmem_slot + 2;  // epilogue: "this CTA finishes the tile"
  uint32_t* const order_slot = tmem_slot + 3;  // die-aware order: this CTA pair's number

  const uint32_t warp = threadIdx.x >> 5;
  const uint32_t lane = threadIdx.x & 31u;
  const uint32_t rank = (CTAS == 2) ? ptx::cluster_ctarank() : 0u;
  const uint32_t hw_cluster = (CTAS == 2) ? ptx::cluster_id_x() : blockIdx.x;
  const uint32_t num_clusters = (CTAS == 2) ? ptx::num_clusters_x() : gridDim.x;

  const detail::Abort ab{abort_flag, p.status, p.wait_limit_ns};

  // ------------------------------------------------------------ set-up
  // The producers need only the mbarriers, which warp 0 initialises itself; the tensor-memory
  // allocation concerns the MMA and epilogue warps.  So nobody waits for everybody: warp 0 releases
  // warp 6 through named barrier 2 and the rest through named barrier 3, which the MMA warp joins
  // after allocating, and the first loads are in flight while tensor memory is still being set up.
  // With a CTA pair every thread arrives at the cluster barrier as early as it can (warp 0 after
  // its initialisation, which is what the peer must not run ahead of) and waits on it only when
  // it is about to touch the peer.
  if (warp == 0) {
    // The descriptor fetches are the first thing on the path to the first operand bytes.
    if (lane == 31u) ptx::prefetch_tensormap(&tm_a);
    if (lane == 30u && p.epilogue_tma) ptx::prefetch_tensormap(&tm_d);
    for (uint32_t s = lane; s < STAGES; s += 32u) {
      ptx::mbar_init(full_bar(s), 2);  // one arrive.expect_tx per producer warp
      ptx::mbar_init(empty_bar(s), 1);
    }
    if (lane < 2u) {
      ptx::mbar_init(tmem_full_bar(lane), 1);
      ptx::mbar_init(tmem_empty_bar(lane), Cfg::EPI_WARPS * CTAS);  // one arrival per epilogue warp
    }
    if (lane == 2u) {
      ptx::mbar_init(drain_bar, 1);
      *abort_flag = 0u;
      *split_flag = 0u;
    }
    ptx::fence_mbar_init_cluster();
    __syncwarp();
    ptx::named_barrier_arrive(2, 64);
    ptx::named_barrier_arrive(3, Cfg::THREADS - 32);
    if constexpr (CTAS == 2) ptx::cluster_arrive_release();
  } else if (warp == 6) {
    if (lane == 0) ptx::prefetch_tensormap(&tm_b);
    if constexpr (CTAS == 2) ptx::cluster_arrive_release();
    ptx::named_barrier_sync(2, 64);
  } else {
    if constexpr (CTAS == 2) ptx::cluster_arrive_release();
    if (warp == 1) {
      ptx::tmem_alloc<CTAS>(ptx::smem_u32(tmem_slot), Cfg::TMEM_COLS);
      ptx::tmem_relinquish<CTAS>();
    }
    ptx::tc_fence_before_sync();
    ptx::named_barrier_sync(3, Cfg::THREADS - 32);
    ptx::tc_fence_after_sync();
  }
  if constexpr (CTAS == 2) ptx::cluster_wait_acquire();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);
  const long long setup_clocks = PROF ? clock64() - kernel_t0 : 0;

  // Everything above touched only this CTA's shared and tensor memory and the kernel's parameters,
  // so it may overlap the tail of the previous kernel of the stream.  The next kernel may start
  // its own set-up as soon as SMs come free.
  ptx::grid_launch_dependents();
  // Each role waits for the launch's dependencies itself, as late as it can: the producers after
  // they have worked out their first piece (index arithmetic and parameter reads, which miss the
  // constant cache in a fresh launch, then overlap the previous kernel's tail), the epilogue warps
  // before their first access to C or D, the MMA warp before its first bounded wait.  The ticket
  // draw of the die-aware order is a global-memory access, so such launches wait here.
  if (p.die_tickets != nullptr) ptx::grid_dependency_wait();

  // Which tiles this CTA (pair) takes: those of its hardware index, or, with the die-aware order,
  // those of the number it draws now (see GemmParams::die_tickets).
  uint32_t cluster = hw_cluster;
  if (p.die_tickets != nullptr) {
    if (rank == 0 && threadIdx.x == 0) {
      const uint32_t die = p.die_of_sm[ptx::smid() % 160u] & 1u;
      uint32_t r = atomicAdd(p.die_tickets + die, 1u);
      if (r >= num_clusters) r = num_clusters - 1u;  // counters were not zero: another launch shares them
      const uint32_t v = die == 0u ? r : num_clusters - 1u - r;
      *reinterpret_cast<volatile uint32_t*>(order_slot) = v;
      if constexpr (CTAS == 2) ptx::st_cluster_u32(ptx::mapa(ptx::smem_u32(order_slot), 1), v);
    }
    if constexpr (CTAS == 2) {
      ptx::cluster_arrive_release();
      ptx::cluster_wait_acquire();
    } else {
      __syncthreads();
    }
    cluster = *reinterpret_cast<volatile uint32_t*>(order_slot);
  }

  const uint32_t k_blocks = p.k_blocks;
  // What the teardown has to do besides freeing tensor memory, read now and kept in a register:
  // the teardown runs once, at the very end, where every parameter read is a constant-cache miss
  // that nothing overlaps.  Bit 0: completion signal, bit 1: die tickets, bit 2: timeline.
  uint32_t late_work = (p.signal_count != 0u ? 1u : 0u) | (p.die_tickets != nullptr ? 2u : 0u) |
                       ((PROF && p.prof != nullptr) ? 4u : 0u);
  asm volatile("" : "+r"(late_work));

  if (warp == 0 || warp == 6) {
    // ---------------------------------------------------------- TMA producers
    // Two producer warps, one per operand (warp 0: A, warp 6: B), because the
    // issue cost of a tensor copy is per instruction: split across two
    // instruction streams, neither limits the main loop.  Each whole warp walks
    // the loop (loop state stays warp-uniform); one elected lane issues.
    const bool is_b = warp == 6;
    const OperandDesc& od = is_b ? p.b : p.a;
    const void* const tmap = is_b ? static_cast<const void*>(&tm_b) : static_cast<const void*>(&tm_a);
    const uint32_t boxes = od.boxes, box_bytes = od.box_bytes, box_mn = od.box_mn;
    const bool mn_major = od.mn_major != 0u;
    const uint32_t my_bytes = is_b ? Cfg::B_BYTES : Cfg::A_BYTES;
    const uint32_t smem_off = is_b ? Cfg::A_BYTES : 0u;
    const uint32_t bk = p.bk;
    uint32_t stage = 0, phase = 0;
    bool ok = true;
    bool dep_waited = false;
    long long prof_wait = 0, prof_issue = 0;
    const long long prof_t0 = PROF ? clock64() : 0;
    detail::WorkIter work(p, cluster, num_clusters, BN);
    uint32_t t = 0, kb_lo = 0, kb_hi = 0;
    while (ok && work.next(t, kb_lo, kb_hi)) {
      uint32_t tm, tn;
      const uint32_t bidx = t / p.grid.num_tiles;  // problem of the batch
      tile_coords(p.grid, t - bidx * p.grid.num_tiles, tm, tn);
      const int32_t bz = od.broadcast ? 0 : static_cast<int32_t>(bidx);
      const int32_t row0 = is_b ? static_cast<int32_t>(tn * BN + work.col_off + rank * (work.cols / CTAS))
                                : static_cast<int32_t>(tm * (Cfg::BM * CTAS) + rank * Cfg::BM);
      const uint32_t nkb = kb_hi - kb_lo;
      const uint32_t rot = (p.tune & TUNE_K_STAGGER) ? (t * 31u) % nkb : 0u;
      if (!dep_waited) {
        ptx::grid_dependency_wait();
        dep_waited = true;
        if constexpr (PROF) {
          if (p.prof && !is_b && lane == 0) {
            p.prof[PROF_WORDS * blockIdx.x + 14] = setup_clocks;
            p.prof[PROF_WORDS * blockIdx.x + 16] = tl_entry;
            p.prof[PROF_WORDS * blockIdx.x + 17] = ptx::globaltimer_ns();
          }
        }
      }
      for (uint32_t kb = kb_lo; kb < kb_hi; ++kb) {
        const long long w0 = PROF ? clock64() : 0;
        const bool got = detail::wait(empty_bar(stage), phase ^ 1u, ab, WAIT_PRODUCER_EMPTY, t, kb);
        ok = __all_sync(0xFFFFFFFFu, got);
        if (!ok) break;
        const long long w1 = PROF ? clock64() : 0;
        if constexpr (PROF) prof_wait += w1 - w0;
        if (ptx::elect_one()) {
          const uint32_t dst = base + stage * Cfg::STAGE_BYTES + smem_off;
          uint32_t kk = kb + rot;  // K block fetched in this step
          if (kk >= kb_hi) kk -= nkb;
          const int32_t k0 = static_cast<int32_t>(kk * bk);
          uint32_t fb;
          if constexpr (CTAS == 1) {
            fb = full_bar(stage);
            ptx::mbar_arrive_expect_tx(fb, my_bytes);
          } else {
            // Both CTAs' bytes are counted on the leader's barrier.
            fb = ptx::mapa(full_bar(stage), 0);
            if (rank == 0) ptx::mbar_arrive_expect_tx(full_bar(stage), 2u * my_bytes);
          }
          for (uint32_t i = 0; i < boxes; ++i) {
            const int32_t mn = row0 + static_cast<int32_t>(i * box_mn);
            if constexpr (CTAS == 1)
              ptx::tma_load_3d(dst + i * box_bytes, tmap, mn_major ? mn : k0, mn_major ? k0 : mn, bz, fb);
            else
              ptx::tma_load_3d_pair(dst + i * box_bytes, tmap, mn_major ? mn : k0, mn_major ? k0 : mn, bz, fb);
          }
        }
        __syncwarp();
        if constexpr (PROF) prof_issue += clock64() - w1;
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
    if constexpr (PROF) {
      if (lane == 0 && p.prof) {
        p.prof[PROF_WORDS * blockIdx.x + (is_b ? 10 : 0)] = prof_wait;
        p.prof[PROF_WORDS * blockIdx.x + (is_b ? 11 : 8)] = prof_issue;
        if (!is_b) p.prof[PROF_WORDS * blockIdx.x + 1] = clock64() - prof_t0;
      }
    }
    if (!ok && rank == 0 && lane == 0) {
      // Aborting: give loads already issued a bounded chance to land before
      // the CTA's shared memory is released.  (stage, phase) is the next slot
      // to fill; the STAGES slots before it are the ones that may be in flight.
      const uint64_t t0 = ptx::globaltimer_ns();
      for (uint32_t i = 0; i < STAGES; ++i) {
        const uint32_t s = (stage + STAGES - 1u - i) % STAGES;
        const uint32_t ph = (s < stage) ? phase : (phase ^ 1u);
        while (!ptx::mbar_try_wait(full_bar(s), ph)) {
          if (ptx::globaltimer_ns() - t0 > 2000000ull) break;
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------- MMA issuer
    // Only the leader CTA of a pair issues.  As in the producer, the whole warp
    // walks the loop and one elected lane issues tcgen05.mma / tcgen05.commit.
    // The warp touches no global memory, but its bounded waits must not count the time the
    // launch spends waiting for the kernel before it; no operand can land before that anyway.
    ptx::grid_dependency_wait();
    if (rank == 0) {
      uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
      bool ok = true;
      bool issued = false;
      long long prof_full = 0, prof_tmem = 0, prof_tmem1 = 0, prof_issue = 0;
      const long long prof_t0 = PROF ? clock64() : 0;
      const uint64_t prof_ns0 = PROF ? ptx::globaltimer_ns() : 0;
      uint64_t tl_first = 0;
      const uint32_t a_hi = p.a.desc_hi, b_hi = p.b.desc_hi;
      const uint32_t a_lo0 = ((base >> 4) & 0x3FFFu) | p.a.desc_lo;
      const uint32_t b_lo0 = (((base + Cfg::A_BYTES) >> 4) & 0x3FFFu) | p.b.desc_lo;
      const uint32_t a_step = p.a.k_step16, b_step = p.b.k_step16;
      const uint32_t idesc = p.idesc;
      detail::WorkIter work(p, cluster, num_clusters, BN);
      uint32_t t = 0, kb_lo = 0, kb_hi = 0;
      while (ok && work.next(t, kb_lo, kb_hi)) {
        const long long w0 = PROF ? clock64() : 0;
        const bool got0 = detail::wait(tmem_empty_bar(acc), acc_phase ^ 1u, ab,
                                                  WAIT_MMA_TMEM_EMPTY, t, 0);
        ok = __all_sync(0xFFFFFFFFu, got0);
        if (!ok) break;
        if constexpr (PROF) prof_tmem += clock64() - w0;
        ptx::tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        const uint32_t idesc_cur = (work.cols == static_cast<uint32_t>(BN)) ? idesc : p.idesc_tail;
        // One row block's four MMAs on stage `st` (128 bytes of K per stage, 32 bytes per MMA).
        auto issue_block = [&](uint32_t mb, uint32_t kb, uint32_t st) {
          const uint32_t a_lo = a_lo0 + st * (Cfg::STAGE_BYTES >> 4) + mb * ((128u * 128u) >> 4);
          const uint32_t b_lo = b_lo0 + st * (Cfg::STAGE_BYTES >> 4);
#pragma unroll
          for (uint32_t j = 0; j < 4; ++j) {
            const uint64_t ad = (static_cast<uint64_t>(a_hi) << 32) | (a_lo + j * a_step);
            const uint64_t bd = (static_cast<uint64_t>(b_hi) << 32) | (b_lo + j * b_step);
            ptx::umma<Cfg::KIND, CTAS>(d_tmem + mb * BN, ad, bd, idesc_cur, (kb != kb_lo || j != 0u) ? 1u : 0u);
          }
        };
        // Release stage `st` to the producer(s) once the MMAs issued so far have read it.
        auto release_stage = [&](uint32_t st) {
          ptx::tc_commit<CTAS>(empty_bar(st));
          if constexpr (CTAS == 2) ptx::tc_commit<CTAS>(ptx::mapa(empty_bar(st), 1));
        };
        uint32_t kb = kb_lo;
        if constexpr (Cfg::MB == 2) {
          // The epilogue frees accumulator 0 first and accumulator 1 a little later.  Row block 0
          // therefore runs ahead over the first STAGES - 1 stages (which stay unreleased), then
          // row block 1 catches up on the same stages and releases them.
          const uint32_t pre = (kb_hi - kb_lo < static_cast<uint32_t>(STAGES - 1)) ? (kb_hi - kb_lo)
                                                                                  : static_cast<uint32_t>(STAGES - 1);
          uint32_t st = stage, ph = phase;
          for (uint32_t i = 0; i < pre; ++i) {
            const long long w1 = PROF ? clock64() : 0;
            const bool got = detail::wait(full_bar(st), ph, ab, WAIT_MMA_FULL, t, kb_lo + i);
            ok = __all_sync(0xFFFFFFFFu, got);
            if (!ok) break;
            const long long w2 = PROF ? clock64() : 0;
            if constexpr (PROF) {
              prof_full += w2 - w1;
              if (tl_first == 0) tl_first = ptx::globaltimer_ns();
            }
            ptx::tc_fence_after_sync();
            if (ptx::elect_one()) issue_block(0, kb_lo + i, st);
            __syncwarp();
            if constexpr (PROF) prof_issue += clock64() - w2;
            issued = true;
            if (++st == STAGES) {
              st = 0;
              ph ^= 1u;
            }
          }
          if (!ok) break;
          const long long w3 = PROF ? clock64() : 0;
          const bool got1 = detail::wait(tmem_empty_bar(1), acc_phase ^ 1u, ab,
                                                    WAIT_MMA_TMEM_EMPTY, t, 1);
          ok = __all_sync(0xFFFFFFFFu, got1);
          if (!ok) break;
          const long long w4 = PROF ? clock64() : 0;
          if constexpr (PROF) {
            prof_tmem += w4 - w3;
            prof_tmem1 += w4 - w3;
          }
          ptx::tc_fence_after_sync();
          for (uint32_t i = 0; i < pre; ++i) {
            if (ptx::elect_one()) {
              issue_block(1, kb_lo + i, stage);
              release_stage(stage);
            }
            __syncwarp();
            if (++stage == STAGES) {
              stage = 0;
              phase ^= 1u;
            }
          }
          if constexpr (PROF) prof_issue += clock64() - w4;
          kb = kb_lo + pre;
        }
        for (; kb < kb_hi; ++kb) {
          const long long w1 = PROF ? clock64() : 0;
          const bool got = detail::wait(full_bar(stage), phase, ab, WAIT_MMA_FULL, t, kb);
          ok = __all_sync(0xFFFFFFFFu, got);
          if (!ok) break;
          const long long w2 = PROF ? clock64() : 0;
          if constexpr (PROF) {
            prof_full += w2 - w1;
            if (tl_first == 0) tl_first = ptx::globaltimer_ns();
          }
          ptx::tc_fence_after_sync();
          if (ptx::elect_one()) {
#pragma unroll
            for (uint32_t mb = 0; mb < static_cast<uint32_t>(Cfg::MB); ++mb) issue_block(mb, kb, stage);
            release_stage(stage);
          }
          __syncwarp();
          if constexpr (PROF) prof_issue += clock64() - w2;
          issued = true;
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        if (!(p.test_flags & 1u) && ptx::elect_one()) {
#pragma unroll
          for (uint32_t mb = 0; mb < static_cast<uint32_t>(Cfg::MB); ++mb) {
            const uint32_t fb = tmem_full_bar(acc + mb);
            ptx::tc_commit<CTAS>(fb);
            if constexpr (CTAS == 2) ptx::tc_commit<CTAS>(ptx::mapa(fb, 1));
          }
        }
        __syncwarp();
        if constexpr (Cfg::MB == 2) {
          acc_phase ^= 1u;  // both accumulators are used by every tile
        } else {
          acc ^= 1u;
          if (acc == 0u) acc_phase ^= 1u;
        }
      }
      if constexpr (PROF) {
        if (lane == 0 && p.prof) {
          p.prof[PROF_WORDS * blockIdx.x + 2] = prof_full;
          p.prof[PROF_WORDS * blockIdx.x + 3] = prof_tmem;
          p.prof[PROF_WORDS * blockIdx.x + 4] = clock64() - prof_t0;
          p.prof[PROF_WORDS * blockIdx.x + 7] = ptx::globaltimer_ns() - prof_ns0;
          p.prof[PROF_WORDS * blockIdx.x + 9] = prof_issue;
          p.prof[PROF_WORDS * blockIdx.x + 13] = prof_tmem1;
          p.prof[PROF_WORDS * blockIdx.x + 18] = tl_first;
          p.prof[PROF_WORDS * blockIdx.x + 19] = ptx::globaltimer_ns();
        }
      }
      if ((!ok || (p.test_flags & 1u)) && issued && lane == 0) {
        // Aborting with MMAs possibly in flight: wait (bounded) for them before TMEM is freed.
        ptx::tc_commit<CTAS>(drain_bar);
        const uint64_t t0 = ptx::globaltimer_ns();
        while (!ptx::mbar_try_wait(drain_bar, 0)) {
          if (ptx::globaltimer_ns() - t0 > 2000000ull) break;
        }
      }
    }
  } else {
    // ---------------------------------------------------------- epilogue
    ptx::grid_dependency_wait();  // before the first access to C, D, the epilogue vectors or the split-K workspace
    if constexpr (!Cfg::SWAP) {
      // Four or eight warps; a warp reads the TMEM lanes of its quadrant (warp % 4) and, with
      // eight, one half of the tile's columns.  A warp first copies its whole share of an
      // accumulator to registers and hands the accumulator back at once; only then does it
      // scale, cast and store.  With two row blocks per CTA that hand-over is what the next
      // tile's main loop waits for; with one it merely shortens the epilogue, which shows where
      // a CTA has few tiles.
      constexpr int HALVES = Cfg::EPI_WARPS / 4;
      const uint32_t quad = warp & 3u;
      const uint32_t half = (HALVES == 2 && warp >= 7u) ? 1u : 0u;
      const uint32_t stg = staging_base + (half * 4u + quad) * Cfg::STAGING_WARP_BYTES;
      constexpr int BOX_COLS = 128 / sizeof(TOut);  // columns in one 128-byte staged row
      constexpr int SLICES = BOX_COLS / 32;         // 32-column TMEM slices per staged box
      constexpr int WORDS = 32 * sizeof(TOut) / 4;  // packed words per slice per row
      constexpr int WARP_COLS = BN / HALVES;        // accumulator columns one warp holds at a time
      constexpr int NSL = WARP_COLS / 32;
      static_assert(WARP_COLS % BOX_COLS == 0 && NSL <= 4, "a warp's share: whole boxes, at most 128 registers");
      uint32_t acc = 0, acc_phase = 0;
      bool ok = true;
      const bool prof = PROF && p.prof != nullptr && warp == 2 && lane == 0;
      long long prof_wait = 0, prof_copy = 0;
      uint64_t tl_acc = 0;
      const long long prof_t0 = prof ? clock64() : 0;
      const TOut* const cmat = static_cast<const TOut*>(p.c);
      const uint32_t tmem_empty_target =
          (CTAS == 2) ? ptx::mapa(tmem_empty_bar(0), 0) : tmem_empty_bar(0);
      // The plain path (see plain_tile_epilogue): its scalars are read now, and the routine runs
      // once dry while there is nothing else to do.
      const detail::EpiScalars sc{p.alpha_f, p.beta_f, p.alpha_i, p.beta_i};
      const bool plain_tma = Cfg::MB == 1 && p.epilogue_tma != 0u && p.epi_flags == 0u &&
                             (detail::OutTraits<TOut>::INT ? (p.beta_i == 0) : (p.beta_f == 0.0f));
      if constexpr (Cfg::MB == 1) {
        if (plain_tma)
          detail::plain_tile_epilogue<TOut, ACC_INT, NSL, CTAS>(tmem_base + ((quad * 32u) << 16) + half * WARP_COLS, stg, &tm_d, 0,
                                                                0, 0, sc, 0u, false);
      }
      detail::WorkIter work(p, cluster, num_clusters, BN);
      uint32_t t = 0, kb_lo = 0, kb_hi = 0;
      while (ok && work.next(t, kb_lo, kb_hi)) {
        uint32_t tm, tn;
        const uint32_t bidx = t / p.grid.num_tiles;  // problem of the batch
        tile_coords(p.grid, t - bidx * p.grid.num_tiles, tm, tn);
        const TOut* const cmat_b = cmat + static_cast<int64_t>(bidx) * p.stride_c;
        const uint32_t wcols = work.cols / HALVES;  // columns of this piece that belong to this warp
        const uint32_t col_w = tn * BN + work.col_off + half * wcols;
        // Warm the address translation of this warp's part of the output while the main loop runs
        // (see the swapped epilogue): one prefetch per warp, first row and first column it will store.
        if (lane == 0) {
          const uint32_t pf_row = tm * (Cfg::BM * CTAS) + rank * Cfg::BM + quad * 32u;
          if (pf_row < p.m && col_w < p.n && p.scatter_cols == 0u)  // never a peer GPU's memory
            ptx::prefetch_l2(detail::out_ptr<TOut>(p, pf_row, col_w, bidx));
        }
        if constexpr (Cfg::MB == 2 && sizeof(TOut) == 2) {
          // 16-bit outputs without a C term: a warp's share of BOTH accumulators fits in its
          // registers once packed (2 x 64 words), so both accumulators go back to the MMA warp
          // before a single byte is stored; the stores then drain under the next main loop.
          // (All CTAs finish their tiles at about the same time, so the burst of output stores
          // is slow to drain; it must not hold up tensor memory.)
          const bool plain = detail::OutTraits<TOut>::INT ? false : (p.beta_f == 0.0f && p.epi_flags == 0u);
          if (plain && wcols == static_cast<uint32_t>(WARP_COLS) && col_w + WARP_COLS <= p.n &&
              (p.epilogue_tma || p.d_vec_ok)) {
            uint32_t y[2][NSL][16];
            const uint32_t taddr0 = tmem_base + ((quad * 32u) << 16) + half * wcols;
            const uint32_t row00 = tm * (Cfg::BM * CTAS) + rank * Cfg::BM + quad * 32u;
            const long long w0 = prof ? clock64() : 0;
            if (!detail::wait(tmem_full_bar(0), acc_phase, ab, WAIT_EPILOGUE_TMEM_FULL, t, 0)) {
              ok = false;
              break;
            }
            const long long c0 = prof ? clock64() : 0;
            if (prof) prof_wait += c0 - w0;
            ptx::tc_fence_after_sync();
            {
              uint32_t v[NSL][32];
#pragma unroll
              for (int sl = 0; sl < NSL; ++sl) ptx::tmem_ld_32x32(taddr0 + sl * 32u, v[sl]);
              ptx::tmem_wait_ld();
              ptx::tc_fence_before_sync();
              __syncwarp();
              if (lane == 0) {
                if constexpr (CTAS == 2) ptx::mbar_arrive_cluster(tmem_empty_target);
                else ptx::mbar_arrive(tmem_empty_target);
              }
#pragma unroll
              for (int sl = 0; sl < NSL; ++sl) {
                detail::scale_slice_in_place<TOut, false, ACC_INT>(v[sl], p, nullptr);
#pragma unroll
                for (int i = 0; i < 16; ++i) y[0][sl][i] = v[sl][i];
              }
            }
            if (!detail::wait(tmem_full_bar(1), acc_phase, ab, WAIT_EPILOGUE_TMEM_FULL, t, 1)) {
              ok = false;
              break;
            }
            if (prof) tl_acc = ptx::globaltimer_ns();
            ptx::tc_fence_after_sync();
#pragma unroll
            for (int sl = 0; sl < NSL; ++sl) {
              uint32_t x[32];
              ptx::tmem_ld_32x32(taddr0 + BN + sl * 32u, x);
              ptx::tmem_wait_ld();
              detail::scale_slice_in_place<TOut, false, ACC_INT>(x, p, nullptr);
#pragma unroll
              for (int i = 0; i < 16; ++i) y[1][sl][i] = x[i];
            }
            ptx::tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) {
              if constexpr (CTAS == 2) ptx::mbar_arrive_cluster(tmem_empty_target + 8u);
              else ptx::mbar_arrive(tmem_empty_target + 8u);
            }
            if (prof) prof_copy += clock64() - c0;
            // Both accumulators are free; drain the registers.
#pragma unroll
            for (int mb = 0; mb < 2; ++mb) {
              const uint32_t row0 = row00 + mb * 128u;
              if (row0 >= p.m) break;
#pragma unroll
              for (int box = 0; box < WARP_COLS / BOX_COLS; ++box) {
                if (p.epilogue_tma) {
                  // One staging box per warp: the store issued from it must have read it out.
                  if (lane == 0) ptx::bulk_wait_group_read<0>();
                  __syncwarp();
                }
                {
#pragma unroll
                  for (int j = 0; j < 8; ++j) {  // 16-byte chunk j of the staged row
                    const uint32_t(&x)[16] = y[mb][box * SLICES + j / 4];
                    const uint32_t addr = stg + lane * 128u + ((static_cast<uint32_t>(j) ^ (lane & 7u)) << 4);
                    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(x[4 * (j % 4)]),
                                 "r"(x[4 * (j % 4) + 1]), "r"(x[4 * (j % 4) + 2]), "r"(x[4 * (j % 4) + 3])
                                 : "memory");
                  }
                }
                if (p.epilogue_tma) {
                  ptx::fence_proxy_async_smem();
                  __syncwarp();
                  if (lane == 0) {
                    ptx::tma_store_3d(&tm_d, stg, static_cast<int32_t>(col_w + box * BOX_COLS),
                                      static_cast<int32_t>(row0), static_cast<int32_t>(bidx));
                    ptx::bulk_commit_group();
                  }
                } else {
                  __syncwarp();
                  detail::store_staged_box<TOut>(p, stg, lane, row0, col_w + box * BOX_COLS, bidx);
                  __syncwarp();
                }
              }
            }
            acc_phase ^= 1u;
            continue;
          }
        }
#pragma unroll 1
        for (uint32_t mb = 0; mb < static_cast<uint32_t>(Cfg::MB); ++mb) {
          const uint32_t ai = (Cfg::MB == 2) ? mb : acc;  // accumulator this row block was summed in
          const long long w0 = prof ? clock64() : 0;
          if (!detail::wait(tmem_full_bar(ai), acc_phase, ab, WAIT_EPILOGUE_TMEM_FULL, t, mb)) {
            ok = false;
            break;
          }
          const long long c0 = prof ? clock64() : 0;
          if (prof) {
            prof_wait += c0 - w0;
            tl_acc = ptx::globaltimer_ns();
          }
          ptx::tc_fence_after_sync();
          const uint32_t row0 = tm * (Cfg::BM * CTAS) + rank * Cfg::BM + mb * 128u + quad * 32u;
          const uint32_t row = row0 + lane;
          const bool row_ok = row < p.m;
          const uint32_t taddr = tmem_base + ((quad * 32u) << 16) + ai * BN + half * wcols;
          const bool has_beta = detail::OutTraits<TOut>::INT ? (p.beta_i != 0) : (p.beta_f != 0.0f);
          // Fast path: this warp's whole share lies inside the matrix and C / D rows can be
          // accessed in 16-byte vectors.  Everything else (edge tiles, tail strips, unaligned
          // operands) takes the slice-by-slice path below, which frees the accumulator last.
          const bool fast = wcols == static_cast<uint32_t>(WARP_COLS) && col_w + WARP_COLS <= p.n &&
                            (p.epilogue_tma || p.d_vec_ok) && (!has_beta || p.c_vec_ok) && p.epi_flags == 0u;
          if (Cfg::MB == 1 && fast && plain_tma && row0 + 32u <= p.m) {
            detail::plain_tile_epilogue<TOut, ACC_INT, NSL, CTAS>(taddr, stg, &tm_d, static_cast<int32_t>(col_w),
                                                                  static_cast<int32_t>(row0), static_cast<int32_t>(bidx), sc,
                                                                  tmem_empty_target + 8u * ai, true);
            if (prof) prof_copy += clock64() - c0;
          } else if (fast) {
            uint32_t v[NSL][32];
#pragma unroll
            for (int sl = 0; sl < NSL; ++sl) ptx::tmem_ld_32x32(taddr + sl * 32u, v[sl]);
            ptx::tmem_wait_ld();
            // The accumulator is in registers: the MMA warp may overwrite it.
            ptx::tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) {
              if constexpr (CTAS == 2) ptx::mbar_arrive_cluster(tmem_empty_target + 8u * ai);
              else ptx::mbar_arrive(tmem_empty_target + 8u * ai);
            }
            if (prof) prof_copy += clock64() - c0;
            if (row0 < p.m) {
              const TOut* crow = cmat_b + static_cast<int64_t>(row) * p.ldc + col_w;
#pragma unroll
              for (int box = 0; box < WARP_COLS / BOX_COLS; ++box) {
                if (p.epilogue_tma) {
                  // One staging box per warp: the store issued from it must have read it out.
                  if (lane == 0) ptx::bulk_wait_group_read<0>();
                  __syncwarp();
                }
#pragma unroll
                for (int sl = 0; sl < SLICES; ++sl) {
                  uint32_t(&x)[32] = v[box * SLICES + sl];
                  const int c_off = box * BOX_COLS + sl * 32;
                  if (has_beta) {
                    if (row_ok) detail::scale_slice_in_place<TOut, true, ACC_INT>(x, p, crow + c_off);
                  } else {
                    detail::scale_slice_in_place<TOut, false, ACC_INT>(x, p, nullptr);
                  }
#pragma unroll
                  for (int q = 0; q < WORDS / 4; ++q) {
                    const uint32_t j = static_cast<uint32_t>(sl * (WORDS / 4) + q);
                    const uint32_t addr = stg + lane * 128u + ((j ^ (lane & 7u)) << 4);
                    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(x[4 * q]),
                                 "r"(x[4 * q + 1]), "r"(x[4 * q + 2]), "r"(x[4 * q + 3])
                                 : "memory");
                  }
                }
                if (p.epilogue_tma) {
                  ptx::fence_proxy_async_smem();
                  __syncwarp();
                  if (lane == 0) {
                    ptx::tma_store_3d(&tm_d, stg, static_cast<int32_t>(col_w + box * BOX_COLS),
                                      static_cast<int32_t>(row0), static_cast<int32_t>(bidx));
                    ptx::bulk_commit_group();
                  }
                } else {
                  __syncwarp();
                  detail::store_staged_box<TOut>(p, stg, lane, row0, col_w + box * BOX_COLS, bidx);
                  __syncwarp();
                }
              }
            }
          } else {
            if (row0 < p.m) {
              for (uint32_t box = 0; box * BOX_COLS < wcols; ++box) {
                const uint32_t box_col = col_w + box * BOX_COLS;
                if (box_col >= p.n) break;
                if (p.epilogue_tma) {
                  if (lane == 0) ptx::bulk_wait_group_read<0>();
                  __syncwarp();
                }
#pragma unroll 1
                for (int sl = 0; sl < SLICES; ++sl) {
                  const uint32_t col0 = box_col + sl * 32u;
                  if (col0 >= p.n) break;  // uniform across the warp
                  const uint32_t ncols = (p.n - col0 < 32u) ? (p.n - col0) : 32u;
                  uint32_t x[32];
                  ptx::tmem_ld_32x32(taddr + box * BOX_COLS + sl * 32u, x);
                  ptx::tmem_wait_ld();
                  const TOut* crow = cmat_b + static_cast<int64_t>(row) * p.ldc + col0;
                  detail::epilogue_math<TOut, ACC_INT>(x, p, crow, row_ok, ncols, row, col0);
                  if (p.epilogue_tma) {
#pragma unroll
                    for (int q = 0; q < WORDS / 4; ++q) {
                      const uint32_t j = static_cast<uint32_t>(sl * (WORDS / 4) + q);
                      const uint32_t addr = stg + lane * 128u + ((j ^ (lane & 7u)) << 4);
                      asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(x[4 * q]),
                                   "r"(x[4 * q + 1]), "r"(x[4 * q + 2]), "r"(x[4 * q + 3])
                                   : "memory");
                    }
                  } else if (row_ok) {
                    TOut* drow = detail::out_ptr<TOut>(p, row, col0, bidx);
                    if (GZ_STORE_OK(p, row, col0, ncols, p.m, p.n))
                      detail::store_direct<TOut>(x, drow, ncols, p.d_vec_ok != 0u);
                  }
                }
                if (p.epilogue_tma) {
                  ptx::fence_proxy_async_smem();
                  __syncwarp();
                  if (lane == 0) {
                    ptx::tma_store_3d(&tm_d, stg, static_cast<int32_t>(box_col), static_cast<int32_t>(row0),
                                      static_cast<int32_t>(bidx));
                    ptx::bulk_commit_group();
                  }
                }
              }
            }
            ptx::tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) {
              if constexpr (CTAS == 2) ptx::mbar_arrive_cluster(tmem_empty_target + 8u * ai);
              else ptx::mbar_arrive(tmem_empty_target + 8u * ai);
            }
          }
        }
        if (!ok) break;
        if constexpr (Cfg::MB == 2) {
          acc_phase ^= 1u;  // both accumulators are used by every tile
        } else {
          acc ^= 1u;
          if (acc == 0u) acc_phase ^= 1u;
        }
      }
      // The CTA's shared memory must outlive the reads of its last TMA stores; the writes
      // themselves complete on their own before the grid does.
      const uint64_t tl_issued = prof ? ptx::globaltimer_ns() : 0;
      if (p.epilogue_tma && lane == 0) ptx::bulk_wait_group_read<0>();
      if (prof) {
        p.prof[PROF_WORDS * blockIdx.x + 5] = prof_wait;
        p.prof[PROF_WORDS * blockIdx.x + 6] = clock64() - prof_t0;
        p.prof[PROF_WORDS * blockIdx.x + 12] = prof_copy;
        p.prof[PROF_WORDS * blockIdx.x + 20] = tl_acc;
        p.prof[PROF_WORDS * blockIdx.x + 21] = tl_issued;
        p.prof[PROF_WORDS * blockIdx.x + 22] = ptx::globaltimer_ns();
      }
    } else {
    const uint32_t quad = warp & 3u;  // TMEM lanes [32*quad, 32*quad+32) are readable by this warp
    uint32_t acc = 0, acc_phase = 0;
    bool ok = true;
    const bool prof = PROF && p.prof != nullptr && warp == 2 && lane == 0;
    long long prof_wait = 0, prof_park = 0;
    uint64_t tl_acc = 0;
    const long long prof_t0 = prof ? clock64() : 0;
    const TOut* const cmat = static_cast<const TOut*>(p.c);
    const uint32_t tmem_empty_target =
        (CTAS == 2) ? ptx::mapa(tmem_empty_bar(0), 0) : tmem_empty_bar(0);
    // The plain output path (floating-point output, no C term, no epilogue vectors, no scatter, whole
    // tiles) reads its parameters now and keeps them in registers: after the long wait for the
    // accumulator every parameter read would miss the constant cache again, one after the other,
    // with nothing left to hide it.
    float alpha_r = p.alpha_f;
    TOut* d_r = static_cast<TOut*>(p.d);
    long long ldd_r = p.ldd, sd_r = p.stride_d;
    uint32_t n_r = p.n, m_r = p.m;
#if defined(GZ_BOUNDS_CHECK)
    uint32_t fast_r = 0u;  // the checked build keeps every store on the path that checks its coordinates
#else
    uint32_t fast_r = (!detail::OutTraits<TOut>::INT && p.epi_flags == 0u && p.scatter_cols == 0u && p.beta_f == 0.0f) ? 1u : 0u;
#endif
    asm volatile("" : "+f"(alpha_r), "+l"(d_r), "+l"(ldd_r), "+l"(sd_r), "+r"(n_r), "+r"(m_r), "+r"(fast_r));
    if constexpr (!detail::OutTraits<TOut>::INT) {
      // Dry run of the output code (see swapped_store_plain): nothing is stored.
      if (fast_r != 0u)
        detail::swapped_store_plain<TOut, BN, ACC_INT>(tmem_base + ((quad * 32u) << 16), d_r, ldd_r,
                                                       static_cast<uint32_t>(BN), alpha_r, false);
    }
    detail::WorkIter work(p, cluster, num_clusters, BN);
    uint32_t t = 0, kb_lo = 0, kb_hi = 0;
    while (ok && work.next(t, kb_lo, kb_hi)) {
      uint32_t tm, tn;
      const uint32_t bidx = t / p.grid.num_tiles;  // problem of the batch
      tile_coords(p.grid, t - bidx * p.grid.num_tiles, tm, tn);
      const TOut* const cmat_b = cmat + static_cast<int64_t>(bidx) * p.stride_c;
      // The first store to a page the SM has not touched waits about a microsecond for its address
      // translation, and in a skinny problem the output is first touched after the last MMA, where
      // nothing hides that.  So the output rows of the tile are touched now, while the main loop
      // runs: one prefetch per row, by the first lanes of the warp that will store there.
      {
        const uint32_t pf_col = tm * 128u + quad * 32u;
        const uint32_t pf_row = tn * BN + lane;
        if (lane < static_cast<uint32_t>(BN) && pf_col < p.m && pf_row < p.n && p.scatter_cols == 0u)
          ptx::prefetch_l2(detail::out_ptr<TOut>(p, pf_row, pf_col, bidx));
      }
      const long long w0 = prof ? clock64() : 0;
      if (!detail::wait(tmem_full_bar(acc), acc_phase, ab, WAIT_EPILOGUE_TMEM_FULL, t, 0)) {
        ok = false;
        break;
      }
      if (prof) {
        prof_wait += clock64() - w0;
        tl_acc = ptx::globaltimer_ns();
      }
      ptx::tc_fence_after_sync();
      {
        // Swapped operands: accumulator lane = output column (n), accumulator column = output row (m).
        const uint32_t ncol0 = tm * 128u + quad * 32u;  // first n of this warp
        const uint32_t ncol = ncol0 + lane;
        const bool n_ok = ncol < p.m;                   // p.m is the extent of the 128-row side (N)
        const uint32_t taddr = tmem_base + ((quad * 32u) << 16) + acc * BN;
        const bool partial = (kb_lo != 0u) || (kb_hi != k_blocks);
        uint32_t contributors = 1, my_slot = 0;
        bool finish = true;  // this CTA writes the tile's output
        if (partial && detail::aborted(ab)) {  // never enter the CTA-wide barrier below while aborting
          ok = false;
          break;
        }
        const long long e0 = prof ? clock64() : 0;
        // Workspace layout: [tile][slot][BN / 4][128 accumulator lanes] of float4 (4 consecutive
        // columns of one lane), so that the 32 lanes of a warp always touch 512 contiguous bytes.
        const size_t lane_off = static_cast<size_t>(quad * 32u + lane);
        constexpr size_t SLOT_F4 = static_cast<size_t>(BN) * 128u / 4u;  // float4 per slot
        if (partial) {
          // This CTA holds only part of the tile's K range.  Park the partial accumulator in this
          // CTA's workspace slot; the CTA that arrives last adds the slots in K order and writes
          // the output, so the result does not depend on arrival order.
          const unsigned long long tile_u0 = static_cast<unsigned long long>(t) * k_blocks;
          const uint32_t first = detail::split_owner(tile_u0, p.total_kb, num_clusters);
          const uint32_t last = detail::split_owner(tile_u0 + k_blocks - 1u, p.total_kb, num_clusters);
          contributors = last - first + 1u;
          my_slot = cluster - first;
#if defined(GZ_BOUNDS_CHECK)
          // the workspace holds max_contrib slots per tile (rows = slots, cols = tiles of the launch)
          if (!detail::store_in_bounds(p, my_slot, t, 1u, p.max_contrib, static_cast<uint32_t>(p.total_kb / k_blocks))) {
            *reinterpret_cast<volatile uint32_t*>(ab.flag) = 1u;  // every role of the CTA gives up
            ok = false;
            break;
          }
#endif
          float4* slot = reinterpret_cast<float4*>(p.ws) +
                         (static_cast<size_t>(t) * p.max_contrib + my_slot) * SLOT_F4 + lane_off;
#pragma unroll
          for (int sl = 0; sl < BN / 16; ++sl) {
            uint32_t v[16];
            ptx::tmem_ld_32x16(taddr + sl * 16u, v);
            ptx::tmem_wait_ld();
#pragma unroll
            for (int q = 0; q < 4; ++q)
              slot[(sl * 4 + q) * 128] = make_float4(__uint_as_float(v[4 * q]), __uint_as_float(v[4 * q + 1]),
                                                     __uint_as_float(v[4 * q + 2]), __uint_as_float(v[4 * q + 3]));
          }
          __threadfence();
          ptx::named_barrier_sync(1, 128);  // all four epilogue warps have parked their rows
          if (warp == 2 && lane == 0) {
            const int old = atomicAdd(p.counters + t, 1);
            const bool is_last = static_cast<uint32_t>(old) == contributors - 1u;
            if (is_last) p.counters[t] = 0;  // leave the counter clean for the next launch
            *split_flag = is_last ? 1u : 0u;
          }
          ptx::named_barrier_sync(1, 128);
          finish = *reinterpret_cast<volatile uint32_t*>(split_flag) != 0u;
          if (finish) __threadfence();
        }
        const long long e1 = prof ? clock64() : 0;
        if (prof) prof_park += e1 - e0;
        if constexpr (!detail::OutTraits<TOut>::INT) {
          if (finish && !partial && fast_r != 0u) {
            const uint32_t mrow0 = tn * BN;
            if (ncol0 < m_r && mrow0 < n_r) {
              TOut* dp = d_r + static_cast<long long>(bidx) * sd_r + static_cast<long long>(mrow0) * ldd_r + ncol;
              const uint32_t rows = (n_r - mrow0 < static_cast<uint32_t>(BN)) ? n_r - mrow0 : static_cast<uint32_t>(BN);
              detail::swapped_store_plain<TOut, BN, ACC_INT>(taddr, dp, ldd_r, rows, alpha_r, ncol < m_r);
            }
            finish = false;  // the tile is written
          }
        }
        if (finish && ncol0 < p.m) {
          const bool has_beta = detail::OutTraits<TOut>::INT ? (p.beta_i != 0) : (p.beta_f != 0.0f);
#pragma unroll
          for (int sl = 0; sl < BN / 16; ++sl) {
            const uint32_t mrow0 = tn * BN + sl * 16u;
            if (mrow0 >= p.n) break;  // uniform across the warp
            uint32_t v[16];
            if (!partial) {
              ptx::tmem_ld_32x16(taddr + sl * 16u, v);
              ptx::tmem_wait_ld();
            } else {
              // Slots are added in K order, four at a time so that their loads overlap.
              const float4* s0 = reinterpret_cast<const float4*>(p.ws) +
                                 static_cast<size_t>(t) * p.max_contrib * SLOT_F4 + lane_off + (sl * 4) * 128;
              float4 sum[4];
              for (uint32_t c0 = 0; c0 < contributors; c0 += 4u) {
                float4 x[4][4];
#pragma unroll
                for (int cc = 0; cc < 4; ++cc) {
                  const bool have = c0 + cc < contributors;
                  const float4* sc = s0 + static_cast<size_t>(c0 + cc) * SLOT_F4;
#pragma unroll
                  for (int q = 0; q < 4; ++q)
                    x[cc][q] = have ? __ldcg(sc + q * 128) : make_float4(0.f, 0.f, 0.f, 0.f);
                }
#pragma unroll
                for (int cc = 0; cc < 4; ++cc) {
                  if (c0 + cc >= contributors) break;
#pragma unroll
                  for (int q = 0; q < 4; ++q) {
                    if (c0 + cc == 0u) {
                      sum[q] = x[cc][q];
                    } else if constexpr (ACC_INT) {
                      sum[q].x = __uint_as_float(__float_as_uint(sum[q].x) + __float_as_uint(x[cc][q].x));
                      sum[q].y = __uint_as_float(__float_as_uint(sum[q].y) + __float_as_uint(x[cc][q].y));
                      sum[q].z = __uint_as_float(__float_as_uint(sum[q].z) + __float_as_uint(x[cc][q].z));
                      sum[q].w = __uint_as_float(__float_as_uint(sum[q].w) + __float_as_uint(x[cc][q].w));
                    } else {
                      sum[q].x += x[cc][q].x;
                      sum[q].y += x[cc][q].y;
                      sum[q].z += x[cc][q].z;
                      sum[q].w += x[cc][q].w;
                    }
                  }
                }
              }
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                v[4 * q] = __float_as_uint(sum[q].x);
                v[4 * q + 1] = __float_as_uint(sum[q].y);
                v[4 * q + 2] = __float_as_uint(sum[q].z);
                v[4 * q + 3] = __float_as_uint(sum[q].w);
              }
            }
            if (n_ok) {
              // Column i of the slice is output row mrow0 + i; for each, the 32 lanes of the warp
              // write 32 consecutive elements of that row.
              const uint32_t cnt = (p.n - mrow0 < 16u) ? (p.n - mrow0) : 16u;
              TOut* dp = detail::out_ptr<TOut>(p, mrow0, ncol, bidx);
              const TOut* cp = cmat_b + static_cast<int64_t>(mrow0) * p.ldc + ncol;
              if (has_beta) {
#pragma unroll
                for (int i = 0; i < 16; ++i)
                  if (static_cast<uint32_t>(i) < cnt && GZ_STORE_OK(p, mrow0 + i, ncol, 1u, p.n, p.m))
                    dp[static_cast<int64_t>(i) * p.ldd] =
                        detail::epilogue_scalar<TOut, true, ACC_INT>(v[i], p, cp + static_cast<int64_t>(i) * p.ldc,
                                                                     mrow0 + i, ncol);
              } else {
#pragma unroll
                for (int i = 0; i < 16; ++i)
                  if (static_cast<uint32_t>(i) < cnt && GZ_STORE_OK(p, mrow0 + i, ncol, 1u, p.n, p.m))
                    dp[static_cast<int64_t>(i) * p.ldd] =
                        detail::epilogue_scalar<TOut, false, ACC_INT>(v[i], p, nullptr, mrow0 + i, ncol);
              }
            }
          }
        }
      }
      // This accumulator may now be overwritten by the MMA warp.
      ptx::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        if constexpr (CTAS == 2) ptx::mbar_arrive_cluster(tmem_empty_target + 8u * acc);
        else ptx::mbar_arrive(tmem_empty_target + 8u * acc);
      }
      acc ^= 1u;
      if (acc == 0u) acc_phase ^= 1u;
    }
    if (prof) {
      p.prof[PROF_WORDS * blockIdx.x + 5] = prof_wait;
      p.prof[PROF_WORDS * blockIdx.x + 6] = clock64() - prof_t0;
      p.prof[PROF_WORDS * blockIdx.x + 12] = prof_park;
      p.prof[PROF_WORDS * blockIdx.x + 20] = tl_acc;
      p.prof[PROF_WORDS * blockIdx.x + 21] = ptx::globaltimer_ns();
      p.prof[PROF_WORDS * blockIdx.x + 22] = p.prof[PROF_WORDS * blockIdx.x + 21];
    }
    }
  }

  // -------------------------------------------------------------- teardown
  __syncwarp();
  ptx::tc_fence_before_sync();
  __syncthreads();
  // Every thread passes the dependency wait before it leaves (a CTA without work has not yet; for
  // the others it is satisfied): this grid then never completes before the one it follows, and
  // the counters touched below are safe to touch.
  ptx::grid_dependency_wait();
  if (detail::aborted(ab)) {
    // Loads issued by a peer CTA's producer are counted on the leader's
    // barriers; give anything still in flight time to land.
    const uint64_t t0 = ptx::globaltimer_ns();
    while (ptx::globaltimer_ns() - t0 < 100000ull) __nanosleep(1000);
  }
  if constexpr (CTAS == 2) {
    // Neither CTA may exit (or free TMEM) while its partner can still signal
    // its barriers or read its shared memory.
    ptx::cluster_arrive_release();
    ptx::cluster_wait_acquire();
  }
  if (warp == 1) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc<CTAS>(tmem_base, Cfg::TMEM_COLS);
  }
  if ((late_work & 1u) && threadIdx.x == 0) {
    // The barriers above ordered this CTA's output stores before this thread; the fence makes
    // them visible to the other GPUs before the arrival is counted.
    __threadfence_system();
    if (atomicAdd(p.signal_counter, 1u) == gridDim.x - 1u) {
      *p.signal_counter = 0u;
      __threadfence_system();
      for (uint32_t g = 0; g < p.signal_count; ++g) *reinterpret_cast<volatile uint32_t*>(p.signal_ptrs[g]) = p.signal_value;
      __threadfence_system();
    }
  }
  if ((late_work & 2u) && rank == 0 && threadIdx.x == 0) {
    // Every pair drew its ticket before it did anything else, so when the last one leaves nobody
    // needs the counters any more.
    if (atomicAdd(p.die_tickets + 2, 1u) == num_clusters - 1u) {
      p.die_tickets[0] = 0u;
      p.die_tickets[1] = 0u;
      p.die_tickets[2] = 0u;
      __threadfence();
    }
  }
  if constexpr (PROF) {
    if ((late_work & 4u) && threadIdx.x == 32) {
      p.prof[PROF_WORDS * blockIdx.x + 15] = clock64() - kernel_t0;
      p.prof[PROF_WORDS * blockIdx.x + 23] = ptx::globaltimer_ns();
    }
  }
}

}  // namespace gz
#endif
