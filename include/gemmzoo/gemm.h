/*
 * gemmzoo C ABI — dense GEMM  D = alpha * A * B + beta * C  on NVIDIA B200 (sm_100a).
 *
 * This is the launch layer that sits under the C++ functor
 * nvidia::kernel_functors::sm100_gemm (nvidia/kernel_functors/sm100_gemm.cuh).
 * It replaces, for the reference project AD2605/gemm-zoo, what its header-only
 * functors do inline:
 *   - constructor of a functor (geometry, shared-memory opt-in)
 *       nvidia/kernel_functors/bf16_mma_gemm.cuh:17-49
 *       nvidia/kernel_functors/fp16_mma_gemm.cuh:17-47
 *       nvidia/kernel_functors/tf32_mma_gemm.cuh:16-41
 *       nvidia/kernel_functors/generic_gemm.cuh:15-24      -> gz_gemm_plan_create
 *   - operator() of a functor (one asynchronous launch on a stream)
 *       nvidia/kernel_functors/bf16_mma_gemm.cuh:51-63
 *       nvidia/kernel_functors/generic_gemm.cuh:26-35      -> gz_gemm_run
 *   - the s8*s8->s32 contract of intel/xe_gemm_s8_s8_s32_m8k16.hpp:27-40
 *       (int32 alpha/beta, int32 C/D)                      -> GZ_DT_S8 / GZ_DT_S32
 *   - the fill of operand buffers, nvidia/utils/fill_data.cuh:33-49
 *                                                          -> gz_fill
 *
 * Conventions
 *   - All pointers given to gz_gemm_run are DEVICE pointers owned by the caller.
 *     gz_gemm_run_host takes HOST pointers and performs the copies itself.
 *   - C and D are row-major (ldc, ldd = elements between rows), as everywhere in
 *     the reference.  A is M x K, B is K x N; each may be row- or column-major.
 *     Reference default: A row-major lda=K, B row-major ldb=N, C/D ld=N
 *     (nvidia/kernels/naive_gemm.cuh:18-20).
 *   - alpha and beta are passed by HOST pointer in the scale type of the
 *     problem: int32_t when the output type is s32, float otherwise.
 *   - C is not read when beta == 0 (the rule of nvidia/kernels/generic_gemm.cuh:55).
 *     D may alias C.
 *   - Nothing here exits the process or throws; every entry point returns a
 *     gz_status.  There is no CPU fallback: without a usable sm_100 device
 *     plan creation fails with GZ_ERR_NO_DEVICE.
 */
#ifndef GEMMZOO_GEMM_H
#define GEMMZOO_GEMM_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(_WIN32)
#define GZ_API
#else
#define GZ_API __attribute__((visibility("default")))
#endif

typedef enum gz_status {
  GZ_OK = 0,
  GZ_ERR_INVALID_ARG = 1,    /* null pointer, non-positive extent, ld < extent, bad enum */
  GZ_ERR_UNSUPPORTED = 2,    /* dtype pair / config not implemented */
  GZ_ERR_MISALIGNED = 3,     /* pointer not aligned to its element size, or an explicit tensor-core
                                config asked for with a leading dimension that is not 16-byte sized */
  GZ_ERR_CUDA = 4,           /* a CUDA runtime/driver call failed; see gz_last_cuda_error */
  GZ_ERR_DEVICE_TIMEOUT = 5, /* a bounded wait inside the kernel expired */
  GZ_ERR_NO_DEVICE = 6,      /* no CUDA device, or device is not compute capability 10.x */
  GZ_ERR_TOO_LARGE = 7,      /* extent exceeds what the kernel's 32-bit tile coordinates hold */
  GZ_ERR_OUT_OF_MEMORY = 8,
  GZ_ERR_DEBUG_CHECK = 9     /* debug build only (libgemmzoo_dbg.so): an epilogue store failed its bounds check */
} gz_status;

typedef enum gz_dtype {
  GZ_DT_F16 = 0,
  GZ_DT_BF16 = 1,
  GZ_DT_F32 = 2, /* as an input type: fp32 storage, tf32 multiply, fp32 accumulate */
  GZ_DT_S8 = 3,
  GZ_DT_S32 = 4,
  /* 8-bit floating point inputs (outputs: f16, bf16 or f32; fp32 accumulate).  The reference only
   * declares the intent: nvidia/bench/bench_cublaslt_e4m3.cu:6-21, bench_cublaslt_e5m2.cu and the fp8
   * branches of nvidia/kernel_functors/cublaslt_gemm.cuh:85-90,106-109; it has no kernel of its own. */
  GZ_DT_E4M3 = 5, /* 1-4-3, no infinities (CUDA __nv_fp8_e4m3) */
  GZ_DT_E5M2 = 6  /* 1-5-2 (CUDA __nv_fp8_e5m2) */
} gz_dtype;

typedef enum gz_layout { GZ_ROW_MAJOR = 0, GZ_COL_MAJOR = 1 } gz_layout;

/* Kernel configuration.  GZ_CFG_AUTO lets the plan choose.  The explicit values
 * exist so that tests and benchmarks can pin one variant. */
typedef enum gz_config {
  GZ_CFG_AUTO = 0,
  GZ_CFG_1CTA_N256 = 1, /* 128x256 tile, one CTA */
  GZ_CFG_1CTA_N128 = 2, /* 128x128 tile, one CTA */
  GZ_CFG_1CTA_N64 = 3,  /* 128x64 tile, one CTA  */
  GZ_CFG_2CTA_N256 = 4, /* 256x256 tile on a 2-CTA pair (tcgen05 cta_group::2) */
  GZ_CFG_2CTA_N128 = 5, /* 256x128 tile on a 2-CTA pair */
  /* Skinny problems: operand roles exchanged, 128 output columns x up to 16/32/64/128 output rows per tile */
  GZ_CFG_SWAP_M16 = 6,
  GZ_CFG_SWAP_M32 = 7,
  GZ_CFG_SWAP_M64 = 8,
  GZ_CFG_SWAP_M128 = 9,
  /* 512x256 tile on a 2-CTA pair: each CTA holds two 128-row blocks of A against its half of B, so
   * a quarter less operand data moves per flop than with GZ_CFG_2CTA_N256.  For large problems. */
  GZ_CFG_2CTA_M512_N256 = 10,
  GZ_CFG_SIMT = 15      /* plain CUDA-core kernel; chosen automatically when TMA alignment rules fail */
} gz_config;

/* flags */
#define GZ_FLAG_EPILOGUE_DIRECT 0x1u /* registers -> global stores, no TMA store */
#define GZ_FLAG_EPILOGUE_TMA 0x2u    /* force the shared-memory + TMA-store epilogue */
#define GZ_FLAG_BROADCAST_A 0x10u    /* batched: every problem reads the same A (stride_a ignored) */
#define GZ_FLAG_BROADCAST_B 0x20u    /* batched: every problem reads the same B (stride_b ignored) */
/* Split-K (skinny problems only): the K range of a tile may be shared by several CTAs, which
 * park fp32 partial sums in a workspace owned by the plan; the last CTA to arrive adds them in K
 * order.  Chosen automatically when it balances the SMs better; these flags override the choice.
 * A plan that uses the workspace must not run concurrently with itself on two streams. */
/* Large problems on a two-die part: by default the plan measures once per device which die each SM
 * sits on and lets the CTAs of one die take neighbouring tiles of each wave (less die-to-die
 * traffic).  Results do not depend on it.  The order keeps 32 small sets of counters per plan, one
 * per launch in flight; a caller that keeps MORE than 32 launches of one plan in flight at the
 * same time on different streams must switch it off. */
#define GZ_FLAG_NO_DIE_ORDER 0x40u
#define GZ_FLAG_NO_SPLIT_K 0x4u
#define GZ_FLAG_SPLIT_K 0x8u
/* Test knob: the MMA warp never signals "accumulator ready", so the epilogue's
 * bounded wait expires and the launch reports GZ_ERR_DEVICE_TIMEOUT.  Nothing
 * faults or hangs; use with a small wait_limit_ns. */
#define GZ_FLAG_TEST_WITHHOLD_ACC_READY 0x80000000u

typedef struct gz_gemm_desc {
  uint32_t struct_size; /* = sizeof(gz_gemm_desc) */
  int32_t in_type;      /* gz_dtype of A and B */
  int32_t out_type;     /* gz_dtype of C and D */
  int32_t layout_a;     /* gz_layout */
  int32_t layout_b;     /* gz_layout */
  int32_t device;       /* CUDA device ordinal */
  int32_t config;       /* gz_config */
  uint32_t flags;
  int64_t m, n, k;
  int64_t lda, ldb, ldc, ldd; /* 0 = packed default for the layout */
  uint64_t wait_limit_ns;     /* 0 = default (2 s); bound on every in-kernel wait */
  /* Batched GEMM: `batch` independent problems of the same shape in one launch, problem i reading
   * A + i * stride_a, B + i * stride_b, C + i * stride_c and writing D + i * stride_d (strides in
   * elements).  batch 0 or 1 = a single problem; a stride of 0 = packed (rows x leading dimension);
   * stride_a or stride_b may be given as 0 with GZ_FLAG_BROADCAST_A / _B to share one matrix.
   * No counterpart in the reference. */
  int64_t batch;
  int64_t stride_a, stride_b, stride_c, stride_d;
} gz_gemm_desc;

typedef struct gz_plan gz_plan;

/* What the plan decided; filled by gz_gemm_plan_info. */
typedef struct gz_plan_info {
  int32_t config;       /* gz_config actually used */
  int32_t tile_m, tile_n, tile_k;
  int32_t stages;
  int32_t ctas_per_tile;
  int32_t grid;         /* CTAs launched */
  int32_t smem_bytes;   /* dynamic shared memory per CTA */
  int32_t epilogue_tma; /* 1 if the TMA-store epilogue is used */
  int32_t sm_count;
  int32_t split_k;      /* 1 if K ranges are shared between CTAs (uses the plan's workspace) */
  int32_t reserved;
  int64_t tiles;        /* output tiles */
  int64_t workspace_bytes; /* device scratch memory owned by the plan */
  int64_t lda, ldb, ldc, ldd;
  int32_t die_order;    /* 1 if the die-aware tile order is on (see GZ_FLAG_NO_DIE_ORDER) */
  int32_t reserved2;
} gz_plan_info;

/* Host-only validation of a descriptor: every argument error is reachable
 * without a GPU.  On success *cfg (if non-null) receives the configuration
 * that would be chosen for a device with sm_count SMs (0 = assume 148). */
GZ_API gz_status gz_gemm_desc_validate(const gz_gemm_desc* desc, int sm_count, gz_plan_info* info);

GZ_API gz_status gz_gemm_plan_create(gz_plan** plan, const gz_gemm_desc* desc);
GZ_API gz_status gz_gemm_plan_destroy(gz_plan* plan);
GZ_API gz_status gz_gemm_plan_info(const gz_plan* plan, gz_plan_info* info);

/* Diagnostics: give the plan a device buffer of GZ_PROFILE_WORDS_PER_CTA * info.grid 64-bit words and
 * every later launch records, per CTA, the clocks its producer, MMA and epilogue roles spent
 * waiting (words 0..15) and a timeline in global-timer nanoseconds (words 16..23: entry, set-up
 * done and dependencies satisfied, first operands landed, last MMA issued, last accumulator ready,
 * last stores issued, their shared memory read out, exit); layout: GemmParams::prof in
 * csrc/sm100_gemm.cuh.  NULL switches it off again.  The buffer must hold at least that many
 * words: nothing checks a raw pointer's size.  Counters are compiled in for bf16 -> bf16 plans of one tile shape per
 * family (GZ_CFG_1CTA_N64, GZ_CFG_2CTA_N256, GZ_CFG_2CTA_M512_N256, GZ_CFG_SWAP_M16); other plans
 * return GZ_ERR_UNSUPPORTED.  No counterpart in the reference. */
#define GZ_PROFILE_WORDS_PER_CTA 24
GZ_API gz_status gz_gemm_plan_set_profile(gz_plan* plan, void* device_words);

/* Diagnostics of the die-aware tile order (no counterpart in the reference, which predates
 * two-die parts).  gz_device_placement: die (0 or 1) of every SM of `device` as the library
 * measured it (die_of_sm: one byte per SM, at least 160 bytes), and the SMs per die;
 * GZ_ERR_UNSUPPORTED when the device did not show two dies.  gz_classify_dies is the host-only
 * half of that measurement: clocks[sm * lines + j] is what a load of probe line j cost from SM sm. */
GZ_API gz_status gz_device_placement(int32_t device, uint8_t* die_of_sm, int32_t sms_on_die[2]);
GZ_API gz_status gz_classify_dies(const uint32_t* clocks, int32_t sms, int32_t lines, uint8_t* die_of_sm,
                                  int32_t sms_on_die[2]);

/* Asynchronous on `stream` (a cudaStream_t passed as void*; NULL = legacy default stream).
 * a, b, c, d: device pointers.  c may be NULL when *beta == 0. */
GZ_API gz_status gz_gemm_run(gz_plan* plan, const void* a, const void* b, const void* c, void* d,
                             const void* alpha, const void* beta, void* stream);

/* Optional epilogue terms for floating-point outputs, applied in fp32 inside the GEMM's epilogue:
 *
 *     D[i][j] = act(alpha * row_scale[i] * col_scale[j] * acc[i][j] + beta * C[i][j] + bias[j])
 *
 * Any pointer may be NULL (term absent).  With s8 inputs and an f16/bf16/f32 output type this is
 * the dequantising GEMM (int32 accumulation, per-row and per-column scales).  No counterpart in the
 * reference's own kernels; the nearest thing is the bias its Intel test passes to the library
 * (intel/test/utils.hpp:133-136). */
typedef enum gz_activation {
  GZ_ACT_NONE = 0,
  GZ_ACT_RELU = 1,
  GZ_ACT_GELU = 2,      /* 0.5 x (1 + erf(x / sqrt 2)) */
  GZ_ACT_GELU_TANH = 3, /* 0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3))) */
  GZ_ACT_SILU = 4       /* x / (1 + exp(-x)) */
} gz_activation;

typedef struct gz_epilogue {
  uint32_t struct_size; /* sizeof(gz_epilogue) */
  int32_t activation;   /* gz_activation */
  const float* bias;      /* n floats on the device, or NULL */
  const float* row_scale; /* m floats on the device, or NULL */
  const float* col_scale; /* n floats on the device, or NULL */
} gz_epilogue;

/* gz_gemm_run with the optional terms (ep may be NULL: identical to gz_gemm_run).
 * GZ_ERR_UNSUPPORTED for plans with an s32 output. */
GZ_API gz_status gz_gemm_run_ex(gz_plan* plan, const void* a, const void* b, const void* c, void* d,
                                const void* alpha, const void* beta, const gz_epilogue* ep, void* stream);

/* Same computation with HOST operands: copies A, B (and C when beta != 0) to
 * device staging owned by the plan, runs, copies D back, and synchronises the
 * stream before returning.  Large problems are pipelined: B, C and D travel in
 * column blocks on two internal copy streams while the GEMM of each block runs
 * on `stream`, so uploads, compute and downloads overlap (give it pinned host
 * memory; pageable memory works but serialises the copies). */
GZ_API gz_status gz_gemm_run_host(gz_plan* plan, const void* a, const void* b, const void* c, void* d,
                                  const void* alpha, const void* beta, void* stream);

/* gz_gemm_run_host for one GPU of a column-partitioned run (one plan per GPU, each for its own
 * column block; the reference harness is single-GPU, nvidia/utils/benchmark.cuh:20, so this has no
 * counterpart there).  With GZ_HOST_A_ON_DEVICE, `a` is a DEVICE pointer on the plan's GPU whose
 * contents are valid in the order of `stream`: the replicated operand, of which every GPU uploaded
 * only a slice and which was then gathered GPU to GPU, instead of crossing the host's PCIe fabric
 * once per GPU.  b, c, d stay host pointers.  Everything the call does is ordered after the work
 * already queued on `stream` (the slice's upload and the gather): the slice has the link to itself
 * first, the blocks of B follow.  host_flags == 0 is gz_gemm_run_host. */
#define GZ_HOST_A_ON_DEVICE 0x1u
GZ_API gz_status gz_gemm_run_host_ex(gz_plan* plan, const void* a, const void* b, const void* c, void* d,
                                     const void* alpha, const void* beta, void* stream, uint32_t host_flags);

/* The same skinny (M <= 128) split-K GEMM for hosts that must not allocate.  This entry point has
 * no counterpart in the reference.  It exists for callers that gave all device memory to their own
 * allocator at start-up and may not call cudaMalloc afterwards (it could fail against their budget
 * and it synchronises the device inside a latency-critical loop), so they cannot create a plan.
 * Nothing is allocated here, neither on the device nor through any allocating library routine:
 * the partial sums, arrival counters and status words of the kernel live in a fixed array inside
 * the library image, GZ_STATIC_SCRATCH_BYTES per GPU that loads the library, held until exit.
 *   - `desc` describes the problem as for gz_gemm_plan_create; a, b, c, d are device pointers that
 *     TMA can address (16-byte aligned A and B, leading dimensions sized in multiples of 16 bytes).
 *     GZ_ERR_UNSUPPORTED for m > 128, GZ_ERR_MISALIGNED for operands TMA cannot describe.
 *   - A problem whose partial sums do not fit the array is refused with GZ_ERR_TOO_LARGE
 *     (gz_last_cuda_error() then says how many bytes it needs); use a plan for it.
 *   - The first call on a device looks up the array's device address and opts the kernel into its
 *     shared-memory size; make that first call before any stream capture.
 *   - Every call on a device shares the one array.  It keeps the previous call's contents; what
 *     must start at zero (the arrival counters) is cleared on `stream` before the launch.  Two
 *     calls that overlap on the GPU (different streams, or different threads) race on it:
 *     serialise them.
 *   - A bounded wait that expires inside the kernel is reported by gz_static_last_device_status,
 *     not by this call (which only launches).
 * Asynchronous on `stream`. */
#define GZ_STATIC_SCRATCH_BYTES (8u << 20)
GZ_API gz_status gz_gemm_skinny_static(const gz_gemm_desc* desc, const void* a, const void* b, const void* c,
                                       void* d, const void* alpha, const void* beta, void* stream);

/* Failure detection for gz_gemm_skinny_static, which has no plan to ask (no counterpart in the
 * reference; allocates nothing either).  The kernel's four status words live at the end of the
 * same fixed array.  They keep the FIRST bounded wait that expired in any gz_gemm_skinny_static
 * launch on `device` until this call reads them: it blocks until `stream` is idle, copies the 16
 * bytes, clears them if set, and returns GZ_ERR_DEVICE_TIMEOUT (detail as for
 * gz_last_device_status; may be NULL) or GZ_OK.  After a timeout D is partly written; the array
 * and the context stay usable, and the next gz_gemm_skinny_static call clears what the aborted
 * launch left in the arrival counters. */
GZ_API gz_status gz_static_last_device_status(int32_t device, void* stream, uint32_t detail[4]);

/* Synchronises the plan's device status word: returns GZ_OK, or
 * GZ_ERR_DEVICE_TIMEOUT if a bounded wait expired in any launch since the last
 * call (detail[0] = role/barrier code, detail[1] = block, detail[2] = tile,
 * detail[3] = k-block; may be NULL).  Blocks until `stream` is idle.
 * The debug build of the library (libgemmzoo_dbg.so, compiled with -DGZ_BOUNDS_CHECK: every plain
 * global store of the epilogue checks its coordinates against the output matrix first, and a
 * store that fails is skipped) reports GZ_ERR_DEBUG_CHECK here, with detail = {32, block, row,
 * column} of the first refused store. */
GZ_API gz_status gz_last_device_status(gz_plan* plan, void* stream, uint32_t detail[4]);

GZ_API const char* gz_status_string(gz_status s);
/* Text of the last CUDA error seen by this thread inside the library. */
GZ_API const char* gz_last_cuda_error(void);

/* Seeded synthetic operands (replaces nvidia/utils/fill_data.cuh:33-49, which
 * needs 48 bytes of generator state per element).  Element i of a buffer gets a
 * value that depends only on (seed, stream_id, i):
 *   dist 0: uniform in [-1, 1)         (scale multiplies it)
 *   dist 1: normal(0, 1) * scale
 *   dist 2: uniform integers in [-128, 127] (s8) or [-scale, scale] rounded (others)
 * Values are rounded to `dtype` once.  `ptr` is a device pointer. */
GZ_API gz_status gz_fill(void* ptr, int32_t dtype, int64_t count, uint64_t seed, uint32_t stream_id,
                         int32_t dist, float scale, void* stream);

/* Tile-order function of the persistent scheduler, exposed for host tests:
 * linear tile index t -> (tile_m, tile_n) for a tiles_m x tiles_n grid with
 * row-group size group_m. */
GZ_API void gz_tile_coords(uint32_t tiles_m, uint32_t tiles_n, uint32_t group_m, uint32_t t,
                           uint32_t* tile_m, uint32_t* tile_n);

/* Column partition of N over `parts` devices: part p owns [*begin, *end).
 * Boundaries are multiples of `align` columns except the last. */
GZ_API gz_status gz_partition_columns(int64_t n, int32_t parts, int32_t p, int64_t align,
                                      int64_t* begin, int64_t* end);

GZ_API int32_t gz_version(void);

#ifdef __cplusplus
}
#endif
#endif /* GEMMZOO_GEMM_H */
