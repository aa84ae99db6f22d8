/* K-sharded GEMM across the GPUs of one node, with the reduce-scatter fused into the GEMM.
 *
 *   D[:, J_r] = alpha * sum_g A[:, K_g] * B[K_g, J_r] + beta * C[:, J_r]      on rank r
 *
 * Rank g holds the K slice (A[:, K_g], B[K_g, :]) and ends up with the column block J_r of D
 * (N / world columns).  No counterpart exists in the reference (it is single-GPU): this serves
 * weights that are already sharded along K, whose fp32 partial products must be reduce-scattered
 * over N.  Instead of computing a full partial and then calling a collective, the
 * GEMM's epilogue stores every column block of its fp32 (int32 for s8) partial sums straight into
 * the memory of the GPU that owns the block (plain peer stores over NVLink, tile by tile while the
 * main loop runs); the CTA of that GEMM that finishes last raises a flag on every peer, and the owner's reduce kernel
 * waits (bounded) for the world's flags, adds the slots in rank order (deterministic), applies
 * alpha/beta and casts.  Two sets of slots alternate, so a rank may start its next GEMM while a
 * slower peer still reduces the previous one.
 *
 * The workspaces are ordinary device allocations shared with the CUDA IPC calls below; how the 64
 * handle bytes travel between the ranks' processes is the caller's business (the Python host side
 * uses torch.distributed).  No multicast object and no TMA load of peer memory is involved.
 */
#ifndef GEMMZOO_KSHARDED_H
#define GEMMZOO_KSHARDED_H

#include "gemmzoo/gemm.h"

#ifdef __cplusplus
extern "C" {
#endif

#define GZ_KS_MAX_WORLD 8
#define GZ_IPC_HANDLE_BYTES 64

typedef struct gz_ks_desc {
  uint32_t struct_size; /* sizeof(gz_ks_desc) */
  int32_t in_type;      /* gz_dtype of A and B */
  int32_t out_type;     /* gz_dtype of C and D (any output type gz_gemm accepts for in_type) */
  int32_t layout_a;     /* of the local slice A[:, K_g] (m x k_local) */
  int32_t layout_b;     /* of the local slice B[K_g, :] (k_local x n) */
  int64_t m, n, k_local;
  int64_t lda, ldb;     /* 0 = packed */
  int32_t world, rank;  /* 1 <= world <= GZ_KS_MAX_WORLD; n must be a multiple of 32 * world */
  int32_t device;
  int32_t reserved;
  uint64_t wait_limit_ns; /* bound on the reduce kernel's wait for the peers' flags; 0 = 2 s */
} gz_ks_desc;

typedef struct gz_ks_plan gz_ks_plan;

/* Bytes of workspace every rank must provide (the same on all ranks). */
GZ_API gz_status gz_ks_workspace_bytes(const gz_ks_desc* desc, size_t* bytes);

/* A zero-filled device allocation on the current device and the IPC handle that lets another
 * process on the node map it; mapping, unmapping and freeing. */
GZ_API gz_status gz_ipc_alloc(size_t bytes, void** ptr, unsigned char handle[GZ_IPC_HANDLE_BYTES]);
GZ_API gz_status gz_ipc_open(const unsigned char handle[GZ_IPC_HANDLE_BYTES], void** ptr);
GZ_API gz_status gz_ipc_close(void* ptr);
GZ_API gz_status gz_ipc_free(void* ptr);

/* workspaces[g] is this process's address of rank g's workspace (its own allocation for g == rank,
 * gz_ipc_open'ed mappings otherwise).  The plan keeps the pointers; it does not own them. */
GZ_API gz_status gz_ks_plan_create(gz_ks_plan** plan, const gz_ks_desc* desc, void* const* workspaces);
GZ_API gz_status gz_ks_plan_destroy(gz_ks_plan* plan);

/* One K-sharded GEMM, asynchronous on `stream`: push (GEMM with scattered output + flag raise),
 * then reduce.  c may be NULL when beta == 0.  c and d are this rank's m x (n / world) blocks with
 * row pitches ldc, ldd (0 = packed).  alpha and beta as for gz_gemm_run (typed by out_type's
 * arithmetic: float, or int32 for s8). */
GZ_API gz_status gz_ks_run(gz_ks_plan* plan, const void* a, const void* b, const void* c, void* d,
                           int64_t ldc, int64_t ldd, const void* alpha, const void* beta, void* stream);

/* The two halves separately, for callers that put other work between them.  Every rank must have
 * issued gz_ks_push before any rank's gz_ks_reduce can complete. */
GZ_API gz_status gz_ks_push(gz_ks_plan* plan, const void* a, const void* b, void* stream);
GZ_API gz_status gz_ks_reduce(gz_ks_plan* plan, const void* c, void* d, int64_t ldc, int64_t ldd,
                              const void* alpha, const void* beta, void* stream);

/* Synchronises `stream` and reports whether a bounded wait gave up since the last call:
 * GZ_ERR_DEVICE_TIMEOUT with detail = {code, block, awaited rank, epoch} (code 16: the reduce
 * kernel's wait for a peer's flag; otherwise the GEMM kernel's codes), GZ_OK otherwise. */
GZ_API gz_status gz_ks_status(gz_ks_plan* plan, void* stream, uint32_t detail[4]);

#ifdef __cplusplus
}
#endif
#endif
