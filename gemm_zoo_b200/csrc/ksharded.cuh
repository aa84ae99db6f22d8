// K-sharded GEMM with the reduce-scatter fused into the GEMM's epilogue (see
// include/gemmzoo/ksharded.h).  Included at the end of gemm_api.cu: it launches the GEMM through
// run_impl with a ScatterSpec whose pointers are the peers' slot areas.
//
// Workspace of one rank (the owner of one column block), identical on every rank:
//   slots [2 sets][world][m][cols] 4-byte partial sums   (cols = n / world)
//   flags [2 sets][GZ_KS_MAX_WORLD] uint32                (flag[set][g] = epoch of rank g's last push)
// Rank g writes slot [set][g] of EVERY rank's workspace during its GEMM; the last CTA of that GEMM
// to leave then writes flag [set][g] of every rank (GemmParams::signal_count: no second launch);
// the owner reads all of its slots once all of its flags show the current epoch.
#ifndef GZ_KSHARDED_CUH
#define GZ_KSHARDED_CUH

#include "gemmzoo/ksharded.h"

namespace {

constexpr uint32_t KS_WAIT_PEER_FLAG = 16;  // status code: the reduce kernel gave up waiting for a peer

struct KsLayout {
  size_t slot_elems;  // m * cols
  size_t set_elems;   // world * slot_elems
  size_t flags_off;   // byte offset of the flags
  size_t bytes;
};

KsLayout ks_layout(int64_t m, int64_t cols, int world) {
  KsLayout l;
  l.slot_elems = (size_t)m * (size_t)cols;
  l.set_elems = l.slot_elems * (size_t)world;
  l.flags_off = (2 * l.set_elems * 4 + 255) & ~(size_t)255;
  l.bytes = l.flags_off + 2 * GZ_KS_MAX_WORLD * sizeof(uint32_t);
  l.bytes = (l.bytes + 255) & ~(size_t)255;
  return l;
}


template <typename TOut>
struct KsOut;
template <>
struct KsOut<float> {
  static __device__ float load(const float* p) { return *p; }
  static __device__ void store(float* p, float v) { *p = v; }
};
template <>
struct KsOut<__half> {
  static __device__ float load(const __half* p) { return __half2float(*p); }
  static __device__ void store(__half* p, float v) { *p = __float2half_rn(v); }
};
template <>
struct KsOut<__nv_bfloat16> {
  static __device__ float load(const __nv_bfloat16* p) { return __bfloat162float(*p); }
  static __device__ void store(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
};

struct KsReduceParams {
  const void* slots;       // this rank's set: [world][m][cols] partial sums
  const uint32_t* flags;   // this rank's flags of the set: [GZ_KS_MAX_WORLD]
  const void* c;
  void* d;
  int64_t ldc, ldd;
  uint32_t m, cols;
  int world;
  uint32_t epoch;
  float alpha_f, beta_f;
  int32_t alpha_i, beta_i;
  uint32_t* status;  // 4 words
  uint64_t wait_limit_ns;
};

// Wait (bounded) until every rank's flag shows `epoch`, then D = alpha * sum_g slot[g] + beta * C.
// The slots are added in rank order, so the result does not depend on arrival order.
template <typename TOut, bool INT>
__global__ void __launch_bounds__(256) ks_reduce_kernel(const KsReduceParams p) {
  __shared__ uint32_t give_up;
  if (threadIdx.x == 0) {
    uint32_t bad = 0;
    uint64_t t0 = 0;
    for (int g = 0; g < p.world && !bad; ++g) {
      const volatile uint32_t* f = p.flags + g;
      uint32_t spins = 0;
      while (*f != p.epoch) {
        if ((++spins & 63u) == 0u) {
          const uint64_t now = gz::ptx::globaltimer_ns();
          if (t0 == 0) {
            t0 = now;
          } else if (now - t0 > p.wait_limit_ns) {
            if (atomicCAS(p.status, 0u, KS_WAIT_PEER_FLAG) == 0u) {
              p.status[1] = blockIdx.x;
              p.status[2] = static_cast<uint32_t>(g);
              p.status[3] = p.epoch;
            }
            bad = 1;
            break;
          }
          __nanosleep(200);
        }
      }
    }
    __threadfence_system();
    give_up = bad;
  }
  __syncthreads();
  if (give_up) return;

  const size_t slot_elems = static_cast<size_t>(p.m) * p.cols;
  const uint32_t quads_per_row = p.cols / 4u;  // cols is a multiple of 32
  const size_t total = static_cast<size_t>(p.m) * quads_per_row;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const uint32_t row = static_cast<uint32_t>(i / quads_per_row);
    const uint32_t col = static_cast<uint32_t>(i % quads_per_row) * 4u;
    const size_t off = static_cast<size_t>(row) * p.cols + col;
    if constexpr (INT) {
      const int32_t* s = static_cast<const int32_t*>(p.slots);
      uint32_t acc[4] = {0u, 0u, 0u, 0u};
      for (int g = 0; g < p.world; ++g) {
        const int4 v = __ldcg(reinterpret_cast<const int4*>(s + g * slot_elems + off));
        acc[0] += static_cast<uint32_t>(v.x);
        acc[1] += static_cast<uint32_t>(v.y);
        acc[2] += static_cast<uint32_t>(v.z);
        acc[3] += static_cast<uint32_t>(v.w);
      }
      int32_t* drow = static_cast<int32_t*>(p.d) + static_cast<int64_t>(row) * p.ldd + col;
      const int32_t* crow = static_cast<const int32_t*>(p.c) + static_cast<int64_t>(row) * p.ldc + col;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        uint32_t v = static_cast<uint32_t>(p.alpha_i) * acc[e];
        if (p.beta_i != 0) v += static_cast<uint32_t>(p.beta_i) * static_cast<uint32_t>(crow[e]);
        drow[e] = static_cast<int32_t>(v);
      }
    } else {
      const float* s = static_cast<const float*>(p.slots);
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
      for (int g = 0; g < p.world; ++g) {
        const float4 v = __ldcg(reinterpret_cast<const float4*>(s + g * slot_elems + off));
        acc[0] += v.x;
        acc[1] += v.y;
        acc[2] += v.z;
        acc[3] += v.w;
      }
      TOut* drow = static_cast<TOut*>(p.d) + static_cast<int64_t>(row) * p.ldd + col;
      const TOut* crow = static_cast<const TOut*>(p.c) + static_cast<int64_t>(row) * p.ldc + col;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float v = p.alpha_f * acc[e];
        if (p.beta_f != 0.0f) v = fmaf(p.beta_f, KsOut<TOut>::load(crow + e), v);
        KsOut<TOut>::store(drow + e, v);
      }
    }
  }
}

}  // namespace

struct gz_ks_plan {
  gz_ks_desc d;
  gz_plan* gemm;  // local GEMM into 4-byte partial sums, alpha = 1, beta = 0
  KsLayout layout;
  int64_t cols;
  void* ws[GZ_KS_MAX_WORLD];
  uint32_t epoch;      // of the last push
  uint32_t* status;    // device, 4 words
  int sm_count;
};

extern "C" {

GZ_API gz_status gz_ks_workspace_bytes(const gz_ks_desc* desc, size_t* bytes) {
  if (!desc || !bytes || desc->struct_size != sizeof(gz_ks_desc)) return GZ_ERR_INVALID_ARG;
  if (desc->world < 1 || desc->world > GZ_KS_MAX_WORLD || desc->rank < 0 || desc->rank >= desc->world)
    return GZ_ERR_INVALID_ARG;
  if (desc->m <= 0 || desc->n <= 0 || desc->k_local <= 0) return GZ_ERR_INVALID_ARG;
  if (desc->n % (32 * desc->world) != 0) return GZ_ERR_UNSUPPORTED;
  *bytes = ks_layout(desc->m, desc->n / desc->world, desc->world).bytes;
  return GZ_OK;
}

GZ_API gz_status gz_ipc_alloc(size_t bytes, void** ptr, unsigned char handle[GZ_IPC_HANDLE_BYTES]) {
  static_assert(sizeof(cudaIpcMemHandle_t) == GZ_IPC_HANDLE_BYTES, "IPC handle size");
  if (!ptr || !handle || bytes == 0) return GZ_ERR_INVALID_ARG;
  *ptr = nullptr;
  void* p = nullptr;
  if (!cuda_ok(cudaMalloc(&p, bytes), "cudaMalloc(shared workspace)")) return GZ_ERR_OUT_OF_MEMORY;
  cudaIpcMemHandle_t h;
  if (!cuda_ok(cudaMemset(p, 0, bytes), "cudaMemset(shared workspace)") ||
      !cuda_ok(cudaDeviceSynchronize(), "cudaDeviceSynchronize") ||
      !cuda_ok(cudaIpcGetMemHandle(&h, p), "cudaIpcGetMemHandle")) {
    cudaFree(p);
    return GZ_ERR_CUDA;
  }
  std::memcpy(handle, &h, sizeof(h));
  *ptr = p;
  return GZ_OK;
}

GZ_API gz_status gz_ipc_open(const unsigned char handle[GZ_IPC_HANDLE_BYTES], void** ptr) {
  if (!ptr || !handle) return GZ_ERR_INVALID_ARG;
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle, sizeof(h));
  void* p = nullptr;
  if (!cuda_ok(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle"))
    return GZ_ERR_CUDA;
  *ptr = p;
  return GZ_OK;
}

GZ_API gz_status gz_ipc_close(void* ptr) {
  if (!ptr) return GZ_ERR_INVALID_ARG;
  return cuda_ok(cudaIpcCloseMemHandle(ptr), "cudaIpcCloseMemHandle") ? GZ_OK : GZ_ERR_CUDA;
}

GZ_API gz_status gz_ipc_free(void* ptr) {
  if (!ptr) return GZ_ERR_INVALID_ARG;
  return cuda_ok(cudaFree(ptr), "cudaFree") ? GZ_OK : GZ_ERR_CUDA;
}

GZ_API gz_status gz_ks_plan_create(gz_ks_plan** out, const gz_ks_desc* desc, void* const* workspaces) {
  if (!out) return GZ_ERR_INVALID_ARG;
  *out = nullptr;
  size_t bytes = 0;
  gz_status st = gz_ks_workspace_bytes(desc, &bytes);
  if (st != GZ_OK) return st;
  if (!workspaces) return GZ_ERR_INVALID_ARG;
  for (int g = 0; g < desc->world; ++g)
    if (!workspaces[g] || reinterpret_cast<uintptr_t>(workspaces[g]) % 256 != 0) return GZ_ERR_INVALID_ARG;
  const bool s8 = desc->in_type == GZ_DT_S8;
  if (!pair_supported(desc->in_type, desc->out_type)) return GZ_ERR_UNSUPPORTED;
  if (s8 && desc->out_type != GZ_DT_S32) return GZ_ERR_UNSUPPORTED;  // int32 slots are added as integers

  gz_gemm_desc gd;
  std::memset(&gd, 0, sizeof(gd));
  gd.struct_size = sizeof(gd);
  gd.in_type = desc->in_type;
  gd.out_type = s8 ? GZ_DT_S32 : GZ_DT_F32;
  gd.layout_a = desc->layout_a;
  gd.layout_b = desc->layout_b;
  gd.m = desc->m;
  gd.n = desc->n;
  gd.k = desc->k_local;
  gd.lda = desc->lda;
  gd.ldb = desc->ldb;
  gd.ldd = desc->n;  // only validated; the launch writes through the scatter pointers
  gd.device = desc->device;
  gd.config = GZ_CFG_AUTO;
  gd.flags = GZ_FLAG_EPILOGUE_DIRECT;
  gd.wait_limit_ns = desc->wait_limit_ns;

  gz_ks_plan* pl = new (std::nothrow) gz_ks_plan();
  if (!pl) return GZ_ERR_OUT_OF_MEMORY;
  pl->d = *desc;
  if (pl->d.wait_limit_ns == 0) pl->d.wait_limit_ns = 2000000000ull;
  pl->gemm = nullptr;
  pl->status = nullptr;
  pl->epoch = 0;
  pl->cols = desc->n / desc->world;
  pl->layout = ks_layout(desc->m, pl->cols, desc->world);
  for (int g = 0; g < GZ_KS_MAX_WORLD; ++g) pl->ws[g] = g < desc->world ? workspaces[g] : nullptr;
  st = gz_gemm_plan_create(&pl->gemm, &gd);
  if (st == GZ_OK && pl->gemm->info.config == GZ_CFG_SIMT) st = GZ_ERR_MISALIGNED;
  if (st != GZ_OK) {
    if (pl->gemm) gz_gemm_plan_destroy(pl->gemm);
    delete pl;
    return st;
  }
  pl->sm_count = pl->gemm->info.sm_count;
  DeviceGuard guard(desc->device);
  // four status words and the arrival counter of the completion signal
  if (!guard.ok() || !cuda_ok(cudaMalloc(&pl->status, 8 * sizeof(uint32_t)), "cudaMalloc(status)") ||
      !cuda_ok(cudaMemset(pl->status, 0, 8 * sizeof(uint32_t)), "cudaMemset(status)")) {
    if (pl->status) cudaFree(pl->status);
    gz_gemm_plan_destroy(pl->gemm);
    delete pl;
    return GZ_ERR_CUDA;
  }
  *out = pl;
  return GZ_OK;
}

GZ_API gz_status gz_ks_plan_destroy(gz_ks_plan* pl) {
  if (!pl) return GZ_ERR_INVALID_ARG;
  DeviceGuard guard(pl->d.device);
  if (pl->status) cudaFree(pl->status);
  if (pl->gemm) gz_gemm_plan_destroy(pl->gemm);
  delete pl;
  return GZ_OK;
}

GZ_API gz_status gz_ks_push(gz_ks_plan* pl, const void* a, const void* b, void* stream_v) {
  if (!pl || !a || !b) return GZ_ERR_INVALID_ARG;
  DeviceGuard guard(pl->d.device);
  if (!guard.ok()) return GZ_ERR_CUDA;
  const uint32_t epoch = pl->epoch + 1u;
  const uint32_t set = epoch & 1u;
  ScatterSpec sc;
  sc.cols = (uint32_t)pl->cols;
  sc.parts = pl->d.world;
  sc.ld = pl->cols;
  sc.signal_count = pl->d.world;
  sc.signal_value = epoch;
  sc.signal_counter = pl->status + 4;  // the word after the four status words
  for (int g = 0; g < GZ_KS_MAX_WORLD; ++g) {
    sc.ptrs[g] = nullptr;
    sc.signal_ptrs[g] = nullptr;
    if (g >= pl->d.world) continue;
    char* base = static_cast<char*>(pl->ws[g]);
    // my slot in owner g's set, and my flag there
    sc.ptrs[g] = base + (set * pl->layout.set_elems + (size_t)pl->d.rank * pl->layout.slot_elems) * 4;
    sc.signal_ptrs[g] = reinterpret_cast<uint32_t*>(base + pl->layout.flags_off) + set * GZ_KS_MAX_WORLD + pl->d.rank;
  }
  const float one_f = 1.0f, zero_f = 0.0f;
  const int32_t one_i = 1, zero_i = 0;
  const bool s8 = pl->d.in_type == GZ_DT_S8;
  gz_status st = run_impl(pl->gemm, a, b, nullptr, sc.ptrs[pl->d.rank], s8 ? (const void*)&one_i : (const void*)&one_f,
                          s8 ? (const void*)&zero_i : (const void*)&zero_f, stream_v, &sc);
  if (st != GZ_OK) return st;
  pl->epoch = epoch;
  return GZ_OK;
}

GZ_API gz_status gz_ks_reduce(gz_ks_plan* pl, const void* c, void* d, int64_t ldc, int64_t ldd,
                              const void* alpha, const void* beta, void* stream_v) {
  if (!pl || !d || pl->epoch == 0) return GZ_ERR_INVALID_ARG;
  DeviceGuard guard(pl->d.device);
  if (!guard.ok()) return GZ_ERR_CUDA;
  float af, bf;
  int32_t ai, bi;
  gz_status st = read_scalars(pl->gemm->pr, alpha, beta, &af, &bf, &ai, &bi);
  if (st != GZ_OK) return st;
  const bool s8 = pl->d.in_type == GZ_DT_S8;
  const bool beta_zero = s8 ? (bi == 0) : (bf == 0.0f);
  if (!beta_zero && !c) return GZ_ERR_INVALID_ARG;
  if (ldc == 0) ldc = pl->cols;
  if (ldd == 0) ldd = pl->cols;
  if (ldd < pl->cols || (!beta_zero && ldc < pl->cols)) return GZ_ERR_INVALID_ARG;
  const uint32_t set = pl->epoch & 1u;
  char* base = static_cast<char*>(pl->ws[pl->d.rank]);
  KsReduceParams rp;
  rp.slots = base + set * pl->layout.set_elems * 4;
  rp.flags = reinterpret_cast<const uint32_t*>(base + pl->layout.flags_off) + set * GZ_KS_MAX_WORLD;
  rp.c = beta_zero ? nullptr : c;
  rp.d = d;
  rp.ldc = ldc;
  rp.ldd = ldd;
  rp.m = (uint32_t)pl->d.m;
  rp.cols = (uint32_t)pl->cols;
  rp.world = pl->d.world;
  rp.epoch = pl->epoch;
  rp.alpha_f = af;
  rp.beta_f = beta_zero ? 0.0f : bf;
  rp.alpha_i = ai;
  rp.beta_i = beta_zero ? 0 : bi;
  rp.status = pl->status;
  rp.wait_limit_ns = pl->d.wait_limit_ns;
  const size_t quads = (size_t)pl->d.m * (size_t)(pl->cols / 4);
  size_t blocks = (quads + 255) / 256;
  const size_t cap = (size_t)pl->sm_count * 4;  // every block polls the flags: keep them co-resident
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  switch (pl->d.out_type) {
    case GZ_DT_F32: ks_reduce_kernel<float, false><<<(unsigned)blocks, 256, 0, stream>>>(rp); break;
    case GZ_DT_F16: ks_reduce_kernel<__half, false><<<(unsigned)blocks, 256, 0, stream>>>(rp); break;
    case GZ_DT_BF16: ks_reduce_kernel<__nv_bfloat16, false><<<(unsigned)blocks, 256, 0, stream>>>(rp); break;
    case GZ_DT_S32: ks_reduce_kernel<float, true><<<(unsigned)blocks, 256, 0, stream>>>(rp); break;
    default: return GZ_ERR_UNSUPPORTED;
  }
  if (!cuda_ok(cudaGetLastError(), "reduce kernel launch")) return GZ_ERR_CUDA;
  return GZ_OK;
}

GZ_API gz_status gz_ks_run(gz_ks_plan* pl, const void* a, const void* b, const void* c, void* d,
                           int64_t ldc, int64_t ldd, const void* alpha, const void* beta, void* stream_v) {
  gz_status st = gz_ks_push(pl, a, b, stream_v);
  if (st != GZ_OK) return st;
  return gz_ks_reduce(pl, c, d, ldc, ldd, alpha, beta, stream_v);
}

GZ_API gz_status gz_ks_status(gz_ks_plan* pl, void* stream_v, uint32_t detail[4]) {
  if (!pl) return GZ_ERR_INVALID_ARG;
  uint32_t inner[4] = {0, 0, 0, 0};
  gz_status st = gz_last_device_status(pl->gemm, stream_v, inner);  // synchronises the stream
  if (st == GZ_ERR_CUDA) return st;
  DeviceGuard guard(pl->d.device);
  if (!guard.ok()) return GZ_ERR_CUDA;
  uint32_t h[4] = {0, 0, 0, 0};
  if (!cuda_ok(cudaMemcpy(h, pl->status, sizeof(h), cudaMemcpyDeviceToHost), "read status")) return GZ_ERR_CUDA;
  if (h[0] != 0) (void)cudaMemset(pl->status, 0, sizeof(h));
  if (st == GZ_ERR_DEVICE_TIMEOUT) {
    if (detail) std::memcpy(detail, inner, sizeof(inner));
    return st;
  }
  if (detail) std::memcpy(detail, h, sizeof(h));
  return h[0] != 0 ? GZ_ERR_DEVICE_TIMEOUT : GZ_OK;
}

}  // extern "C"
#endif
