// Which die each SM of a B200 sits on, measured.
//
// A B200 is two dies behind one device; each die has its own SMs, its own half of the L2 and its
// own HBM stacks, and every address has a home on one of them.  A load that misses in the
// requesting die's L2 and is homed on the other die crosses the die-to-die link, which shows as
// extra latency.  Nothing in the programming model names the die of an SM (or of an address), and
// parts differ in which SMs are fused off, so the plan measures it once per device: one CTA per SM
// chases a pointer through each of a set of L2-resident lines and records clocks per load.  For
// every line the SMs fall into a near and a far group; SMs that are near for the same lines share
// a die.  If the picture is not cleanly two-sided (another architecture, a partitioned GPU,
// noise), the result is "unknown" and the die-aware tile order stays off.
#ifndef GZ_PLACEMENT_CUH
#define GZ_PLACEMENT_CUH

#include <cuda_runtime.h>
#include <stdint.h>

#include <vector>

namespace gz {

struct DevicePlacement {
  bool known = false;
  int sm_count = 0;
  int sms_on_die[2] = {0, 0};
  uint8_t die_of_sm[160] = {};
};

namespace placement_detail {

constexpr int kLines = 48;          // probed addresses
constexpr int kLineStride = 163840 + 256;  // bytes between them (spread over L2 slices and both dies)
constexpr int kChase = 24;          // dependent loads per timing
constexpr int kRepeats = 6;         // best of

__global__ void placement_init_kernel(unsigned long long* buf) {
  const int j = threadIdx.x;
  if (j < kLines) {
    unsigned long long* p = buf + static_cast<size_t>(j) * (kLineStride / 8);
    *p = reinterpret_cast<unsigned long long>(p);  // every probed line points at itself
  }
}

// One CTA per SM (the launch asks for enough dynamic shared memory that two cannot share one).
__global__ void placement_probe_kernel(const unsigned long long* buf, uint32_t* out_smid, uint32_t* out_clocks,
                                       unsigned long long* sink) {
  extern __shared__ unsigned char placement_smem[];
  if (threadIdx.x != 0) return;
  uint32_t smid;
  asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
  out_smid[blockIdx.x] = smid;
  unsigned long long acc = 0;
  for (int j = 0; j < kLines; ++j) {
    const volatile unsigned long long* p =
        reinterpret_cast<const volatile unsigned long long*>(buf + static_cast<size_t>(j) * (kLineStride / 8));
    p = reinterpret_cast<const volatile unsigned long long*>(*p);  // bring the line into L2
    uint32_t best = 0xFFFFFFFFu;
    for (int r = 0; r < kRepeats; ++r) {
      const long long t0 = clock64();
#pragma unroll 1
      for (int i = 0; i < kChase; ++i) p = reinterpret_cast<const volatile unsigned long long*>(*p);
      acc += reinterpret_cast<unsigned long long>(p);
      const long long t1 = clock64();
      const uint32_t d = static_cast<uint32_t>(t1 - t0);
      if (d < best) best = d;
    }
    out_clocks[blockIdx.x * kLines + j] = best;
  }
  if (acc == 1ull) *sink = acc;  // keeps the chase alive
}

}  // namespace placement_detail

// Host-side classification, separated from the measurement so that it can be tested without a GPU:
// clocks[sm * lines + j] = cost of line j seen from SM sm.  Returns false unless the SMs split
// cleanly in two.
inline bool classify_dies(const std::vector<uint32_t>& clocks, int sms, int lines, uint8_t* die_of_sm,
                          int sms_on_die[2]) {
  if (sms < 4 || lines < 8 || clocks.size() < static_cast<size_t>(sms) * lines) return false;
  // SMs differ in how far they sit from the L2 as a whole, by about as much as the two dies differ,
  // so every SM is compared with itself: a line is "far" for an SM if it costs more than that SM's
  // mean over all lines (each SM sees about half of the lines on either die).
  std::vector<uint8_t> far(static_cast<size_t>(sms) * lines);
  for (int s = 0; s < sms; ++s) {
    unsigned long long sum = 0;
    for (int j = 0; j < lines; ++j) sum += clocks[static_cast<size_t>(s) * lines + j];
    for (int j = 0; j < lines; ++j)
      far[static_cast<size_t>(s) * lines + j] =
          static_cast<unsigned long long>(clocks[static_cast<size_t>(s) * lines + j]) * lines > sum ? 1 : 0;
  }
  // A line tells something only if a fair share of the SMs sits on either side of it.
  int usable = 0;
  std::vector<uint8_t> line_ok(lines, 0);
  for (int j = 0; j < lines; ++j) {
    int nfar = 0;
    for (int s = 0; s < sms; ++s) nfar += far[static_cast<size_t>(s) * lines + j];
    if (nfar * 5 >= sms && (sms - nfar) * 5 >= sms) {
      line_ok[j] = 1;
      ++usable;
    }
  }
  if (usable < 8) return false;
  // SMs that agree with SM 0 on (nearly) every usable line share its die; those that disagree on
  // (nearly) every line sit on the other; anything in between means the picture is not two-sided.
  sms_on_die[0] = sms_on_die[1] = 0;
  for (int s = 0; s < sms; ++s) {
    int agree = 0;
    for (int j = 0; j < lines; ++j)
      if (line_ok[j] && far[static_cast<size_t>(s) * lines + j] == far[j]) ++agree;
    int die;
    if (agree * 4 >= usable * 3) die = 0;
    else if (agree * 4 <= usable) die = 1;
    else return false;
    die_of_sm[s] = static_cast<uint8_t>(die);
    ++sms_on_die[die];
  }
  return sms_on_die[0] * 4 >= sms && sms_on_die[1] * 4 >= sms;
}

// Measures the placement of `device` (which must be current).  Allocates and frees its own scratch
// memory and synchronises the device: call it from plan creation, never from a launch path.
inline DevicePlacement measure_placement(int sm_count) {
  using namespace placement_detail;
  DevicePlacement out;
  out.sm_count = sm_count;
  if (sm_count < 4 || sm_count > 160) return out;
  const size_t buf_bytes = static_cast<size_t>(kLines) * kLineStride + 4096;
  unsigned long long* buf = nullptr;
  uint32_t *d_smid = nullptr, *d_clocks = nullptr;
  cudaStream_t stream = nullptr;
  const int smem = 160 * 1024;  // more than half of an SM's shared memory: one CTA per SM
  bool ok = cudaMalloc(&buf, buf_bytes) == cudaSuccess && cudaMalloc(&d_smid, sm_count * 4) == cudaSuccess &&
            cudaMalloc(&d_clocks, static_cast<size_t>(sm_count) * kLines * 4) == cudaSuccess &&
            cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking) == cudaSuccess &&
            cudaMemsetAsync(buf, 0, buf_bytes, stream) == cudaSuccess &&
            cudaMemsetAsync(d_smid, 0xFF, sm_count * 4, stream) == cudaSuccess &&
            cudaFuncSetAttribute(placement_probe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) == cudaSuccess;
  if (ok) {
    placement_init_kernel<<<1, 64, 0, stream>>>(buf);
    placement_probe_kernel<<<sm_count, 32, smem, stream>>>(buf, d_smid, d_clocks, buf + 1);
    ok = cudaGetLastError() == cudaSuccess && cudaStreamSynchronize(stream) == cudaSuccess;
  }
  if (ok) {
    std::vector<uint32_t> smid(sm_count), raw(static_cast<size_t>(sm_count) * kLines), by_sm(raw.size(), 0);
    ok = cudaMemcpy(smid.data(), d_smid, sm_count * 4, cudaMemcpyDeviceToHost) == cudaSuccess &&
         cudaMemcpy(raw.data(), d_clocks, raw.size() * 4, cudaMemcpyDeviceToHost) == cudaSuccess;
    std::vector<uint8_t> seen(sm_count, 0);
    for (int b = 0; ok && b < sm_count; ++b) {
      if (smid[b] >= static_cast<uint32_t>(sm_count) || seen[smid[b]]) ok = false;  // not one CTA per SM
      else {
        seen[smid[b]] = 1;
        for (int j = 0; j < kLines; ++j) by_sm[static_cast<size_t>(smid[b]) * kLines + j] = raw[static_cast<size_t>(b) * kLines + j];
      }
    }
    if (ok) out.known = classify_dies(by_sm, sm_count, kLines, out.die_of_sm, out.sms_on_die);
    // The two SMs of a TPC (2t, 2t + 1) sit side by side: a picture that splits one is noise.
    for (int s = 0; out.known && s + 1 < sm_count; s += 2)
      if (out.die_of_sm[s] != out.die_of_sm[s + 1]) out.known = false;
  }
  (void)cudaGetLastError();
  if (stream) cudaStreamDestroy(stream);
  if (buf) cudaFree(buf);
  if (d_smid) cudaFree(d_smid);
  if (d_clocks) cudaFree(d_clocks);
  return out;
}

}  // namespace gz
#endif
