// Stateless counter-based generator for synthetic operands, identical on host
// and device: value i of a buffer depends only on (seed, stream_id, i).
//
// The reference fills buffers with one XORWOW state per element, all buffers
// from the same seed (nvidia/utils/fill_data.cuh:13-17,42), so A, B and C hold
// the same numbers.  Here each operand has its own stream_id, and no state is
// stored.
#ifndef GZ_RNG_H
#define GZ_RNG_H

#include <stdint.h>

#if defined(__CUDACC__)
#define GZ_RNG_HD __host__ __device__ __forceinline__
#else
#define GZ_RNG_HD inline
#endif

namespace gz {

GZ_RNG_HD uint64_t mix64(uint64_t z) {
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

GZ_RNG_HD uint64_t rng_bits(uint64_t seed, uint32_t stream_id, uint64_t index) {
  return mix64(mix64(seed * 0x100000001B3ull + stream_id) ^ (index * 0xD1342543DE82EF95ull));
}

// uniform in [-1, 1): 24 random bits.
GZ_RNG_HD float rng_uniform_pm1(uint64_t bits) {
  return static_cast<float>(static_cast<uint32_t>(bits >> 40)) * (1.0f / 8388608.0f) - 1.0f;
}

// uniform integer in [-128, 127].
GZ_RNG_HD int32_t rng_int8(uint64_t bits) {
  return static_cast<int32_t>(static_cast<int8_t>(bits & 0xFF));
}

}  // namespace gz
#endif
