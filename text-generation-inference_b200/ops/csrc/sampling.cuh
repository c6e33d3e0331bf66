// Device helpers shared by the single-GPU sampler (fused_ops.cu) and the vocabulary-parallel sampler
// (peer_comm.cu): order-preserving integer image of a float, Philox4x32-10 and the Gumbel noise of entry j.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace tgi_sampling {

__device__ __forceinline__ uint32_t order_bits(float x) {
  const uint32_t u = __float_as_uint(x);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__device__ __forceinline__ uint4 philox4x32(uint32_t c0, uint32_t c1, uint32_t k0, uint32_t k1) {
  uint32_t c[4] = {c0, c1, 0u, 0u};
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, c[0]), lo0 = 0xD2511F53u * c[0];
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, c[2]), lo1 = 0xCD9E8D57u * c[2];
    const uint32_t n0 = hi1 ^ c[1] ^ k0, n1 = lo1, n2 = hi0 ^ c[3] ^ k1, n3 = lo0;
    c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  return make_uint4(c[0], c[1], c[2], c[3]);
}

// j is the index of the entry in the WHOLE vocabulary, so a vocabulary shard draws the same noise for its
// entries as a single GPU that holds all of them
__device__ __forceinline__ float gumbel_noise(uint32_t j, uint32_t step, uint64_t seed) {
  const uint4 r = philox4x32(j >> 2, step, static_cast<uint32_t>(seed), static_cast<uint32_t>(seed >> 32));
  const uint32_t w = (j & 3) == 0 ? r.x : (j & 3) == 1 ? r.y : (j & 3) == 2 ? r.z : r.w;
  const float u = (static_cast<float>(w >> 8) + 0.5f) * (1.0f / 16777216.0f);   // (0, 1)
  return -__logf(-__logf(u));
}

}  // namespace tgi_sampling
