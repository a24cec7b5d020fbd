// Philox4x32-10 (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3", SC'11):
// counter-based, so the dropout mask of an element depends only on the seed and on the
// element's own coordinates, never on which thread or tile computes it. The mask of
// element (pair, column c) of h is word c % 4 of the block with counter
// (c / 4, pair, 0, 0) and key (seed_lo, seed_hi); tests/philox_ref.py restates the same
// function in numpy so that the CPU oracle can apply the identical mask
// (reference model.py:164,183: nn.Dropout on h).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace moe {

__host__ __device__ __forceinline__ uint4 philox4x32_10(uint32_t c0, uint32_t c1, uint32_t k0,
                                                        uint32_t k1) {
  constexpr uint32_t kM0 = 0xD2511F53u, kM1 = 0xCD9E8D57u;
  constexpr uint32_t kW0 = 0x9E3779B9u, kW1 = 0xBB67AE85u;
  uint32_t c2 = 0u, c3 = 0u;
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint64_t p0 = (uint64_t)kM0 * c0;
    const uint64_t p1 = (uint64_t)kM1 * c2;
    const uint32_t n0 = (uint32_t)(p1 >> 32) ^ c1 ^ k0;
    const uint32_t n1 = (uint32_t)p1;
    const uint32_t n2 = (uint32_t)(p0 >> 32) ^ c3 ^ k1;
    const uint32_t n3 = (uint32_t)p0;
    c0 = n0; c1 = n1; c2 = n2; c3 = n3;
    k0 += kW0;
    k1 += kW1;
  }
  return make_uint4(c0, c1, c2, c3);
}

}  // namespace moe
