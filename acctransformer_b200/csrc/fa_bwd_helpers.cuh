// Device helpers shared by the two backward kernels (head_dim <= 128 and head_dim in (128, 256]).
#pragma once
#include "fa_common.cuh"
#include "fa_kernels.cuh"

namespace acct {

// Keep bits of in-kernel dropout for one key row and 32 consecutive queries q0 .. q0+31 (bit e = query q0 + e).
// The generator works on (query, 16 consecutive keys); the 32 lanes of a warp hold 32 consecutive key rows, i.e.
// two such groups of 16.  Every lane makes the calls of two of the 32 queries for its half-warp's key group and
// the 16-bit results are handed round by shuffles, so a warp makes 64 calls for its 32 x 32 decisions.
// All 32 lanes must call this together.
__device__ __forceinline__ uint32_t philox_keep_column(const ScoreMods& mods, int bh, int q0, int q_max, int kv_idx,
                                                       int lane) {
  const DropoutRng rng = {mods.drop_seed_lo, mods.drop_seed_hi, mods.drop_offset, mods.drop_threshold};
  const uint32_t key16 = static_cast<uint32_t>(kv_idx) >> 4;
  uint32_t mine[2];
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    const int q = min(q0 + 2 * (lane & 15) + u, q_max);
    mine[u] = dropout_keep16(rng, static_cast<uint32_t>(bh), static_cast<uint32_t>(q), key16);
  }
  uint32_t bits = 0;
#pragma unroll
  for (int e = 0; e < 32; ++e) {
    const uint32_t m16 = __shfl_sync(0xffffffffu, mine[e & 1], (lane & 16) | (e >> 1));
    bits |= ((m16 >> (kv_idx & 15)) & 1u) << e;
  }
  return bits;
}

}  // namespace acct
