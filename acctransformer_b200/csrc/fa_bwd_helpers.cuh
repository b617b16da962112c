// Device helpers shared by the two backward kernels (head_dim <= 128 and head_dim in (128, 256]).
#pragma once
#include "fa_common.cuh"
#include "fa_kernels.cuh"

namespace acct {

// Keep bits of in-kernel dropout for one key row and 32 consecutive queries q0 .. q0+31 (bit e = query q0 + e).
// The generator works on (query, 16 consecutive keys); the 32 lanes of a warp hold 32 consecutive key rows, i.e.
// two such groups of 16.  Every lane makes the calls of two of the 32 queries (q0 + s and q0 + 16 + s, s = lane % 16)
// for its half-warp's key group, which gives each half-warp a 32 x 16 bit matrix spread over its lanes (lane s holds
// rows s and 16 + s, one 16-bit result each); what a lane needs is COLUMN (lane % 16) of it.  The two 16 x 16 blocks
// are transposed in place by four butterfly rounds (one shuffle and a few logic operations each) instead of one
// shuffle per query: a warp makes 64 calls and 4 shuffles per lane for its 32 x 32 decisions.
// All 32 lanes must call this together.
__device__ __forceinline__ uint32_t philox_keep_column(const ScoreMods& mods, int bh, int q0, int q_max, int kv_idx,
                                                       int lane) {
  const DropoutRng rng = {mods.drop_seed_lo, mods.drop_seed_hi, mods.drop_offset, mods.drop_threshold};
  const uint32_t key16 = static_cast<uint32_t>(kv_idx) >> 4;
  uint32_t w = 0;
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    const int q = min(q0 + 16 * u + (lane & 15), q_max);
    w |= dropout_keep16(rng, static_cast<uint32_t>(bh), static_cast<uint32_t>(q), key16) << (16 * u);
  }
  // w: bit 16u + b = (query q0 + 16u + s, key 16*key16 + b).  After the rounds: bit 16u + s' of lane d = the decision
  // of (query q0 + 16u + s', key 16*key16 + d), i.e. bit e of the result belongs to query q0 + e.
#pragma unroll
  for (int k = 3; k >= 0; --k) {
    const uint32_t m = k == 3 ? 0x00ff00ffu : k == 2 ? 0x0f0f0f0fu : k == 1 ? 0x33333333u : 0x55555555u;
    const uint32_t x = __shfl_xor_sync(0xffffffffu, w, 1 << k);
    w = (lane & (1 << k)) ? ((w & ~m) | ((x & ~m) >> (1 << k))) : ((w & m) | ((x & m) << (1 << k)));
  }
  return w;
}

// The same 32 keep bits (bit e = query q0 + e keeps this lane's key) read from a uint8 {0,1} dropout mask
// [units, S_q, S_k]: a lane would otherwise make 32 single-byte loads down a column of the mask, twice per tile.
// Instead lane L loads, for 8 queries q0 + 4i + L/8, the FOUR bytes of keys 4 (L%8) .. +3 of the warp's 32 keys (a
// warp instruction then reads 32 contiguous bytes of each of 4 mask rows), squeezes each word into a nibble, and the
// nibbles travel to the lanes that own the keys by 4 shuffles.  Needs S_k % 4 == 0 and a 4-byte aligned mask;
// addresses are clamped into the row, so keys past S_k get bits of other keys (their P is 0 anyway).
// All 32 lanes must call this together.
// Split in two so that the loads can be in flight under other work: u8_keep_load issues them, u8_keep_bits turns
// the eight words into this lane's 32 bits.
__device__ __forceinline__ void u8_keep_load(const void* drop, int64_t unit_row0, int q0, int q_max, int S_k, int kv_warp0,
                                             int lane, uint32_t (&raw)[8]) {
  const uint8_t* base = reinterpret_cast<const uint8_t*>(drop) + min(kv_warp0 + 4 * (lane & 7), S_k - 4);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int q = min(q0 + 4 * i + (lane >> 3), q_max);
    raw[i] = *reinterpret_cast<const uint32_t*>(base + (unit_row0 + q) * S_k);
  }
}
__device__ __forceinline__ uint32_t u8_keep_bits(const uint32_t (&raw)[8], int lane) {
  uint32_t pw = 0;
#pragma unroll
  for (int i = 0; i < 8; ++i) pw |= ((((raw[i] & 0x01010101u) * 0x01020408u) >> 24) & 0xfu) << (4 * i);
  uint32_t bits = 0;
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    const uint32_t x = __shfl_sync(0xffffffffu, pw, g * 8 + (lane >> 2));
    bits |= ((x >> (lane & 3)) & 0x11111111u) << g;
  }
  return bits;
}

}  // namespace acct
