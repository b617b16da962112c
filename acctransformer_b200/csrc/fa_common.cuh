// Device helpers shared by the forward and backward attention kernels.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

namespace acct {

constexpr float kNegInf = -INFINITY;

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// max of three values in one instruction
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

// Two-wide fp32 arithmetic on a register pair: one issue slot for two lanes of work.
__device__ __forceinline__ uint64_t f2_pack(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void f2_unpack(uint64_t r, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(r));
}
__device__ __forceinline__ uint64_t f2_fma(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t f2_add(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ uint64_t f2_mul(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}

template <bool BF16>
__device__ __forceinline__ uint32_t pack2(float a, float b) {
  if constexpr (BF16) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  } else {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
}

template <bool BF16>
__device__ __forceinline__ float load16(const void* base, int64_t idx) {
  if constexpr (BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(base)[idx]);
  else return __half2float(reinterpret_cast<const __half*>(base)[idx]);
}

__device__ __forceinline__ float load_mask_value(const void* base, int dtype, int64_t idx) {
  if (dtype == 2 /*U8*/) return static_cast<float>(reinterpret_cast<const uint8_t*>(base)[idx]);
  if (dtype == 1 /*BF16*/) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(base)[idx]);
  return __half2float(reinterpret_cast<const __half*>(base)[idx]);
}

// 32 consecutive values (elements idx0 .. idx0+31 of a u8 / f16 / bf16 array) as floats, times `mul`.
// `vec` (uniform): idx0 is a multiple of 16 elements and all 32 elements exist, so 128-bit loads are used;
// otherwise element loads, with elements at or past `n_valid` read as 0.
__device__ __forceinline__ void load_row32(const void* base, int dtype, int64_t idx0, int n_valid, bool vec, float mul,
                                           float (&out)[32]) {
  if (vec) {
    if (dtype == 2 /*U8*/) {
      const uint4* p = reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(base) + idx0);
#pragma unroll
      for (int v = 0; v < 2; ++v) {
        const uint4 u = p[v];
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int k = 0; k < 4; ++k)
#pragma unroll
          for (int bb = 0; bb < 4; ++bb) out[v * 16 + k * 4 + bb] = static_cast<float>((w[k] >> (8 * bb)) & 0xffu) * mul;
      }
    } else {
      const uint4* p = reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(base) + idx0);
#pragma unroll
      for (int v = 0; v < 4; ++v) {
        const uint4 u = p[v];
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          float lo, hi;
          if (dtype == 1 /*BF16*/) {
            lo = __uint_as_float(w[k] << 16);
            hi = __uint_as_float(w[k] & 0xffff0000u);
          } else {
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[k]));
            lo = f.x;
            hi = f.y;
          }
          out[v * 8 + k * 2] = lo * mul;
          out[v * 8 + k * 2 + 1] = hi * mul;
        }
      }
    }
  } else {
    // element loads from clamped (always valid) addresses, all issued before the first conversion
    const int last = max(n_valid, 1) - 1;
    if (dtype == 2 /*U8*/) {
      const uint8_t* p = reinterpret_cast<const uint8_t*>(base) + idx0;
      uint8_t raw[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) raw[i] = p[min(i, last)];
#pragma unroll
      for (int i = 0; i < 32; ++i) out[i] = i < n_valid ? static_cast<float>(raw[i]) * mul : 0.f;
    } else {
      const uint16_t* p = reinterpret_cast<const uint16_t*>(base) + idx0;
      uint16_t raw[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) raw[i] = p[min(i, last)];
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const float f = dtype == 1 ? __uint_as_float(static_cast<uint32_t>(raw[i]) << 16) : __half2float(__ushort_as_half(raw[i]));
        out[i] = i < n_valid ? f * mul : 0.f;
      }
    }
  }
}

// 32 values taken down a column of a row-major u8 / f16 / bf16 matrix: element (row_base + min(row0 + e, row_max),
// col) for e = 0..31, as floats times `mul`.  The element-type switch sits outside the loops and all 32 loads
// are issued before the first conversion, so that their latencies overlap.
__device__ __forceinline__ void load_col32(const void* base, int dtype, int64_t row_base, int row0, int row_max,
                                           int64_t row_stride, int col, float mul, float (&out)[32]) {
  if (dtype == 2 /*U8*/) {
    const uint8_t* p = reinterpret_cast<const uint8_t*>(base) + col;
    uint8_t raw[32];
#pragma unroll
    for (int e = 0; e < 32; ++e) raw[e] = p[(row_base + min(row0 + e, row_max)) * row_stride];
#pragma unroll
    for (int e = 0; e < 32; ++e) out[e] = static_cast<float>(raw[e]) * mul;
  } else {
    const uint16_t* p = reinterpret_cast<const uint16_t*>(base) + col;
    uint16_t raw[32];
#pragma unroll
    for (int e = 0; e < 32; ++e) raw[e] = p[(row_base + min(row0 + e, row_max)) * row_stride];
    if (dtype == 1 /*BF16*/) {
#pragma unroll
      for (int e = 0; e < 32; ++e) out[e] = __uint_as_float(static_cast<uint32_t>(raw[e]) << 16) * mul;
    } else {
#pragma unroll
      for (int e = 0; e < 32; ++e) out[e] = __half2float(__ushort_as_half(raw[e])) * mul;
    }
  }
}

// The same 32 values as load_col32, left raw and packed two to a register (element e in the low or high half of
// word e / 2), so that 32 loads can be in flight at a cost of 16 registers; col_value() converts one on use.
template <int NW>   // NW words = 2 * NW values
__device__ __forceinline__ void load_col_raw(const void* base, int dtype, int64_t row_base, int row0, int row_max,
                                             int64_t row_stride, int col, uint32_t (&raw)[NW]) {
  if (dtype == 2 /*U8*/) {
    const uint8_t* p = reinterpret_cast<const uint8_t*>(base) + col;
#pragma unroll
    for (int e = 0; e < NW; ++e) {
      const uint32_t lo = p[(row_base + min(row0 + 2 * e, row_max)) * row_stride];
      const uint32_t hi = p[(row_base + min(row0 + 2 * e + 1, row_max)) * row_stride];
      raw[e] = lo | (hi << 16);
    }
  } else {
    const uint16_t* p = reinterpret_cast<const uint16_t*>(base) + col;
#pragma unroll
    for (int e = 0; e < NW; ++e) {
      const uint32_t lo = p[(row_base + min(row0 + 2 * e, row_max)) * row_stride];
      const uint32_t hi = p[(row_base + min(row0 + 2 * e + 1, row_max)) * row_stride];
      raw[e] = lo | (hi << 16);
    }
  }
}
__device__ __forceinline__ void load_col32_raw(const void* base, int dtype, int64_t row_base, int row0, int row_max,
                                               int64_t row_stride, int col, uint32_t (&raw)[16]) {
  load_col_raw<16>(base, dtype, row_base, row0, row_max, row_stride, col, raw);
}

// element `odd` (0 or 1) of a word written by load_col32_raw, as a float
__device__ __forceinline__ float col_value(uint32_t word, int dtype, int odd) {
  const uint32_t h = odd ? (word >> 16) : (word & 0xffffu);
  if (dtype == 2 /*U8*/) return static_cast<float>(h);
  if (dtype == 1 /*BF16*/) return __uint_as_float(h << 16);
  return __half2float(__ushort_as_half(static_cast<unsigned short>(h)));
}

// Philox4x32-10 (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3", SC'11): a counter-based generator,
// so every (batch*head, query, key) position gets its random byte from its coordinates alone and the forward and
// the backward reproduce the same dropout mask without storing it.
__device__ __forceinline__ uint4 philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, uint32_t k0, uint32_t k1) {
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
    c0 = hi1 ^ c1 ^ k0;
    c1 = lo1;
    c2 = hi0 ^ c3 ^ k1;
    c3 = lo0;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  return make_uint4(c0, c1, c2, c3);
}

// In-kernel dropout.  One Philox call, counter (query, key >> 4, batch*heads + head, offset) and key
// (seed low, seed high), yields 16 bytes; the byte of key position k is byte (k & 15) of the result, taken
// little-endian from the four words; the position is KEPT iff that byte < threshold, threshold =
// round(keep_prob * 256).  Bit i of the returned word: position (key16 * 16 + i) is kept.
struct DropoutRng {
  uint32_t seed_lo, seed_hi, offset, threshold;
};
__device__ __forceinline__ uint32_t dropout_keep16(const DropoutRng& g, uint32_t bh, uint32_t q, uint32_t key16) {
  const uint4 r = philox4x32_10(q, key16, bh, g.offset, g.seed_lo, g.seed_hi);
  const uint32_t w[4] = {r.x, r.y, r.z, r.w};
  if (g.threshold >= 256u) return 0xffffu;         // keep everything (a byte is always below 256)
  const uint32_t t4 = g.threshold * 0x01010101u;
  uint32_t bits = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    // four byte compares at once, then the four 0/1 bytes gathered into a nibble by one multiplication
    // (the partial products land on distinct bits: 24..27 hold byte 0..3's decision)
    const uint32_t ones = __vcmpltu4(w[i], t4) & 0x01010101u;
    bits |= ((ones * 0x01020408u) >> 24 & 0xfu) << (4 * i);
  }
  return bits;
}

// The same decisions as dropout_keep16, left as byte masks: byte i of word i / 4 ... i.e. m[w] has 0xff in byte k iff
// key 4 * w + k of the 16 is kept.  One four-byte compare per word instead of sixteen extractions.
__device__ __forceinline__ void dropout_keep16_bytes(const DropoutRng& g, uint32_t bh, uint32_t q, uint32_t key16,
                                                     uint32_t (&m)[4]) {
  const uint4 r = philox4x32_10(q, key16, bh, g.offset, g.seed_lo, g.seed_hi);
  const uint32_t t4 = min(g.threshold, 255u) * 0x01010101u;   // (the kernels use the generator only below 256)
  m[0] = __vcmpltu4(r.x, t4);
  m[1] = __vcmpltu4(r.y, t4);
  m[2] = __vcmpltu4(r.z, t4);
  m[3] = __vcmpltu4(r.w, t4);
}

}  // namespace acct
