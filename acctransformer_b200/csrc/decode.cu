// Decode (one query token per sequence) over a KV cache: split-KV streaming + merge.
//
// The step is bound by reading K and V once from HBM, so it runs on CUDA cores with 128-bit
// loads: a group of LPR lanes covers one cache row (8 elements each), a warp covers 32/LPR
// consecutive rows per load instruction (one contiguous span of memory), and every thread keeps
// 2*kChunk such loads in flight.  Each lane group carries its own online-softmax state
// (max, sum, partial output slice); states are merged inside the CTA, written per split to the
// workspace, and merged across splits by a second small kernel.
//
// Semantics: y[b,n,0,:] = softmax(scale * q K[:len_b]^T) V[:len_b] -- the q_len = 1 case of the
// reference's inference op (infer/flash_attention/tik/tbe/impl/flash_attention_fwd.py:583-705
// computes the same recurrence with m, l, O kept in global memory).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "fa_kernels.cuh"

namespace acct {
namespace {

constexpr int kDecodeThreads = 128;
constexpr int kChunk = 8;

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ uint4 ld_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

// two fp32 values in one 64-bit register and the two-wide fp32 instructions on them
__device__ __forceinline__ uint64_t pack2f(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2f(uint64_t r, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(r));
}
__device__ __forceinline__ uint64_t fma2f(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t mul2f(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}

template <bool BF16>
__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if constexpr (BF16) {
      f[2 * i] = __uint_as_float(w[i] << 16);
      f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    } else {
      const __half2 h = *reinterpret_cast<const __half2*>(&w[i]);
      const float2 t = __half22float2(h);
      f[2 * i] = t.x;
      f[2 * i + 1] = t.y;
    }
  }
}

// G = query heads per key/value head (grouped-query attention): the G heads of a group share one pass over their
// cache rows, so the cache is read once per group instead of once per query head.
template <int LPR, bool BF16, int G>
__global__ void __launch_bounds__(kDecodeThreads) decode_split_kernel(const DecodeParams p) {
  constexpr int RPW = 32 / LPR;                 // cache rows per warp per load instruction
  constexpr int kWarps = kDecodeThreads / 32;
  constexpr int kGroups = kWarps * RPW;         // independent softmax states per CTA and query head
  constexpr int DMAX = LPR * 8;
  constexpr int kCh = G >= 4 ? kChunk / 2 : kChunk;   // fewer loads in flight when G heads of state are held

  __shared__ float s_m[G][kGroups], s_l[G][kGroups];
  __shared__ float s_acc[G][kGroups][DMAX];

  const int split = blockIdx.x;
  const int n_kv = p.N / G;
  const int unit_kv = blockIdx.y;               // (batch, key/value head)
  const int b = unit_kv / n_kv, h_kv = unit_kv % n_kv;
  int len = p.S_max;
  if (p.seq_lens != nullptr) len = min(p.S_max, max(0, p.seq_lens[b]));
  const int per = (((len + p.splits - 1) / p.splits) + 63) & ~63;
  const int k0 = split * per;
  const int k1 = min(len, k0 + per);

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int sub = lane % LPR, rsub = lane / LPR;
  const int dcol = sub * 8;
  const bool active = dcol < p.D;

  float qf[G][8];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    const int64_t unit = static_cast<int64_t>(b) * p.N + h_kv * G + g;
    uint4 qu = make_uint4(0, 0, 0, 0);
    if (active) qu = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(p.q) + unit * p.D + dcol);
    unpack8<BF16>(qu, qf[g]);
#pragma unroll
    for (int e = 0; e < 8; ++e) qf[g][e] *= p.scale_log2;
  }
  // Contiguous caches: row r of this (batch, head) sits at base + r * row stride.  Paged caches: the page number
  // comes from the block table (rows past the sequence are never dereferenced: the loads below are guarded).
  const bool paged = p.block_table != nullptr;
  const int* table = paged ? p.block_table + static_cast<int64_t>(b) * p.max_pages : nullptr;
  const int64_t head_off = h_kv * p.kv_stride_h + dcol;
  const uint16_t* kbase = reinterpret_cast<const uint16_t*>(p.k) + (paged ? 0 : b * p.kv_stride_b) + head_off;
  const uint16_t* vbase = reinterpret_cast<const uint16_t*>(p.v) + (paged ? 0 : b * p.kv_stride_b) + head_off;
  auto row_offset = [&](int row) -> int64_t {
    if (!paged) return static_cast<int64_t>(row) * p.kv_stride_s;
    const int page = table[row >> p.page_shift];
    return static_cast<int64_t>(page) * p.kv_stride_b + static_cast<int64_t>(row & ((1 << p.page_shift) - 1)) * p.kv_stride_s;
  };

  float m[G], l[G];
  float acc[G][8];
  // G >= 4 (and at least G lanes per row): one head's softmax per lane, see the loop below
  constexpr bool kScatter = G >= 4 && LPR >= G;
  float m_own = -INFINITY, l_own = 0.f;
  uint64_t acc2[G][4];                  // the accumulators as pairs (elements 2e, 2e+1)
  uint64_t q2[(G + 1) / 2][8];          // the scaled queries of heads 2gp, 2gp+1 as pairs
#pragma unroll
  for (int g = 0; g < G; ++g)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc2[g][e] = 0ull;
  if constexpr (kScatter) {
#pragma unroll
    for (int gp = 0; gp < G / 2; ++gp)
#pragma unroll
      for (int e = 0; e < 8; ++e) q2[gp][e] = pack2f(qf[2 * gp][e], qf[2 * gp + 1][e]);
  }
#pragma unroll
  for (int g = 0; g < G; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[g][e] = 0.f;
  }

  // the K and V rows of one step of this warp (kCh row pairs), all loads issued back to back
  auto issue_loads = [&](int row0, uint4 (&ku)[kCh], uint4 (&vu)[kCh]) {
    int64_t off[kCh];
#pragma unroll
    for (int i = 0; i < kCh; ++i) {
      const int row = row0 + i * RPW + rsub;
      off[i] = row < k1 ? row_offset(row) : 0;
    }
#pragma unroll
    for (int i = 0; i < kCh; ++i) {
      const int row = row0 + i * RPW + rsub;
      ku[i] = (active && row < k1) ? ld_stream(kbase + off[i]) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int i = 0; i < kCh; ++i) {
      const int row = row0 + i * RPW + rsub;
      vu[i] = (active && row < k1) ? ld_stream(vbase + off[i]) : make_uint4(0, 0, 0, 0);
    }
  };
  // With several heads of state per thread few CTAs fit an SM, and a warp that only loads, waits and then computes
  // leaves the memory system idle while it computes: there the next step's rows are requested before this step's
  // arithmetic (kAhead).  With one or two heads enough warps are resident for that to happen by itself.
  constexpr int kStep = kWarps * RPW * kCh;
  uint4 ku[kCh], vu[kCh], ku_next[kCh], vu_next[kCh];
  const int row_first = k0 + warp * (RPW * kCh);
  constexpr bool kAhead = kScatter && G >= 8;   // (at G = 4 the registers it takes cost a resident CTA: slower)
  if constexpr (kAhead) { if (row_first < k1) issue_loads(row_first, ku, vu); }
  for (int row0 = row_first; row0 < k1; row0 += kStep) {
    if constexpr (kAhead) {
      if (row0 + kStep < k1) issue_loads(row0 + kStep, ku_next, vu_next);
    } else {
      issue_loads(row0, ku, vu);
    }
    if constexpr (kScatter) {
      // G >= 4: the G partial dot products of a lane are reduce-scattered over the LPR lanes of its row (halving
      // exchanges on the high lane bits, then plain butterfly sums on the rest), so that a lane ends up with the
      // complete score of ONE head, h_own: 8 shuffles instead of 32 per row at G = 8.  The lane runs that head's
      // online softmax alone (one exponential per row instead of G) and hands the rescaling factor and the
      // probabilities (rounded to 16 bits, two to a word, as the training kernels round P) round by shuffles.
      float s_own[kCh];
#pragma unroll
      for (int i = 0; i < kCh; ++i) {
        float kf[8];
        unpack8<BF16>(ku[i], kf);
        uint64_t k2[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) k2[e] = pack2f(kf[e], kf[e]);
        float v[G];
#pragma unroll
        for (int gp = 0; gp < G / 2; ++gp) {
          uint64_t d2 = 0ull;
#pragma unroll
          for (int e = 0; e < 8; ++e) d2 = fma2f(k2[e], q2[gp][e], d2);
          unpack2f(d2, v[2 * gp], v[2 * gp + 1]);
        }
        int cnt = G;
#pragma unroll
        for (int bit = LPR / 2; bit >= 1; bit >>= 1) {
          if (cnt > 1) {
            const bool up = (sub & bit) != 0;
            const int half = cnt / 2;
#pragma unroll
            for (int jj = 0; jj < G / 2; ++jj) {
              if (jj < half) {
                const float send = up ? v[jj] : v[jj + half];
                const float keep = up ? v[jj + half] : v[jj];
                v[jj] = keep + __shfl_xor_sync(0xffffffffu, send, bit);
              }
            }
            cnt = half;
          } else {
            v[0] += __shfl_xor_sync(0xffffffffu, v[0], bit);
          }
        }
        const int row = row0 + i * RPW + rsub;
        s_own[i] = row < k1 ? v[0] : -INFINITY;
      }
      float cmax_own = s_own[0];
#pragma unroll
      for (int i = 1; i < kCh; ++i) cmax_own = fmaxf(cmax_own, s_own[i]);
      const float m_new = fmaxf(m_own, cmax_own);
      const bool any = m_new != -INFINITY;
      const float alpha_own = any ? ex2(m_own - m_new) : 1.0f;   // m_own = -inf gives 0; nothing accumulated then
      float pr_own[kCh];
      float psum = 0.f;
#pragma unroll
      for (int i = 0; i < kCh; ++i) {
        pr_own[i] = any ? ex2(s_own[i] - m_new) : 0.f;
        psum += pr_own[i];
      }
      l_own = fmaf(l_own, alpha_own, psum);
      m_own = m_new;
      uint32_t pr_pack[kCh / 2];
#pragma unroll
      for (int i = 0; i < kCh / 2; ++i) {
        const __half2 h2 = __floats2half2_rn(pr_own[2 * i], pr_own[2 * i + 1]);
        pr_pack[i] = *reinterpret_cast<const uint32_t*>(&h2);
      }
      float vf[kCh][8];
#pragma unroll
      for (int i = 0; i < kCh; ++i) unpack8<BF16>(vu[i], vf[i]);
      uint64_t v2[kCh][4];
#pragma unroll
      for (int i = 0; i < kCh; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) v2[i][e] = pack2f(vf[i][2 * e], vf[i][2 * e + 1]);
#pragma unroll
      for (int g = 0; g < G; ++g) {
        const int src = (lane & ~(LPR - 1)) | (g * (LPR / G));   // first lane of my row that owns head g
        const float alpha = __shfl_sync(0xffffffffu, alpha_own, src);
        const uint64_t alpha2 = pack2f(alpha, alpha);
#pragma unroll
        for (int e = 0; e < 4; ++e) acc2[g][e] = mul2f(acc2[g][e], alpha2);
#pragma unroll
        for (int i2 = 0; i2 < kCh / 2; ++i2) {
          const uint32_t w = __shfl_sync(0xffffffffu, pr_pack[i2], src);
          const float2 pp = __half22float2(*reinterpret_cast<const __half2*>(&w));
          const uint64_t p0 = pack2f(pp.x, pp.x), p1 = pack2f(pp.y, pp.y);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            acc2[g][e] = fma2f(p0, v2[2 * i2][e], acc2[g][e]);
            acc2[g][e] = fma2f(p1, v2[2 * i2 + 1][e], acc2[g][e]);
          }
        }
      }
      if constexpr (kAhead) if (row0 + kStep < k1) {
#pragma unroll
        for (int i = 0; i < kCh; ++i) { ku[i] = ku_next[i]; vu[i] = vu_next[i]; }
      }
    } else {
      float s[G][kCh];
      float cmax[G];
  #pragma unroll
      for (int g = 0; g < G; ++g) cmax[g] = -INFINITY;
  #pragma unroll
      for (int i = 0; i < kCh; ++i) {
        float kf[8];
        unpack8<BF16>(ku[i], kf);
        const int row = row0 + i * RPW + rsub;
  #pragma unroll
        for (int g = 0; g < G; ++g) {
          float d = 0.f;
  #pragma unroll
          for (int e = 0; e < 8; ++e) d = fmaf(kf[e], qf[g][e], d);
  #pragma unroll
          for (int off = 1; off < LPR; off <<= 1) d += __shfl_xor_sync(0xffffffffu, d, off);
          s[g][i] = row < k1 ? d : -INFINITY;
          cmax[g] = fmaxf(cmax[g], s[g][i]);
        }
      }
      float vf[kCh][8];
  #pragma unroll
      for (int i = 0; i < kCh; ++i) unpack8<BF16>(vu[i], vf[i]);
  #pragma unroll
      for (int g = 0; g < G; ++g) {
        const float m_new = fmaxf(m[g], cmax[g]);
        if (m_new != -INFINITY) {
          const float alpha = ex2(m[g] - m_new);   // m = -inf gives 0
          l[g] *= alpha;
  #pragma unroll
          for (int e = 0; e < 8; ++e) acc[g][e] *= alpha;
          m[g] = m_new;
  #pragma unroll
          for (int i = 0; i < kCh; ++i) {
            const float pr = ex2(s[g][i] - m_new);
            l[g] += pr;
  #pragma unroll
            for (int e = 0; e < 8; ++e) acc[g][e] = fmaf(pr, vf[i][e], acc[g][e]);
          }
        }
      }
  
    }
  }
  if constexpr (kScatter) {
    // back to the per-head state the merge below expects
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const int src = (lane & ~(LPR - 1)) | (g * (LPR / G));
      m[g] = __shfl_sync(0xffffffffu, m_own, src);
      l[g] = __shfl_sync(0xffffffffu, l_own, src);
#pragma unroll
      for (int e = 0; e < 4; ++e) unpack2f(acc2[g][e], acc[g][2 * e], acc[g][2 * e + 1]);
    }
  }

  // merge the CTA's groups, per query head
  const int grp = warp * RPW + rsub;
#pragma unroll
  for (int g = 0; g < G; ++g) {
    if (sub == 0) { s_m[g][grp] = m[g]; s_l[g][grp] = l[g]; }
#pragma unroll
    for (int e = 0; e < 8; ++e) s_acc[g][grp][dcol + e] = acc[g][e];
  }
  __syncthreads();
#pragma unroll 1
  for (int g = 0; g < G; ++g) {
    const int64_t unit = static_cast<int64_t>(b) * p.N + h_kv * G + g;
    const int64_t slot = unit * p.splits + split;
    float big = -INFINITY;
#pragma unroll
    for (int i = 0; i < kGroups; ++i) big = fmaxf(big, s_m[g][i]);
    for (int t = threadIdx.x; t < p.D; t += kDecodeThreads) {
      float a = 0.f;
#pragma unroll
      for (int i = 0; i < kGroups; ++i) {
        const float w = (s_m[g][i] == -INFINITY) ? 0.f : ex2(s_m[g][i] - big);
        a = fmaf(s_acc[g][i][t], w, a);
      }
      p.part_acc[slot * p.D + t] = a;
    }
    if (threadIdx.x == 0) {
      float lsum = 0.f;
#pragma unroll
      for (int i = 0; i < kGroups; ++i) lsum += (s_m[g][i] == -INFINITY) ? 0.f : s_l[g][i] * ex2(s_m[g][i] - big);
      p.part_ml[slot * 2] = big;
      p.part_ml[slot * 2 + 1] = lsum;
    }
  }
}

template <bool BF16>
__global__ void decode_merge_kernel(const DecodeParams p) {
  const int unit = blockIdx.x;
  const float* ml = p.part_ml + static_cast<int64_t>(unit) * p.splits * 2;
  float big = -INFINITY;
  for (int s = 0; s < p.splits; ++s) big = fmaxf(big, ml[2 * s]);
  float lsum = 0.f;
  for (int s = 0; s < p.splits; ++s) lsum += (ml[2 * s] == -INFINITY) ? 0.f : ml[2 * s + 1] * ex2(ml[2 * s] - big);
  const float inv = lsum > 0.f ? 1.0f / lsum : 0.f;
  for (int t = threadIdx.x; t < p.D; t += blockDim.x) {
    float a = 0.f;
    for (int s = 0; s < p.splits; ++s) {
      const float w = (ml[2 * s] == -INFINITY) ? 0.f : ex2(ml[2 * s] - big);
      a = fmaf(p.part_acc[(static_cast<int64_t>(unit) * p.splits + s) * p.D + t], w, a);
    }
    a *= inv;
    if constexpr (BF16) reinterpret_cast<__nv_bfloat16*>(p.y)[static_cast<int64_t>(unit) * p.D + t] = __float2bfloat16(a);
    else reinterpret_cast<__half*>(p.y)[static_cast<int64_t>(unit) * p.D + t] = __float2half(a);
  }
}

cudaError_t launch_merge(const DecodeParams& p, bool bf16, cudaStream_t stream) {
  const int threads = p.D <= 64 ? 64 : (p.D <= 128 ? 128 : 256);
  if (bf16) decode_merge_kernel<true><<<p.B * p.N, threads, 0, stream>>>(p);
  else decode_merge_kernel<false><<<p.B * p.N, threads, 0, stream>>>(p);
  return cudaGetLastError();
}

template <int LPR, int G>
cudaError_t launch_decode_g(const DecodeParams& p, bool bf16, cudaStream_t stream) {
  dim3 grid(p.splits, p.B * (p.N / G));
  if (bf16) decode_split_kernel<LPR, true, G><<<grid, kDecodeThreads, 0, stream>>>(p);
  else decode_split_kernel<LPR, false, G><<<grid, kDecodeThreads, 0, stream>>>(p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  return launch_merge(p, bf16, stream);
}

template <int LPR>
cudaError_t launch_decode_lpr(const DecodeParams& p, bool bf16, cudaStream_t stream) {
  switch (p.kv_group) {
    case 1: return launch_decode_g<LPR, 1>(p, bf16, stream);
    case 2: return launch_decode_g<LPR, 2>(p, bf16, stream);
    case 4: return launch_decode_g<LPR, 4>(p, bf16, stream);
    case 8: return launch_decode_g<LPR, 8>(p, bf16, stream);
    default: return cudaErrorInvalidValue;   // the entry point admits 1, 2, 4, 8 only
  }
}

}  // namespace

cudaError_t launch_decode(const DecodeParams& p, bool bf16, cudaStream_t stream) {
  // several query heads per cache head, head_dim <= 128: the group goes on the rows of a tensor-core MMA
  if (p.kv_group >= kDecodeGqaMinGroup && p.D <= 128) {
    cudaError_t e = launch_decode_gqa_split(p, bf16, stream);
    if (e != cudaSuccess) return e;
    return launch_merge(p, bf16, stream);
  }
  if (p.D <= 64) return launch_decode_lpr<8>(p, bf16, stream);
  if (p.D <= 128) return launch_decode_lpr<16>(p, bf16, stream);
  return launch_decode_lpr<32>(p, bf16, stream);
}

}  // namespace acct
