// Decode over a KV cache whose heads are shared by a GROUP of query heads (grouped-query / multi-query
// attention): split-KV streaming with the group on the M dimension of a warp-level tensor-core MMA.
//
// With one query head per cache head the step is pure streaming and runs on CUDA cores (decode.cu).  With G query
// heads per cache head every cache row is used G times: G x 256 multiply-adds per 512 bytes at head_dim 128, which
// CUDA cores cannot keep up with once G reaches 4 (the per-thread state of G heads also leaves too few warps
// resident to cover the memory latency).  Here the G heads are the rows of the A operand of
// mma.sync.m16n8k16 (rows G..15 are zero), so one warp does
//   S[16 x 16 keys] = Q[16 x D] K_tile^T              D/16 x 2 MMAs, fp32 accumulate
//   P = exp2(S * scale*log2e - m)   (online softmax per head, in the accumulator fragment layout)
//   O[16 x D]     += P[16 x 16] V_tile                 D/8 MMAs
// per tile of 16 cache rows, and the cache rows travel global -> shared memory by cp.async (16 bytes per lane,
// whole rows contiguous, no registers held while in flight) through a per-warp ring of kRing tiles, from where
// ldmatrix delivers the B fragments (K as stored, V transposed).  The step is then bound by HBM again.
//
// Output: the same per-split partial results (acc[D], max, sum per query head) as decode.cu writes, merged by its
// merge kernel.  Any group size from 2 to 16 and head_dim <= 128 take this path.
//
// Semantics as in decode.cu: y[b,n,0,:] = softmax(scale * q K[:len_b]^T) V[:len_b], the q_len = 1 case of the
// reference's inference op (infer/flash_attention/tik/tbe/impl/flash_attention_fwd.py:583-705).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "fa_kernels.cuh"

namespace acct {
namespace {

constexpr int kGqaThreads = 128;
constexpr int kGqaWarps = 4;
constexpr int kRing = 3;          // tiles in flight per warp
constexpr int kTileRows = 16;

__device__ __forceinline__ float ex2f(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

// 16 bytes global -> shared, bypassing L1; src_bytes = 0 writes zeros (the source is then not read)
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, uint32_t src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

// D (16x8, fp32) += A (16x16, row) * B (16x8, col); 16-bit operands
template <bool BF16>
__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  if constexpr (BF16)
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  else
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <bool BF16>
__device__ __forceinline__ uint32_t pack16(float a, float b) {
  if constexpr (BF16) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  } else {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
}

// DPAD: head_dim rounded up to 64 or 128 (cache rows are zero-filled past head_dim in shared memory).
// UPPER: the group has more than 8 query heads, i.e. rows 8..15 of the MMAs carry heads too.
template <int DPAD, bool BF16, bool UPPER>
__global__ void __launch_bounds__(kGqaThreads) decode_gqa_kernel(const DecodeParams p) {
  constexpr int kRowBytes = DPAD * 2 + 16;               // 16 bytes of padding: ldmatrix rows fall on distinct banks
  constexpr int kTileBytes = kTileRows * kRowBytes;
  constexpr int kChunksPerRow = DPAD / 8;                // 16-byte chunks
  constexpr int kCopies = kTileRows * kChunksPerRow / 32;  // cp.async per lane per tile (K or V)
  constexpr int kKSteps = DPAD / 16, kNTiles = DPAD / 8;

  extern __shared__ __align__(128) uint8_t gsm[];
  const int G = p.kv_group;
  const int split = blockIdx.x;
  const int n_kv = p.N / G;
  const int unit_kv = blockIdx.y;
  const int b = unit_kv / n_kv, h_kv = unit_kv % n_kv;
  int len = p.S_max;
  if (p.seq_lens != nullptr) len = min(p.S_max, max(0, p.seq_lens[b]));
  const int per = (((len + p.splits - 1) / p.splits) + 63) & ~63;
  const int k0 = split * per;
  const int k1 = min(len, k0 + per);

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;                 // fragment coordinates: row group, column pair
  uint8_t* ring = gsm + warp * (kRing * 2 * kTileBytes);

  // ---- the query heads of the group as A fragments (unscaled 16-bit inputs; the scale is applied to S in fp32)
  uint32_t qa[kKSteps][UPPER ? 4 : 2];
  {
    const uint16_t* qrow = reinterpret_cast<const uint16_t*>(p.q) + (static_cast<int64_t>(b) * p.N + h_kv * G) * p.D;
#pragma unroll
    for (int ks = 0; ks < kKSteps; ++ks) {
#pragma unroll
      for (int hi = 0; hi < (UPPER ? 2 : 1); ++hi) {
        const int head = g + 8 * hi;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const int d = ks * 16 + half * 8 + 2 * t;
          uint32_t w = 0;
          if (head < G && d < p.D) w = *reinterpret_cast<const uint32_t*>(qrow + static_cast<int64_t>(head) * p.D + d);
          qa[ks][UPPER ? (half * 2 + hi) : half] = w;    // a0, a1 (rows +8), a2, a3 (rows +8)
        }
      }
    }
  }

  const bool paged = p.block_table != nullptr;
  const int* table = paged ? p.block_table + static_cast<int64_t>(b) * p.max_pages : nullptr;
  const int64_t head_off = h_kv * p.kv_stride_h;
  const uint16_t* kbase = reinterpret_cast<const uint16_t*>(p.k) + (paged ? 0 : b * p.kv_stride_b) + head_off;
  const uint16_t* vbase = reinterpret_cast<const uint16_t*>(p.v) + (paged ? 0 : b * p.kv_stride_b) + head_off;
  auto row_offset = [&](int row) -> int64_t {
    if (!paged) return static_cast<int64_t>(row) * p.kv_stride_s;
    const int page = table[row >> p.page_shift];
    return static_cast<int64_t>(page) * p.kv_stride_b + static_cast<int64_t>(row & ((1 << p.page_shift) - 1)) * p.kv_stride_s;
  };

  // tiles of 16 rows, dealt to the warps in turn
  const int n_tiles = k1 > k0 ? (k1 - k0 + kTileRows - 1) / kTileRows : 0;
  const int my_tiles = n_tiles > warp ? (n_tiles - warp + kGqaWarps - 1) / kGqaWarps : 0;
  // A copy instruction moves 32 consecutive 16-byte chunks: kRowsPerCopy whole rows.  This lane always copies chunk
  // `lcol` of row `lrow` (+ kRowsPerCopy per instruction), so everything but the tile's first row is constant.
  constexpr int kRowsPerCopy = 32 / kChunksPerRow;
  const int lrow = lane / kChunksPerRow, lcol = lane % kChunksPerRow;
  const bool col_ok = lcol * 8 < p.D;
  const uint32_t dst_lane = lrow * kRowBytes + lcol * 16;
  const int64_t copy_step = static_cast<int64_t>(kRowsPerCopy) * p.kv_stride_s;
  auto issue_tile = [&](int it) {     // `it`-th tile of this warp into ring slot it % kRing
    const int row0 = k0 + (warp + it * kGqaWarps) * kTileRows;
    const uint32_t dstK = smem_addr(ring + (it % kRing) * 2 * kTileBytes) + dst_lane;
    const uint32_t dstV = dstK + kTileBytes;
    if (!paged && row0 + kTileRows <= k1) {
      // whole tile inside the split, contiguous cache: one address, stepped by a constant
      int64_t off = static_cast<int64_t>(row0 + lrow) * p.kv_stride_s + lcol * 8;
      const uint32_t nbytes = col_ok ? 16u : 0u;
      if (!col_ok) off = 0;
#pragma unroll
      for (int c = 0; c < kCopies; ++c) {
        cp_async16(dstK + c * kRowsPerCopy * kRowBytes, kbase + off, nbytes);
        cp_async16(dstV + c * kRowsPerCopy * kRowBytes, vbase + off, nbytes);
        if (col_ok) off += copy_step;
      }
    } else {
#pragma unroll
      for (int c = 0; c < kCopies; ++c) {
        const int row = row0 + c * kRowsPerCopy + lrow;
        const bool ok = row < k1 && col_ok;
        const int64_t off = ok ? row_offset(row) + lcol * 8 : 0;
        cp_async16(dstK + c * kRowsPerCopy * kRowBytes, kbase + off, ok ? 16u : 0u);
        cp_async16(dstV + c * kRowsPerCopy * kRowBytes, vbase + off, ok ? 16u : 0u);
      }
    }
  };

  float o[kNTiles][UPPER ? 4 : 2];
#pragma unroll
  for (int nt = 0; nt < kNTiles; ++nt)
#pragma unroll
    for (int e = 0; e < (UPPER ? 4 : 2); ++e) o[nt][e] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};   // rows g and g + 8; l is this thread's share

#pragma unroll
  for (int it = 0; it < kRing - 1; ++it) {
    if (it < my_tiles) issue_tile(it);
    cp_async_commit();
  }
  // ldmatrix row addresses of this lane inside a tile: matrix = lane / 8, row = lane % 8
  const int mi = lane >> 3, mr = lane & 7;
  const uint32_t k_lane = ((mi >> 1) * 8 + mr) * kRowBytes + (mi & 1) * 16;     // K: (keys 0-7 | 8-15) x (chunk 2ks | 2ks+1)
  const uint32_t v_lane = ((mi & 1) * 8 + mr) * kRowBytes + (mi >> 1) * 16;     // V: (keys 0-7 | 8-15) x (chunk nt | nt+1)

  for (int it = 0; it < my_tiles; ++it) {
    if (it + kRing - 1 < my_tiles) issue_tile(it + kRing - 1);
    cp_async_commit();
    cp_async_wait<kRing - 1>();
    __syncwarp();
    const uint32_t sK = smem_addr(ring + (it % kRing) * 2 * kTileBytes);
    const uint32_t sV = sK + kTileBytes;
    const int row0 = k0 + (warp + it * kGqaWarps) * kTileRows;

    // ---- S = Q K^T for keys row0 .. row0+15: two 8-key halves
    float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int ks = 0; ks < kKSteps; ++ks) {
      uint32_t kb[4];
      ldsm_x4(sK + k_lane + ks * 32, kb);
      if constexpr (UPPER) {
        mma16816<BF16>(s0, qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], kb[0], kb[1]);
        mma16816<BF16>(s1, qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], kb[2], kb[3]);
      } else {
        mma16816<BF16>(s0, qa[ks][0], 0u, qa[ks][1], 0u, kb[0], kb[1]);
        mma16816<BF16>(s1, qa[ks][0], 0u, qa[ks][1], 0u, kb[2], kb[3]);
      }
    }
    // ---- online softmax; this thread holds, per row, keys 2t, 2t+1 of each half
    const int kcol = row0 + 2 * t;
    const bool v00 = kcol < k1, v01 = kcol + 1 < k1, v10 = kcol + 8 < k1, v11 = kcol + 9 < k1;
    uint32_t pa[4] = {0u, 0u, 0u, 0u};
#pragma unroll
    for (int hi = 0; hi < (UPPER ? 2 : 1); ++hi) {
      const float x0 = v00 ? s0[2 * hi] * p.scale_log2 : -INFINITY, x1 = v01 ? s0[2 * hi + 1] * p.scale_log2 : -INFINITY;
      const float x2 = v10 ? s1[2 * hi] * p.scale_log2 : -INFINITY, x3 = v11 ? s1[2 * hi + 1] * p.scale_log2 : -INFINITY;
      float mx = fmaxf(fmaxf(x0, x1), fmaxf(x2, x3));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float m_new = fmaxf(m_run[hi], mx);           // row0 < k1, so key 0 of the tile exists: m_new is finite
      const float alpha = ex2f(m_run[hi] - m_new);        // 0 on the first tile (m_run = -inf)
      const float p0 = ex2f(x0 - m_new), p1 = ex2f(x1 - m_new), p2 = ex2f(x2 - m_new), p3 = ex2f(x3 - m_new);
      l_run[hi] = fmaf(l_run[hi], alpha, (p0 + p1) + (p2 + p3));
      m_run[hi] = m_new;
      pa[hi] = pack16<BF16>(p0, p1);                       // a0 / a1: keys 0-7
      pa[2 + hi] = pack16<BF16>(p2, p3);                   // a2 / a3: keys 8-15
      if (__any_sync(0xffffffffu, alpha != 1.0f)) {
#pragma unroll
        for (int nt = 0; nt < kNTiles; ++nt) {
          o[nt][2 * hi] *= alpha;
          o[nt][2 * hi + 1] *= alpha;
        }
      }
    }
    // ---- O += P V
#pragma unroll
    for (int nt = 0; nt < kNTiles; nt += 2) {
      uint32_t vb[4];
      ldsm_x4_trans(sV + v_lane + nt * 16, vb);
      if constexpr (UPPER) {
        mma16816<BF16>(o[nt], pa[0], pa[1], pa[2], pa[3], vb[0], vb[1]);
        mma16816<BF16>(o[nt + 1], pa[0], pa[1], pa[2], pa[3], vb[2], vb[3]);
      } else {
        float c0[4] = {o[nt][0], o[nt][1], 0.f, 0.f}, c1[4] = {o[nt + 1][0], o[nt + 1][1], 0.f, 0.f};
        mma16816<BF16>(c0, pa[0], 0u, pa[2], 0u, vb[0], vb[1]);
        mma16816<BF16>(c1, pa[0], 0u, pa[2], 0u, vb[2], vb[3]);
        o[nt][0] = c0[0]; o[nt][1] = c0[1];
        o[nt + 1][0] = c1[0]; o[nt + 1][1] = c1[1];
      }
    }
    __syncwarp();     // every lane has read this slot before a later copy may land in it
  }
  cp_async_wait<0>();

  // ---- merge the four warps of the CTA per query head, then write the split's partial result
  // (the ring is dead by now: its memory holds the warps' accumulators)
#pragma unroll
  for (int hi = 0; hi < 2; ++hi) {
    l_run[hi] += __shfl_xor_sync(0xffffffffu, l_run[hi], 1);
    l_run[hi] += __shfl_xor_sync(0xffffffffu, l_run[hi], 2);
  }
  __syncthreads();
  float* s_acc = reinterpret_cast<float*>(gsm);                      // [warp][16 heads][DPAD]
  float* s_m = s_acc + kGqaWarps * 16 * DPAD;                        // [warp][16]
  float* s_l = s_m + kGqaWarps * 16;
#pragma unroll
  for (int hi = 0; hi < (UPPER ? 2 : 1); ++hi) {
    const int head = g + 8 * hi;
    if (t == 0) { s_m[warp * 16 + head] = m_run[hi]; s_l[warp * 16 + head] = l_run[hi]; }
#pragma unroll
    for (int nt = 0; nt < kNTiles; ++nt)
      *reinterpret_cast<float2*>(s_acc + (warp * 16 + head) * DPAD + nt * 8 + 2 * t) = make_float2(o[nt][2 * hi], o[nt][2 * hi + 1]);
  }
  __syncthreads();
  for (int head = 0; head < G; ++head) {
    const int64_t unit = static_cast<int64_t>(b) * p.N + h_kv * G + head;
    const int64_t slot = unit * p.splits + split;
    float big = -INFINITY;
#pragma unroll
    for (int w = 0; w < kGqaWarps; ++w) big = fmaxf(big, s_m[w * 16 + head]);
    for (int d = threadIdx.x; d < p.D; d += kGqaThreads) {
      float a = 0.f;
#pragma unroll
      for (int w = 0; w < kGqaWarps; ++w) {
        const float mw = s_m[w * 16 + head];
        a = fmaf(s_acc[(w * 16 + head) * DPAD + d], mw == -INFINITY ? 0.f : ex2f(mw - big), a);
      }
      p.part_acc[slot * p.D + d] = a;
    }
    if (threadIdx.x == 0) {
      float lsum = 0.f;
#pragma unroll
      for (int w = 0; w < kGqaWarps; ++w) {
        const float mw = s_m[w * 16 + head];
        lsum += mw == -INFINITY ? 0.f : s_l[w * 16 + head] * ex2f(mw - big);
      }
      p.part_ml[slot * 2] = big;
      p.part_ml[slot * 2 + 1] = lsum;
    }
  }
}

template <int DPAD>
cudaError_t launch_gqa(const DecodeParams& p, bool bf16, cudaStream_t stream) {
  const size_t ring = static_cast<size_t>(kGqaWarps) * kRing * 2 * kTileRows * (DPAD * 2 + 16);
  const size_t merge = static_cast<size_t>(kGqaWarps) * 16 * (DPAD + 2) * sizeof(float);
  const size_t smem = ring > merge ? ring : merge;
  const bool upper = p.kv_group > 8;
  void (*kern)(const DecodeParams) =
      bf16 ? (upper ? decode_gqa_kernel<DPAD, true, true> : decode_gqa_kernel<DPAD, true, false>)
           : (upper ? decode_gqa_kernel<DPAD, false, true> : decode_gqa_kernel<DPAD, false, false>);
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  if (e != cudaSuccess) return e;
  dim3 grid(p.splits, p.B * (p.N / p.kv_group));
  kern<<<grid, kGqaThreads, smem, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace

// The split kernel for a group of 2..16 query heads per cache head, head_dim <= 128 (the caller then runs the merge
// kernel of decode.cu over the partial results).
cudaError_t launch_decode_gqa_split(const DecodeParams& p, bool bf16, cudaStream_t stream) {
  if (p.D <= 64) return launch_gqa<64>(p, bf16, stream);
  return launch_gqa<128>(p, bf16, stream);
}

}  // namespace acct
