// FlashAttention-2 backward for head_dim in (128, 256] on sm_100a.
//
// At these widths the dK and dV accumulators of one 128-row K/V tile would fill tensor memory on their own
// (2 x 256 columns), and full-width K, V, Q and dO tiles would not fit shared memory.  So the work of one K/V tile is
// split over TWO CTAs by halves of head_dim: CTA (j, hd) accumulates dK[:, 128*hd .. 128*hd+127] and the same
// columns of dV and of every dQ tile it touches, and the Q tiles are walked 64 query rows at a time:
//   S^T  = K_j Q_m^T           contraction over the whole head_dim (16 steps), M = 128 keys, N = 64 queries
//   dP^T = V_j dO_m^T
//   P^T  = exp2(S^T*scale*log2e + bias - L*log2e);  dS^T = P^T * (dP^T * M - D)            (registers)
//   dV[:, half] += (P^T*M) dO_m[:, half]     A = P^T from tensor memory (over S^T), B = dO half, MN-major
//   dK[:, half] += dS^T Q_m[:, half]         A = dS^T from tensor memory (over dP^T), B = Q half, MN-major
//   dQ_m^T[half] = K_j[:, half]^T dS^T       M = 128 head_dim columns, N = 64 queries; A = K half read MN-major,
//                                            B = dS^T from shared memory, MN-major; columns of its own
// Both CTAs of a tile recompute S^T and dP^T (contractions over the whole width): 56 MMA steps per half instead of
// 40 for an unsplit product, the price of fitting.  Tensor memory: S^T 64 | dP^T 64 | dQ^T 64 | (64 unused) |
// dK half 128 | dV half 128.  Shared memory: K and V whole (2 x 64 KB), one Q and one dO sub-tile of 64 rows
// (2 x 32 KB, single-buffered), dS^T (16 KB), dQ staging (16 KB).  The single Q / dO buffers make this kernel
// latency-bound: it exists so that every head_dim the reference cell accepts (up to 256,
// train/acctransformer/flash_attention/nn/layer/flash_attention.py:26,105-106) trains; the head_dim <= 128 kernel
// is the optimised one.  Mask, alibi, dropout (both forms), band, row groups and valid lengths are all handled on
// one general path, element by element.
//
// Warp roles as in the narrow kernel: warps 0-7 compute (thread = one key row x 32 of the 64 queries), warps 8-11
// drain dQ^T (thread = one head_dim column of the half), warp 12 TMA producer, warp 13 MMA issuer.
//
// Follows the reference's backward (train/acctransformer/flash_attention/ops/flash_attention/
// flash_attention_bwd.py:259-415) like the narrow kernel does.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "fa_bwd_helpers.cuh"
#include "fa_common.cuh"
#include "fa_kernels.cuh"
#include "ptx.cuh"

namespace acct {

namespace {

constexpr int kWThreads = 512;
constexpr int kWComputeThreads = 256;
constexpr int kWDrainWarp0 = 8, kWProducerWarp = 12, kWMmaWarp = 13;
constexpr int kSub = 64;                          // query rows per step
constexpr int kWRegsCompute = 152, kWRegsDrain = 152, kWRegsControl = 56;
constexpr uint32_t kKvTileBytes = 4 * 16384u;     // 128 rows x 256 columns, four 64-column blocks
constexpr uint32_t kSubTileBytes = 4 * 8192u;     // 64 rows x 256 columns

struct WideShared {
  uint64_t kv_full;
  uint64_t q_full, q_empty;        // q_empty: the S^T and dK products reading the Q sub-tile have finished
  uint64_t do_full, do_empty;      // do_empty: the dP^T and dV products reading the dO sub-tile have finished
  uint64_t st_full, dp_full;       // MMA -> compute
  uint64_t p_ready, ds_ready;      // compute -> MMA
  uint64_t dq_full, dq_read;       // MMA -> drain -> MMA
  uint64_t stats_ready;
  uint32_t tmem_base;
  volatile uint32_t abort_flag;
  alignas(16) float lse2[2][kSub];
  alignas(16) float delta[2][kSub];
};

}  // namespace

template <bool BF16>
__global__ void __launch_bounds__(kWThreads, 1) fa_bwd_wide_kernel(const __grid_constant__ BwdParams p) {
  constexpr uint32_t kColST = 0, kColDP = 64, kColDQ = 128, kColDK = 256, kColDV = 384;

  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* sK = smem;
  uint8_t* sV = sK + kKvTileBytes;
  uint8_t* sQ = sV + kKvTileBytes;
  uint8_t* sDO = sQ + kSubTileBytes;
  uint8_t* sDS = sDO + kSubTileBytes;              // dS^T: 128 key rows x 64 queries (one 128-byte-row block)
  uint8_t* sStage = sDS + 16384;                   // dQ^T staging: 2 chunks of 64 query rows x 32 fp32
  WideShared& sh = *reinterpret_cast<WideShared*>(sStage + 16384);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int n_kv = p.N / p.kv_group;
  const int bh_kv = blockIdx.y;
  const int b = bh_kv / n_kv, h_kv = bh_kv % n_kv;
  const int hd = blockIdx.x & 1;                   // which half of head_dim
  // K/V tile; descending when the dQ reduction is ordered (a CTA then only ever waits for CTAs started before it)
  const int jj = blockIdx.x >> 1;
  const int j = p.dq_order != nullptr ? static_cast<int>(gridDim.x >> 1) - 1 - jj : jj;
  const ScoreMods& mods = p.mods;

  if ((smem_u32(smem) & 1023u) != 0u) {
    if (tid == 0) atomicMax(p.status, DEV_BAD_SMEM_BASE);
    return;
  }

  int kv_len = p.S_k;
  if (mods.seq_lens != nullptr) kv_len = min(p.S_k, max(0, mods.seq_lens[b]));

  // 128-row Q tiles i that need K/V tile j (same predicate as the narrow kernel), each walked as two 64-row steps
  const int tiles_q = (p.S_q + kTile - 1) / kTile;
  int i_lo = 0, i_hi = tiles_q - 1;
  if (mods.next_block_num < 65536) i_lo = max(i_lo, j - mods.next_block_num);
  if (mods.prev_block_num < 65536) i_hi = min(i_hi, j + mods.prev_block_num);
  if (mods.causal) i_lo = max(i_lo, j);
  if (mods.tri_block > 0) i_lo = max(i_lo, (((j * kTile) / mods.tri_block) * mods.tri_block) / kTile);
  if (j * kTile >= kv_len) i_hi = i_lo - 1;
  const int n_per = max(0, i_hi - i_lo + 1);
  const int per_head = 2 * n_per;                  // steps per query head
  const int n_steps = per_head * p.kv_group;
  auto head_of = [&](int m) { return h_kv * p.kv_group + m / max(per_head, 1); };
  auto tile_of = [&](int m) { return i_lo + (m % max(per_head, 1)) / 2; };
  auto qbase_of = [&](int m) { return tile_of(m) * kTile + (m & 1) * kSub; };

  if (tid == 0) {
    mbar_init(&sh.kv_full, 1);
    mbar_init(&sh.q_full, 1); mbar_init(&sh.q_empty, 1);
    mbar_init(&sh.do_full, 1); mbar_init(&sh.do_empty, 1);
    mbar_init(&sh.st_full, 1); mbar_init(&sh.dp_full, 1);
    mbar_init(&sh.p_ready, kWComputeThreads); mbar_init(&sh.ds_ready, kWComputeThreads);
    mbar_init(&sh.dq_full, 1); mbar_init(&sh.dq_read, 128);
    mbar_init(&sh.stats_ready, kSub);
    sh.abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == kWProducerWarp) { tmem_alloc(&sh.tmem_base, 512); tmem_relinquish(); }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = sh.tmem_base;
  volatile uint32_t* abort_flag = &sh.abort_flag;

  if (warp >= kWProducerWarp) {
    reg_dealloc<kWRegsControl>();
    if (warp == kWProducerWarp) {
      // ---------------------------------------------------------------- TMA producer
      if (lane == 0 && n_steps > 0) {
        prefetch_tmap(&p.map_q); prefetch_tmap(&p.map_k); prefetch_tmap(&p.map_v); prefetch_tmap(&p.map_do);
        prefetch_tmap(&p.map_dq);
        mbar_expect_tx(&sh.kv_full, 2 * kKvTileBytes);
        for (int nb = 0; nb < 4; ++nb) tma_load_4d(sK + nb * 16384, &p.map_k, &sh.kv_full, nb * 64, j * kTile, h_kv, b);
        for (int nb = 0; nb < 4; ++nb) tma_load_4d(sV + nb * 16384, &p.map_v, &sh.kv_full, nb * 64, j * kTile, h_kv, b);
        for (int m = 0; m < n_steps; ++m) {
          const int q0 = qbase_of(m), h = head_of(m);
          if (m >= 1) mbar_wait(&sh.q_empty, (m - 1) & 1, abort_flag, p.status, DEV_TIMEOUT_SYNC);
          mbar_expect_tx(&sh.q_full, kSubTileBytes);
          for (int nb = 0; nb < 4; ++nb) tma_load_4d(sQ + nb * 8192, &p.map_q, &sh.q_full, nb * 64, q0, h, b);
          if (m >= 1) mbar_wait(&sh.do_empty, (m - 1) & 1, abort_flag, p.status, DEV_TIMEOUT_SYNC);
          mbar_expect_tx(&sh.do_full, kSubTileBytes);
          for (int nb = 0; nb < 4; ++nb) tma_load_4d(sDO + nb * 8192, &p.map_do, &sh.do_full, nb * 64, q0, h, b);
        }
      }
    } else if (warp == kWMmaWarp) {
      // ---------------------------------------------------------------- MMA issuer
      if (lane == 0 && n_steps > 0) {
        const uint32_t idesc_s = make_idesc(BF16, 128, kSub, false, false);    // S^T, dP^T
        const uint32_t idesc_kv = make_idesc(BF16, 128, 128, false, true);     // dV, dK halves
        const uint32_t idesc_dq = make_idesc(BF16, 128, kSub, true, true);     // dQ^T half
        const uint64_t kmajor = make_sdesc_base(16, 1024);
        const uint64_t mn_kv = make_sdesc_base(16384, 1024);    // 64-column blocks of a 128-row tile
        const uint64_t mn_sub = make_sdesc_base(8192, 1024);    // 64-column blocks of a 64-row sub-tile
        const uint32_t k_hi = static_cast<uint32_t>(kmajor >> 32), k_lo = static_cast<uint32_t>(kmajor);
        const uint32_t mkv_hi = static_cast<uint32_t>(mn_kv >> 32), mkv_lo = static_cast<uint32_t>(mn_kv);
        const uint32_t msub_hi = static_cast<uint32_t>(mn_sub >> 32), msub_lo = static_cast<uint32_t>(mn_sub);
        auto lo_of = [](uint32_t base_lo, const uint8_t* ptr) { return base_lo | ((smem_u32(ptr) >> 4) & 0x3fffu); };
        const uint32_t kK = lo_of(k_lo, sK), kV = lo_of(k_lo, sV), kQ = lo_of(k_lo, sQ), kDO = lo_of(k_lo, sDO);
        const uint32_t mKh = lo_of(mkv_lo, sK + hd * 2 * 16384);     // this CTA's half of K, as the A operand of dQ^T
        const uint32_t mQh = lo_of(msub_lo, sQ + hd * 2 * 8192);     // its half of Q / dO, as B operands
        const uint32_t mDOh = lo_of(msub_lo, sDO + hd * 2 * 8192);
        const uint32_t mDS = lo_of(msub_lo, sDS);

        mbar_wait(&sh.kv_full, 0, abort_flag, p.status, DEV_TIMEOUT_TMA);
        for (int m = 0; m < n_steps; ++m) {
          const uint32_t par = m & 1;
          mbar_wait(&sh.q_full, par, abort_flag, p.status, DEV_TIMEOUT_TMA);
          tc_fence_after_sync();
#pragma unroll
          for (int kk = 0; kk < 16; ++kk)   // S^T = K Q^T over the whole width
            umma_ss_lohi(tmem + kColST, kK + (kk >> 2) * 1024u + (kk & 3) * 2u, k_hi, kQ + (kk >> 2) * 512u + (kk & 3) * 2u,
                         k_hi, idesc_s, kk > 0);
          umma_commit(&sh.st_full);
          mbar_wait(&sh.do_full, par, abort_flag, p.status, DEV_TIMEOUT_TMA);
          tc_fence_after_sync();
#pragma unroll
          for (int kk = 0; kk < 16; ++kk)   // dP^T = V dO^T
            umma_ss_lohi(tmem + kColDP, kV + (kk >> 2) * 1024u + (kk & 3) * 2u, k_hi, kDO + (kk >> 2) * 512u + (kk & 3) * 2u,
                         k_hi, idesc_s, kk > 0);
          umma_commit(&sh.dp_full);
          // dV half += P^T dO half: P^T of queries [32h, 32h+32) sits in S^T columns [32h, 32h+16)
          mbar_wait(&sh.p_ready, par, abort_flag, p.status, DEV_TIMEOUT_SYNC);
          tc_fence_after_sync();
#pragma unroll
          for (int kk = 0; kk < kSub / 16; ++kk)
            umma_ts_lohi(tmem + kColDV, tmem + kColST + (kk >> 1) * 32 + (kk & 1) * 8, mDOh + kk * 128u, msub_hi, idesc_kv,
                         m > 0 || kk > 0);
          umma_commit(&sh.do_empty);
          // dK half += dS^T Q half
          mbar_wait(&sh.ds_ready, par, abort_flag, p.status, DEV_TIMEOUT_SYNC);
          tc_fence_after_sync();
#pragma unroll
          for (int kk = 0; kk < kSub / 16; ++kk)
            umma_ts_lohi(tmem + kColDK, tmem + kColDP + (kk >> 1) * 32 + (kk & 1) * 8, mQh + kk * 128u, msub_hi, idesc_kv,
                         m > 0 || kk > 0);
          umma_commit(&sh.q_empty);
          // dQ^T half = K half^T dS^T, once the drain has pulled the previous one out of its columns
          if (m > 0) mbar_wait(&sh.dq_read, (m - 1) & 1, abort_flag, p.status, DEV_TIMEOUT_SYNC);
          tc_fence_after_sync();
#pragma unroll
          for (int kk = 0; kk < kTile / 16; ++kk)
            umma_ss_lohi(tmem + kColDQ, mKh + kk * 128u, mkv_hi, mDS + kk * 128u, msub_hi, idesc_dq, kk > 0);
          umma_commit(&sh.dq_full);
        }
      }
    }
  } else if (warp >= kWDrainWarp0) {
    // ------------------------------------------------------------------ drain: dQ^T (lane = head_dim column of the
    // half, 64 query columns) through a swizzled staging area into the fp32 accumulator by TMA reduce-add.
    // Warp w owns the 32-column chunk w of the half; the staging area holds two chunks: warps 0,1 first, then 2,3.
    reg_alloc<kWRegsDrain>();
    const int r = tid - kWDrainWarp0 * 32;
    const int w = warp & 3;
    const uint32_t t_dq = tmem + (static_cast<uint32_t>(w * 32) << 16) + kColDQ;
    const bool elected = (r == 0);
    for (int m = 0; m < n_steps; ++m) {
      const int q0 = qbase_of(m);
      const int h = head_of(m);
      const int bh = b * p.N + h;
      mbar_wait(&sh.dq_full, m & 1, abort_flag, p.status, DEV_TIMEOUT_MMA);
      tc_fence_after_sync();
      uint32_t dq[2][32];
      tmem_ld32(t_dq, dq[0]);
      tmem_ld32(t_dq + 32, dq[1]);
      tmem_wait_ld();
      tc_fence_before_sync();
      mbar_arrive(&sh.dq_read);
#pragma unroll 1
      for (int rd = 0; rd < 2; ++rd) {
        if (elected) tma_store_wait_read();
        named_barrier(3, 128);
        if ((w >> 1) == rd) {
          uint8_t* dst = sStage + (w & 1) * 8192u + (lane & 3) * 4;
          const uint32_t ch = lane >> 2;
#pragma unroll
          for (int c = 0; c < 2; ++c)
#pragma unroll
            for (int e = 0; e < 32; ++e) {
              const int qrow = c * 32 + e;     // (qrow & 7) == (e & 7)
              *reinterpret_cast<float*>(dst + qrow * 128 + ((ch ^ (e & 7)) << 4)) = __uint_as_float(dq[c][e]) * p.scale;
            }
        }
        fence_proxy_async_smem();
        named_barrier(3, 128);
        if (elected) {
          const int i = tile_of(m);
          unsigned int* slot = p.dq_order != nullptr
                                   ? p.dq_order + (static_cast<int64_t>(bh) * tiles_q + i) * 2 + hd : nullptr;
          if (slot != nullptr && rd == 0 && (m & 1) == 0) {
            // ordered dQ: the K/V tiles that touch Q tile i add their parts in descending tile order
            int j_top = (kv_len + kTile - 1) / kTile - 1;
            if (mods.next_block_num < 65536) j_top = min(j_top, i + mods.next_block_num);
            if (mods.causal) j_top = min(j_top, i);
            if (mods.tri_block > 0) j_top = min(j_top, (((i * kTile + kTile - 1) / mods.tri_block + 1) * mods.tri_block - 1) / kTile);
            const unsigned int my_turn = static_cast<unsigned int>(j_top - j);
            const long long t0 = clock64();
            unsigned int seen;
            while (true) {
              asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(slot) : "memory");
              if (seen >= my_turn || *abort_flag != 0u) break;
              if (clock64() - t0 > kWaitCycleLimit) { *abort_flag = 1u; atomicMax(p.status, DEV_TIMEOUT_SYNC); break; }
            }
          }
#pragma unroll
          for (int cc = 0; cc < 2; ++cc) {
            const int col = hd * 128 + (rd * 2 + cc) * 32;
            if (col < p.D && q0 < p.S_q) tma_reduce_add_4d(&p.map_dq, sStage + cc * 8192u, col, q0, h, b);
          }
          tma_store_commit();
          if (slot != nullptr && rd == 1 && (m & 1) == 1) {
            tma_store_wait_all();
            asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(slot) : "memory");
          }
        }
      }
    }
    if (elected) tma_store_wait_all();
  } else {
    // ------------------------------------------------------------------ compute warps
    reg_alloc<kWRegsCompute>();
    const int hf = warp >> 2;                            // which 32 of the step's 64 queries
    const int r = (warp & 3) * 32 + lane;                // key row inside the tile
    const int kv_idx = j * kTile + r;
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t t_st = tmem + lane_base + kColST + hf * 32;
    const uint32_t t_dp = tmem + lane_base + kColDP + hf * 32;
    const bool kv_ok = kv_idx < kv_len;
    const int kv_c = min(kv_idx, p.S_k - 1);
    auto bias_of = [&](int h) {
      float v = kNegInf;
      if (kv_ok) {
        v = 0.f;
        if (mods.alibi != nullptr) v = load16<BF16>(mods.alibi, (static_cast<int64_t>(b) * p.N + h) * p.S_k + kv_idx) * kLog2e;
        else if (mods.alibi_slopes != nullptr) v = mods.alibi_slopes[h] * static_cast<float>(kv_idx) * kLog2e;
      }
      return v;
    };
    float bias = kNegInf;
    const bool stats_thread = hf == 0 && r < kSub;      // warps 0 and 1: one thread per query of the step

    float nxt_lse = 0.f, nxt_dlt = 0.f;
    bool nxt_ok = false;
    if (stats_thread && n_steps > 0) {
      const int q_row = qbase_of(0) + r;
      const bool q_ok = q_row < p.S_q;
      const int64_t idx = (static_cast<int64_t>(b) * p.N + head_of(0)) * p.S_q + min(q_row, p.S_q - 1);
      sh.lse2[0][r] = q_ok ? p.lse[idx] * kLog2e : INFINITY;
      sh.delta[0][r] = q_ok ? p.delta[idx] : 0.f;
      mbar_arrive(&sh.stats_ready);
    }

    for (int m = 0; m < n_steps; ++m) {
      const int i = tile_of(m);
      const int q0 = qbase_of(m) + hf * 32;              // first of this thread's 32 queries
      const int bh = b * p.N + head_of(m);
      if (m % max(per_head, 1) == 0) bias = bias_of(head_of(m));
      // ---- P part
      mbar_wait(&sh.st_full, m & 1, abort_flag, p.status, DEV_TIMEOUT_MMA);
      tc_fence_after_sync();
      if (stats_thread && m > 0) {
        sh.lse2[m & 1][r] = nxt_ok ? nxt_lse * kLog2e : INFINITY;
        sh.delta[m & 1][r] = nxt_ok ? nxt_dlt : 0.f;
        mbar_arrive(&sh.stats_ready);
      }
      if (stats_thread && m + 1 < n_steps) {
        const int q_row = qbase_of(m + 1) + r;
        nxt_ok = q_row < p.S_q;
        const int64_t idx = (static_cast<int64_t>(b) * p.N + head_of(m + 1)) * p.S_q + min(q_row, p.S_q - 1);
        nxt_lse = p.lse[idx];
        nxt_dlt = p.delta[idx];
      }
      mbar_wait(&sh.stats_ready, m & 1, abort_flag, p.status, DEV_TIMEOUT_SYNC);
      const float* lse2 = sh.lse2[m & 1] + hf * 32;
      const float* dlt = sh.delta[m & 1] + hf * 32;
      const bool use_mask = (mods.mask_kind == 1) || (mods.mask_kind == 2 && i == j);
      const bool diag = mods.causal && (q0 < j * kTile + kTile - 1);

      uint32_t s[32];
      tmem_ld32(t_st, s);
      // dropout factor of each (key, query) pair of this thread: 0 or the rescale value
      uint32_t keep_bits = 0xffffffffu;
      if (mods.drop_philox != 0) keep_bits = philox_keep_column(mods, bh, q0, p.S_q - 1, kv_idx, lane);
      tmem_wait_ld();
      float pr[32];
      uint32_t pk[16];
#pragma unroll
      for (int e = 0; e < 32; ++e) {
        const int q = q0 + e;
        float x = fmaf(__uint_as_float(s[e]), p.scale_log2, bias) - lse2[e];
        if (use_mask) {
          const int qc = min(q, p.S_q - 1);
          const float mv = mods.mask_kind == 1
                               ? load_mask_value(mods.mask, mods.mask_dtype,
                                                 (static_cast<int64_t>(mods.mask_batch > 1 ? b : 0) * p.S_q + qc) * p.S_k + kv_c)
                               : load_mask_value(mods.mask, mods.mask_dtype, static_cast<int64_t>(q - i * kTile) * kTile + r);
          x = fmaf(mv, -10000.0f * kLog2e, x);
        }
        float v = ex2(x);
        if (diag && kv_idx > q) v = 0.f;
        if (mods.tri_block > 0 && kv_idx >= (q / mods.tri_block + 1) * mods.tri_block) v = 0.f;
        pr[e] = v;
      }
      float fac[32];     // dropout factors (1 without dropout)
      if (mods.drop != nullptr) {
#pragma unroll
        for (int e = 0; e < 32; ++e)
          fac[e] = load_mask_value(mods.drop, mods.drop_dtype,
                                   (static_cast<int64_t>(bh) * p.S_q + min(q0 + e, p.S_q - 1)) * p.S_k + kv_c) * mods.drop_scale;
      } else {
#pragma unroll
        for (int e = 0; e < 32; ++e) fac[e] = ((keep_bits >> e) & 1u) ? mods.drop_scale : 0.f;
      }
#pragma unroll
      for (int e = 0; e < 16; ++e) pk[e] = pack2<BF16>(pr[2 * e] * fac[2 * e], pr[2 * e + 1] * fac[2 * e + 1]);
      tmem_st16(t_st, pk);     // over the first 16 of this half's own 32 S^T columns
      tmem_wait_st();
      tc_fence_before_sync();
      mbar_arrive(&sh.p_ready);

      // ---- dS part
      mbar_wait(&sh.dp_full, m & 1, abort_flag, p.status, DEV_TIMEOUT_MMA);
      tc_fence_after_sync();
      uint32_t dp[32];
      tmem_ld32(t_dp, dp);
      tmem_wait_ld();
      uint32_t ds[16];
#pragma unroll
      for (int e = 0; e < 16; ++e) {
        const float d0 = pr[2 * e] * fmaf(__uint_as_float(dp[2 * e]), fac[2 * e], -dlt[2 * e]);
        const float d1 = pr[2 * e + 1] * fmaf(__uint_as_float(dp[2 * e + 1]), fac[2 * e + 1], -dlt[2 * e + 1]);
        ds[e] = pack2<BF16>(d0, d1);
      }
      tmem_st16(t_dp, ds);     // A operand of the dK product
#pragma unroll
      for (int g = 0; g < 4; ++g)   // and row r of the dS^T block in shared memory (B operand of dQ^T)
        *reinterpret_cast<uint4*>(sDS + swz128(r, hf * 4 + g)) = make_uint4(ds[4 * g], ds[4 * g + 1], ds[4 * g + 2], ds[4 * g + 3]);
      tmem_wait_st();
      fence_proxy_async_smem();
      tc_fence_before_sync();
      mbar_arrive(&sh.ds_ready);
    }

    // epilogue: this CTA's 128 columns of dK (scaled) and dV for key row r; each query-half group writes 64 of them
    if (n_steps > 0) mbar_wait(&sh.dq_full, (n_steps - 1) & 1, abort_flag, p.status, DEV_TIMEOUT_MMA);
    tc_fence_after_sync();
    const bool row_ok = kv_idx < p.S_k;
    const int64_t row_off = (static_cast<int64_t>(bh_kv) * p.S_k + kv_idx) * p.D;
#pragma unroll 1
    for (int which = 0; which < 2; ++which) {
      const uint32_t t_src = tmem + lane_base + (which == 0 ? kColDK : kColDV);
      const float mul = which == 0 ? p.scale : 1.0f;
      void* out = which == 0 ? p.dk : p.dv;
#pragma unroll 1
      for (int cq = 0; cq < 2; ++cq) {
        const int c = hf * 2 + cq;                     // 32-column chunk of the half
        uint32_t v[32];
        if (n_steps > 0) { tmem_ld32(t_src + c * 32, v); tmem_wait_ld(); }
        else {
#pragma unroll
          for (int e = 0; e < 32; ++e) v[e] = 0u;
        }
        if (!row_ok) continue;
        const int col0 = hd * 128 + c * 32;
        if (p.grads_f32) {
          float* dst = reinterpret_cast<float*>(out) + row_off;
#pragma unroll
          for (int g = 0; g < 8; ++g) {
            const int col = col0 + g * 4;
            if (col + 4 <= p.D)
              *reinterpret_cast<float4*>(dst + col) =
                  make_float4(__uint_as_float(v[4 * g]) * mul, __uint_as_float(v[4 * g + 1]) * mul,
                              __uint_as_float(v[4 * g + 2]) * mul, __uint_as_float(v[4 * g + 3]) * mul);
          }
        } else {
          uint8_t* dst = reinterpret_cast<uint8_t*>(out) + row_off * 2;
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            const int col = col0 + g * 8;
            if (col + 8 <= p.D) {
              uint32_t wv[4];
#pragma unroll
              for (int e = 0; e < 4; ++e)
                wv[e] = pack2<BF16>(__uint_as_float(v[8 * g + 2 * e]) * mul, __uint_as_float(v[8 * g + 2 * e + 1]) * mul);
              *reinterpret_cast<uint4*>(dst + col * 2) = make_uint4(wv[0], wv[1], wv[2], wv[3]);
            }
          }
        }
      }
    }
    tc_fence_before_sync();
  }

  linger_after_abort(abort_flag);
  __syncthreads();
  if (warp == kWProducerWarp) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, 512);
  }
}

cudaError_t launch_fa_bwd_wide(const BwdParams& p, bool bf16, cudaStream_t stream) {
  const size_t smem = 2 * kKvTileBytes + 2 * kSubTileBytes + 2 * 16384 + sizeof(WideShared);
  dim3 grid(2 * ((p.S_k + kTile - 1) / kTile), p.B * (p.N / p.kv_group));
  void (*kern)(const BwdParams) = bf16 ? fa_bwd_wide_kernel<true> : fa_bwd_wide_kernel<false>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  if (e != cudaSuccess) return e;
  kern<<<grid, kWThreads, smem, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace acct
