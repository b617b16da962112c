// FlashAttention-2 forward for sm_100a.
//
// One CTA owns two consecutive 128-row Q tiles of one (batch, head) slice and walks the K/V tiles
// they need.  Warp roles:
//   warps 0-3   softmax group for Q tile 0 (thread t owns score row t: row max / sum are in-thread)
//   warps 4-7   softmax group for Q tile 1
//   warp  8     TMA producer: Q once, then K_j / V_j into a two-stage ring
//   warp  9     MMA issuer (one elected thread): S = Q K^T and O += P V on tcgen05
// Tensor memory (512 columns): S0 | S1 | O0 | O1, 128 columns each.  The 16-bit probabilities are
// written back over the first 64 columns of their own S buffer and feed the second MMA straight
// from tensor memory.  While one group runs softmax on its tile the tensor pipe works on the other
// group's tile, so the two overlap.  A softmax thread pulls its whole 128-entry score row into
// registers with one wait, so the row maximum, the exponentials and the row sum need a single
// pass over tensor memory.  O leaves through shared memory (the CTA's own Q tile, dead by then)
// and a TMA store.
//
// CTAs are numbered so that, inside a group of `unit_group` (batch, head) slices, the tile pairs
// with the most K/V tiles (the latest rows under a causal mask) start first, while the slices that
// run at the same time stay few enough for their K and V to sit in L2.
//
// Follows the reference's forward (train/acctransformer/flash_attention/ops/flash_attention/
// flash_attention_fwd.py:308-457): per K/V tile  S -> (+alibi, +mask*-10000) -> running max ->
// exp -> row sum (before dropout) -> dropout -> O = O*e^(m_old-m_new) + P V, and at the end
// O / l and L = m + ln l (:258-306).  The running max is only refreshed when it grows by more than
// 8 (in log2 units); P, l and O then share the same stale offset, which cancels in O / l and in L.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "fa_common.cuh"
#include "fa_kernels.cuh"
#include "ptx.cuh"

namespace acct {

namespace {

constexpr int kFwdThreads = 384;   // warps 10 and 11 only complete the third warpgroup (register re-split)
constexpr int kRegsSoftmax = 208, kRegsControl = 88;
constexpr int kStages = 2;   // K/V ring depth for head_dim <= 128 (one stage above that)
constexpr float kRescaleThreshold = 8.0f;   // log2 units

struct TileRange {
  int lo, hi;   // inclusive K/V tile indices; empty when lo > hi
};

// K/V tiles that Q tile `i` needs: the block band  j - next <= i <= j + prev, the causal triangle,
// the TriangleAttention row groups and the valid key length.
__device__ __forceinline__ TileRange kv_tile_range(int i, int s_q, int kv_len, const ScoreMods& m) {
  TileRange r;
  if (i * kTile >= s_q || kv_len <= 0) { r.lo = 0; r.hi = -1; return r; }
  r.lo = 0;
  r.hi = (kv_len + kTile - 1) / kTile - 1;
  if (m.prev_block_num < 65536) r.lo = max(r.lo, i - m.prev_block_num);
  if (m.next_block_num < 65536) r.hi = min(r.hi, i + m.next_block_num);
  if (m.causal) r.hi = min(r.hi, i);
  if (m.tri_block > 0) {
    // the tile's last row belongs to the latest row group of the tile, which sees the most keys
    const int last_row = min(i * kTile + kTile - 1, s_q - 1);
    const int q_end = (last_row / m.tri_block + 1) * m.tri_block;
    r.hi = min(r.hi, (q_end - 1) / kTile);
  }
  return r;
}

struct FwdShared {
  uint64_t q_full;
  uint64_t k_full[kStages], k_empty[kStages];
  uint64_t v_full[kStages], v_empty[kStages];
  uint64_t s_full[2], p_half[2], p_ready[2], o_done[2];
  uint32_t tmem_base;
  volatile uint32_t abort_flag;
  alignas(16) float alibi[2][2][kTile];   // [softmax group][tile parity]: alibi row of the K/V tile, log2 units
};

}  // namespace

// MODS: bit 0 = a mask tensor may be present, bit 1 = alibi may be present.  DROP: 0 no dropout, 1 in-kernel
// generator, 2 dropout mask tensor of any type, 3 uint8 {0,1} mask tensor with 16-byte aligned rows read as byte masks.  Every instantiation carries only the code of what it may meet: code that is
// compiled in but never run still costs the common path of every tile (register allocation, spills).
template <int DPAD, bool BF16, int MODS, int DROP>
__global__ void __launch_bounds__(kFwdThreads, 1) fa_fwd_kernel(const __grid_constant__ FwdParams p) {
  constexpr int NB = DPAD / 64;                 // 64-column (128-byte) blocks per row
  constexpr uint32_t kTileBytes = NB * 16384u;  // one 128-row tile
  // head_dim in (128, 256]: O takes 256 columns of tensor memory and a K or V tile 64 KB of shared memory, so a
  // CTA then owns ONE Q tile (softmax group 1 idles) and K and V have one stage each.
  constexpr int NQ = DPAD > 128 ? 1 : 2;        // Q tiles per CTA
  constexpr int kSt = DPAD > 128 ? 1 : kStages;  // K/V stages
  constexpr uint32_t kColS = 0, kColO = NQ * 128;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;                          // 2 tiles; reused as the staging of O at the end
  uint8_t* sK = sQ + NQ * kTileBytes;          // kSt tiles
  uint8_t* sV = sK + kSt * kTileBytes;         // kSt tiles
  __shared__ FwdShared sh;

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const ScoreMods& mods = p.mods;

  // linear CTA number -> ((batch, head) slice, tile pair): groups of unit_group slices, heaviest pairs first
  const int n_pairs = (p.S_q + NQ * kTile - 1) / (NQ * kTile);
  const int n_units = p.B * p.N;
  int bh, pair;
  {
    const int kUnitGroup = p.unit_group;
    const int per_group = n_pairs * kUnitGroup;
    const int g = blockIdx.x / per_group;
    const int within = blockIdx.x % per_group;
    const int g_units = min(kUnitGroup, n_units - g * kUnitGroup);
    pair = n_pairs - 1 - within / g_units;
    bh = g * kUnitGroup + within % g_units;
  }
  const int b = bh / p.N, h = bh % p.N;
  const int h_kv = h / p.kv_group;   // grouped-query attention: several query heads read one key/value head

  int kv_len = p.S_k;
  if (mods.seq_lens != nullptr) kv_len = min(p.S_k, max(0, mods.seq_lens[b]));

  const TileRange r0 = kv_tile_range(NQ * pair, p.S_q, kv_len, mods);
  TileRange r1 = kv_tile_range(NQ * pair + 1, p.S_q, kv_len, mods);
  if (NQ == 1) { r1.lo = 0; r1.hi = -1; }
  const bool any0 = r0.lo <= r0.hi, any1 = r1.lo <= r1.hi;
  int cta_lo = 0, cta_hi = -1;
  if (any0 && any1) { cta_lo = min(r0.lo, r1.lo); cta_hi = max(r0.hi, r1.hi); }
  else if (any0) { cta_lo = r0.lo; cta_hi = r0.hi; }
  else if (any1) { cta_lo = r1.lo; cta_hi = r1.hi; }

  if (tid == 0) {
    mbar_init(&sh.q_full, 1);
    for (int s = 0; s < kSt; ++s) {
      mbar_init(&sh.k_full[s], 1); mbar_init(&sh.k_empty[s], 1);
      mbar_init(&sh.v_full[s], 1); mbar_init(&sh.v_empty[s], 1);
    }
    for (int q = 0; q < 2; ++q) {
      mbar_init(&sh.s_full[q], 1); mbar_init(&sh.p_half[q], 128); mbar_init(&sh.p_ready[q], 128);
      mbar_init(&sh.o_done[q], 1);
    }
    sh.abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 8) { tmem_alloc(&sh.tmem_base, 512); tmem_relinquish(); }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = sh.tmem_base;
  volatile uint32_t* abort_flag = &sh.abort_flag;

  if (warp == 8) {
    // ------------------------------------------------------------------ TMA producer
    reg_dealloc<kRegsControl>();
    if (lane == 0 && cta_hi >= cta_lo) {
      prefetch_tmap(&p.map_q); prefetch_tmap(&p.map_k); prefetch_tmap(&p.map_v); prefetch_tmap(&p.map_o);
      mbar_expect_tx(&sh.q_full, NQ * kTileBytes);
      for (int qt = 0; qt < NQ; ++qt)
        for (int nb = 0; nb < NB; ++nb)
          tma_load_4d(sQ + qt * kTileBytes + nb * 16384, &p.map_q, &sh.q_full, nb * 64,
                      (NQ * pair + qt) * kTile, h, b);
      int it = 0;
      for (int j = cta_lo; j <= cta_hi; ++j, ++it) {
        const int st = it % kSt;
        const uint32_t reuse_parity = ((it / kSt) - 1) & 1;
        if (it >= kSt) mbar_wait(&sh.k_empty[st], reuse_parity, abort_flag, p.status, DEV_TIMEOUT_SYNC);
        mbar_expect_tx(&sh.k_full[st], kTileBytes);
        for (int nb = 0; nb < NB; ++nb)
          tma_load_4d(sK + st * kTileBytes + nb * 16384, &p.map_k, &sh.k_full[st], nb * 64, j * kTile, h_kv, b);
        if (it >= kSt) mbar_wait(&sh.v_empty[st], reuse_parity, abort_flag, p.status, DEV_TIMEOUT_SYNC);
        mbar_expect_tx(&sh.v_full[st], kTileBytes);
        for (int nb = 0; nb < NB; ++nb)
          tma_load_4d(sV + st * kTileBytes + nb * 16384, &p.map_v, &sh.v_full[st], nb * 64, j * kTile, h_kv, b);
      }
    }
  } else if (warp == 9) {
    // ------------------------------------------------------------------ MMA issuer
    // The tensor pipe takes the MMAs at the rate it executes them and holds only a couple in its queue, so
    // whatever this thread does between two MMAs is time the pipe may idle.  Hence: descriptors are stepped
    // with one 32-bit add, the waits on the K/V ring (long satisfied when they are reached) are placed right
    // behind a burst of MMAs that is still executing, and each hand-off from the softmax groups is waited
    // for once.
    reg_dealloc<kRegsControl>();
    if (lane == 0 && cta_hi >= cta_lo) {
      const uint32_t idesc_s = make_idesc(BF16, 128, 128, false, false);
      const uint32_t idesc_o = make_idesc(BF16, 128, DPAD, false, true);
      const uint64_t kmajor = make_sdesc_base(16, 1024);
      const uint64_t mnmajor = make_sdesc_base(16384, 1024);
      const uint32_t k_hi = static_cast<uint32_t>(kmajor >> 32), k_lo = static_cast<uint32_t>(kmajor);
      const uint32_t mn_hi = static_cast<uint32_t>(mnmajor >> 32), mn_lo = static_cast<uint32_t>(mnmajor);
      const TileRange rng[2] = {r0, r1};
      int n_done[2] = {0, 0};   // P tiles consumed so far per Q tile
      // low descriptor words of the tile bases (all tiles are 1024-byte aligned, so offsets simply add)
      const uint32_t q_lo = k_lo | ((smem_u32(sQ) >> 4) & 0x3fffu);
      const uint32_t kt_lo = k_lo | ((smem_u32(sK) >> 4) & 0x3fffu);
      const uint32_t vt_lo = mn_lo | ((smem_u32(sV) >> 4) & 0x3fffu);
      constexpr uint32_t kTileUnits = kTileBytes >> 4;
      mbar_wait(&sh.q_full, 0, abort_flag, p.status, DEV_TIMEOUT_TMA);

      auto issue_s = [&](int qt, int st) {
        const uint32_t a0 = q_lo + qt * kTileUnits, b0 = kt_lo + st * kTileUnits;
#pragma unroll
        for (int kk = 0; kk < DPAD / 16; ++kk) {
          const uint32_t off = (kk >> 2) * 1024u + (kk & 3) * 2u;   // 16-byte units
          umma_ss_lohi(tmem + kColS + qt * 128, a0 + off, k_hi, b0 + off, k_hi, idesc_s, kk > 0);
        }
        umma_commit(&sh.s_full[qt]);
      };

      // prologue: scores of the first K/V tile
      mbar_wait(&sh.k_full[0], 0, abort_flag, p.status, DEV_TIMEOUT_TMA);
      for (int qt = 0; qt < 2; ++qt)
        if (cta_lo >= rng[qt].lo && cta_lo <= rng[qt].hi) issue_s(qt, 0);
      umma_commit(&sh.k_empty[0]);
      mbar_wait(&sh.v_full[0], 0, abort_flag, p.status, DEV_TIMEOUT_TMA);
      int it = 0;
      for (int j = cta_lo; j <= cta_hi; ++j, ++it) {
        const int st = it % kSt;
        const int stn = (it + 1) % kSt;
        const uint32_t full_parity_n = ((it + 1) / kSt) & 1;
        const bool more = j + 1 <= cta_hi;
        bool k_seen = false;   // K tile j+1 seen full
        for (int qt = 0; qt < 2; ++qt) {
          const bool pv = j >= rng[qt].lo && j <= rng[qt].hi;
          const bool sn = more && j + 1 >= rng[qt].lo && j + 1 <= rng[qt].hi;
          const uint32_t t_s = tmem + kColS + qt * 128, t_o = tmem + kColO + qt * DPAD;
          const uint32_t v0 = vt_lo + st * kTileUnits;
          if (pv) {
            // P arrives in two halves (key rows 0-63, then 64-127 of the V tile, which was seen full before)
            mbar_wait(&sh.p_half[qt], n_done[qt] & 1, abort_flag, p.status, DEV_TIMEOUT_SYNC);
            tc_fence_after_sync();
#pragma unroll
            for (int kk = 0; kk < kTile / 32; ++kk)
              umma_ts_lohi(t_o, t_s + kk * 8, v0 + kk * 128u, mn_hi, idesc_o, n_done[qt] > 0 || kk > 0);
          }
          if (sn && !k_seen) {
            mbar_wait(&sh.k_full[stn], full_parity_n, abort_flag, p.status, DEV_TIMEOUT_TMA);
            k_seen = true;
          }
          if (pv) {
            mbar_wait(&sh.p_ready[qt], n_done[qt] & 1, abort_flag, p.status, DEV_TIMEOUT_SYNC);
            tc_fence_after_sync();
#pragma unroll
            for (int kk = kTile / 32; kk < kTile / 16; ++kk)
              umma_ts_lohi(t_o, t_s + kk * 8, v0 + kk * 128u, mn_hi, idesc_o, true);
            // O is only looked at after the Q tile's last K/V tile (the rescaling of earlier tiles is ordered by
            // s_full: the S product it waits for was issued after their P V), so one commit per Q tile is enough --
            // every commit costs this thread 80-95 cycles in which it issues nothing
            if (j == rng[qt].hi) umma_commit(&sh.o_done[qt]);
            ++n_done[qt];
          }
          if (sn) issue_s(qt, stn);
        }
        umma_commit(&sh.v_empty[st]);
        if (more) {
          umma_commit(&sh.k_empty[stn]);
          // the next V tile, waited for while the MMAs just issued still execute
          mbar_wait(&sh.v_full[stn], full_parity_n, abort_flag, p.status, DEV_TIMEOUT_TMA);
        }
      }
    }
  } else if (warp >= 10) {
    reg_dealloc<kRegsControl>();
  } else {
    // ------------------------------------------------------------------ softmax groups
    reg_alloc<kRegsSoftmax>();
    const int qt = warp >> 2;
    const TileRange rng = qt == 0 ? r0 : r1;
    const int q_tile = NQ * pair + qt;
    const int row_in_tile = tid & 127;
    const int q_row = q_tile * kTile + row_in_tile;
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t t_s = tmem + lane_base + kColS + qt * 128;
    const uint32_t t_o = tmem + lane_base + kColO + qt * DPAD;
    constexpr bool GENERIC = MODS != 0;
    const bool has_alibi = (MODS & 2) != 0 && (mods.alibi != nullptr || mods.alibi_slopes != nullptr);
    const float slope_l2 = mods.alibi_slopes != nullptr ? mods.alibi_slopes[h] * kLog2e : 0.f;
    const int64_t alibi_row = static_cast<int64_t>(bh) * p.S_k;
    const int64_t mask_row =
        (static_cast<int64_t>(mods.mask_batch > 1 ? b : 0) * p.S_q + min(q_row, p.S_q - 1)) * p.S_k;
    const int64_t drop_row = (static_cast<int64_t>(bh) * p.S_q + min(q_row, p.S_q - 1)) * p.S_k;

    // Keys at or past `bound` do not exist for this thread's row: valid length, TriangleAttention row
    // group, causal triangle.  `bound_tile` is the smallest bound of any row of the tile.
    const int tri_end = mods.tri_block > 0 ? (min(q_row, p.S_q - 1) / mods.tri_block + 1) * mods.tri_block : 0x7fffffff;
    const int tri_end_tile = mods.tri_block > 0 ? ((q_tile * kTile) / mods.tri_block + 1) * mods.tri_block : 0x7fffffff;
    const int bound = min(min(kv_len, tri_end), mods.causal ? q_row + 1 : 0x7fffffff);
    const int bound_tile = min(min(kv_len, tri_end_tile), mods.causal ? q_tile * kTile + 1 : 0x7fffffff);

    // Optional per-tile summary of a full mask tensor: the class of tile (q_tile, j) is fetched one tile ahead,
    // before the wait for S, so that its latency is not on the path.
    const uint8_t* tile_class = nullptr;
    if constexpr ((MODS & 1) != 0) if (mods.mask_kind == 1 && mods.mask_tiles != nullptr)
      tile_class = mods.mask_tiles + (static_cast<int64_t>(mods.mask_batch > 1 ? b : 0) * ((p.S_q + kTile - 1) / kTile) +
                                      min(q_tile, (p.S_q - 1) / kTile)) * ((p.S_k + kTile - 1) / kTile);
    int mask_class = 1, mask_class_next = 1;
    if (tile_class != nullptr && rng.lo <= rng.hi) mask_class_next = tile_class[rng.lo];
    // alibi tensor: this thread's column of the next K/V tile, fetched one tile ahead and left raw until it is parked
    // in shared memory (arithmetic on a fresh load would stall the warp for the whole memory latency)
    const uint16_t* alibi_raw = reinterpret_cast<const uint16_t*>(mods.alibi) + alibi_row;
    uint16_t al_raw = 0, al_raw_next = 0;
    if constexpr ((MODS & 2) != 0) if (mods.alibi != nullptr && rng.lo <= rng.hi)
      al_raw_next = alibi_raw[min(rng.lo * kTile + row_in_tile, p.S_k - 1)];

    float m_run = kNegInf, l_run = 0.f;
    int n = 0;
    for (int j = rng.lo; j <= rng.hi; ++j, ++n) {
      mask_class = mask_class_next;
      if (tile_class != nullptr && j < rng.hi) mask_class_next = tile_class[j + 1];
      if constexpr ((MODS & 2) != 0) if (mods.alibi != nullptr) {
        al_raw = al_raw_next;
        if (j < rng.hi) al_raw_next = alibi_raw[min((j + 1) * kTile + row_in_tile, p.S_k - 1)];
      }
      mbar_wait(&sh.s_full[qt], n & 1, abort_flag, p.status, DEV_TIMEOUT_MMA);
      tc_fence_after_sync();
      const int col_base = j * kTile;
      // a mask tile that is all 1 adds one constant to every score of the tile: without alibi it is folded into
      // the exponent's offset below and the tile takes the plain path
      const bool mask_const = (MODS & 1) != 0 && mods.mask_kind == 1 && mask_class == 2 && !has_alibi;
      const bool use_mask = (MODS & 1) != 0 && ((mods.mask_kind == 1 && mask_class != 0 && !mask_const) ||
                                                (mods.mask_kind == 2 && j == q_tile));
      const float tile_add = mask_const ? -10000.0f * kLog2e : 0.f;
      const bool generic = GENERIC && (use_mask || has_alibi);
      const bool partial = col_base + kTile > bound_tile;   // some (row, key) pairs of this tile do not exist

      float mult = p.scale_log2;
      if constexpr (GENERIC) if (generic) {
        // general path: alibi and / or a mask tensor; values leave in log2 units
        mult = 1.0f;
        // the alibi row of this K/V tile goes through shared memory: one value per thread of the group,
        // double-buffered by tile parity so that one barrier per tile is enough
        float* al = sh.alibi[qt][n & 1];
        if constexpr ((MODS & 2) != 0) if (mods.alibi != nullptr) {
          const float a = BF16 ? __uint_as_float(static_cast<uint32_t>(al_raw) << 16) : __half2float(__ushort_as_half(al_raw));
          al[row_in_tile] = col_base + row_in_tile < p.S_k ? a * kLog2e : 0.f;
          named_barrier(1 + qt, 128);
        }
        // mask values are read 32 at a time (128-bit loads when the row segment is aligned and complete)
        const bool mask_vec = col_base + kTile <= p.S_k && (p.S_k & 15) == 0 &&
                              (reinterpret_cast<uintptr_t>(mods.mask) & 15u) == 0;
        if constexpr ((MODS & 1) != 0) if (use_mask)
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {   // one 32-column chunk at a time, rewritten in place in tensor memory
          uint32_t sc[32];
          tmem_ld32(t_s + c * 32, sc);
          float add[32];
          if (use_mask) {
            if (mods.mask_kind == 1 && mask_class == 2) {
#pragma unroll
              for (int i = 0; i < 32; ++i) add[i] = -10000.0f * kLog2e;
            } else if (mods.mask_kind == 1)
              load_row32(mods.mask, mods.mask_dtype, mask_row + col_base + c * 32, p.S_k - (col_base + c * 32), mask_vec,
                         -10000.0f * kLog2e, add);
            else
              load_row32(mods.mask, mods.mask_dtype, static_cast<int64_t>(row_in_tile) * kTile + c * 32, 32,
                         (reinterpret_cast<uintptr_t>(mods.mask) & 15u) == 0, -10000.0f * kLog2e, add);
          }
          else {
#pragma unroll
            for (int i = 0; i < 32; ++i) add[i] = 0.f;
          }
          // the branches are on tile-uniform conditions and sit outside the element loops
          if constexpr ((MODS & 2) != 0) if (mods.alibi != nullptr) {
#pragma unroll
            for (int i4 = 0; i4 < 8; ++i4) {
              const float4 a4 = *reinterpret_cast<const float4*>(al + c * 32 + 4 * i4);
              add[4 * i4] += a4.x; add[4 * i4 + 1] += a4.y; add[4 * i4 + 2] += a4.z; add[4 * i4 + 3] += a4.w;
            }
          }
          if constexpr ((MODS & 2) != 0) if (mods.alibi == nullptr && mods.alibi_slopes != nullptr) {
#pragma unroll
            for (int i = 0; i < 32; ++i) add[i] = fmaf(slope_l2, static_cast<float>(col_base + c * 32 + i), add[i]);
          }
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float x = fmaf(__uint_as_float(sc[i]), p.scale_log2, add[i]);
            sc[i] = __float_as_uint(col_base + c * 32 + i >= bound ? kNegInf : x);
          }
          tmem_st32(t_s + c * 32, sc);
        }
        if (use_mask) tmem_wait_st();
      }

      // the whole score row in registers, one wait
      uint32_t s[4][32];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld32(t_s + c * 32, s[c]);
      tmem_wait_ld();

      if constexpr ((MODS & 2) != 0) if (generic && !use_mask) {
        // alibi only: added in registers, in log2 units (no pass through tensor memory), two scores per instruction;
        // positions that do not exist are only looked for in tiles that have any (`partial`)
        const uint64_t sc2 = f2_pack(p.scale_log2, p.scale_log2);
        if (mods.alibi != nullptr) {
          const float* al = sh.alibi[qt][n & 1];
#pragma unroll
          for (int c = 0; c < 4; ++c)
#pragma unroll
            for (int i4 = 0; i4 < 8; ++i4) {
              const float4 a4 = *reinterpret_cast<const float4*>(al + c * 32 + 4 * i4);
              float x0, x1, x2, x3;
              f2_unpack(f2_fma(f2_pack(__uint_as_float(s[c][4 * i4]), __uint_as_float(s[c][4 * i4 + 1])), sc2, f2_pack(a4.x, a4.y)), x0, x1);
              f2_unpack(f2_fma(f2_pack(__uint_as_float(s[c][4 * i4 + 2]), __uint_as_float(s[c][4 * i4 + 3])), sc2, f2_pack(a4.z, a4.w)), x2, x3);
              s[c][4 * i4] = __float_as_uint(x0); s[c][4 * i4 + 1] = __float_as_uint(x1);
              s[c][4 * i4 + 2] = __float_as_uint(x2); s[c][4 * i4 + 3] = __float_as_uint(x3);
            }
        } else {
          // bias = slope * key position = slope * (first key of the tile) + slope * (offset inside the tile): the second
          // factor is a compile-time constant, so no integer-to-float conversion competes with the exponentials
          const float base = slope_l2 * static_cast<float>(col_base);
          const uint64_t base2 = f2_pack(base, base), slope2 = f2_pack(slope_l2, slope_l2);
#pragma unroll
          for (int c = 0; c < 4; ++c)
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
              const uint64_t bias2 = f2_fma(slope2, f2_pack(static_cast<float>(c * 32 + i), static_cast<float>(c * 32 + i + 1)), base2);
              float x0, x1;
              f2_unpack(f2_fma(f2_pack(__uint_as_float(s[c][i]), __uint_as_float(s[c][i + 1])), sc2, bias2), x0, x1);
              s[c][i] = __float_as_uint(x0); s[c][i + 1] = __float_as_uint(x1);
            }
        }
        if (partial) {
#pragma unroll
          for (int c = 0; c < 4; ++c)
#pragma unroll
            for (int i = 0; i < 32; ++i)
              s[c][i] = (col_base + c * 32 + i >= bound) ? __float_as_uint(kNegInf) : s[c][i];
        }
      }
      if (!generic && partial) {
        // only positions that do not exist: one compare + select per element, no branches
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i)
            s[c][i] = (col_base + c * 32 + i >= bound) ? __float_as_uint(kNegInf) : s[c][i];
      }

      // One 32-column chunk: P = exp2(x * mult - m) packed to 16 bits, row sum (before dropout) into `l4`.
      // Two-wide fp32 instructions do the scaling and the sum in half the issue slots.
      const uint64_t mult2 = f2_pack(mult, mult);
      auto exp_chunk = [&](int c, uint64_t negm2, uint64_t (&l4)[4], uint32_t (&pk)[16]) {
        bool dropped = false;
        if constexpr (DROP != 0) {
          dropped = true;
          const int col0 = col_base + c * 32;
          if constexpr (DROP == 1 || DROP == 3) {
            // DROP 1: the mask is computed, not loaded: two generator calls give this row's 32 keep decisions of the
            // chunk as byte masks.  DROP 3: a uint8 {0,1} mask tensor (16-byte aligned rows): the row's 32 bytes come
            // with two 128-bit loads and become byte masks by one multiplication per word (addresses clamped into the
            // row: keys past S_k get other keys' bytes, their P is 0 anyway).  Either way the byte masks are widened
            // to 16-bit lane masks and ANDed onto the packed, scaled probabilities (a dropped probability becomes +0,
            // as p * 0 would).
            uint32_t km[8];
            if constexpr (DROP == 1) {
              const DropoutRng rng = {mods.drop_seed_lo, mods.drop_seed_hi, mods.drop_offset, mods.drop_threshold};
              const uint32_t q_u = static_cast<uint32_t>(min(q_row, p.S_q - 1)), k16 = static_cast<uint32_t>(col0) >> 4;
              dropout_keep16_bytes(rng, static_cast<uint32_t>(bh), q_u, k16, *reinterpret_cast<uint32_t(*)[4]>(&km[0]));
              dropout_keep16_bytes(rng, static_cast<uint32_t>(bh), q_u, k16 + 1, *reinterpret_cast<uint32_t(*)[4]>(&km[4]));
            } else {
              const uint8_t* row = reinterpret_cast<const uint8_t*>(mods.drop) + drop_row;
              const uint4 u0 = *reinterpret_cast<const uint4*>(row + min(col0, p.S_k - 16));
              const uint4 u1 = *reinterpret_cast<const uint4*>(row + min(col0 + 16, p.S_k - 16));
              km[0] = (u0.x & 0x01010101u) * 255u; km[1] = (u0.y & 0x01010101u) * 255u;
              km[2] = (u0.z & 0x01010101u) * 255u; km[3] = (u0.w & 0x01010101u) * 255u;
              km[4] = (u1.x & 0x01010101u) * 255u; km[5] = (u1.y & 0x01010101u) * 255u;
              km[6] = (u1.z & 0x01010101u) * 255u; km[7] = (u1.w & 0x01010101u) * 255u;
            }
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              float x0, x1;
              f2_unpack(f2_fma(f2_pack(__uint_as_float(s[c][2 * i]), __uint_as_float(s[c][2 * i + 1])), mult2, negm2), x0, x1);
              const float p0 = ex2(x0), p1 = ex2(x1);
              l4[i & 3] = f2_add(l4[i & 3], f2_pack(p0, p1));
              // elements 2i, 2i+1 of the chunk are bytes (2i & 3), (2i & 3) + 1 of word i / 2
              const uint32_t lanes = __byte_perm(km[i >> 1], 0u, (i & 1) ? 0x3322u : 0x1100u);
              pk[i] = pack2<BF16>(__fmul_rn(p0, mods.drop_scale), __fmul_rn(p1, mods.drop_scale)) & lanes;
            }
          } else {
            float f[32];
            const bool drop_vec = col_base + kTile <= p.S_k && (p.S_k & 15) == 0 &&
                                  (reinterpret_cast<uintptr_t>(mods.drop) & 15u) == 0;
            load_row32(mods.drop, mods.drop_dtype, drop_row + col0, p.S_k - col0, drop_vec, mods.drop_scale, f);
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              float x0, x1;
              f2_unpack(f2_fma(f2_pack(__uint_as_float(s[c][2 * i]), __uint_as_float(s[c][2 * i + 1])), mult2, negm2), x0, x1);
              const float p0 = ex2(x0), p1 = ex2(x1);
              l4[i & 3] = f2_add(l4[i & 3], f2_pack(p0, p1));
              pk[i] = pack2<BF16>(__fmul_rn(p0, f[2 * i]), __fmul_rn(p1, f[2 * i + 1]));
            }
          }
        }
        if (!dropped) {
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            float x0, x1;
            f2_unpack(f2_fma(f2_pack(__uint_as_float(s[c][2 * i]), __uint_as_float(s[c][2 * i + 1])), mult2, negm2), x0, x1);
            const float p0 = ex2(x0), p1 = ex2(x1);
            l4[i & 3] = f2_add(l4[i & 3], f2_pack(p0, p1));
            pk[i] = pack2<BF16>(p0, p1);
          }
        }
      };

      // The running maximum rarely moves after the first tiles (it is only refreshed when it grows by more than
      // the threshold), so from the second tile on the exponentials of chunk 0 are started with the old maximum
      // while the row maximum of the tile is still being formed (four independent chains of three-input maxima,
      // which fill the gaps the exponential unit leaves).  If some row of the warp does need a new maximum, that
      // chunk is simply computed again.
      uint64_t l_part[4] = {0ull, 0ull, 0ull, 0ull};
      uint32_t pk0[16];
      const bool speculate = n > 0;
      if (speculate) {
        float m_old = (m_run == kNegInf) ? 0.f : m_run;
        if constexpr ((MODS & 1) != 0) m_old -= tile_add;
        exp_chunk(0, f2_pack(-m_old, -m_old), l_part, pk0);
      }
      float mx[4];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        mx[c] = fmaxf(__uint_as_float(s[c][0]), __uint_as_float(s[c][31]));
#pragma unroll
        for (int i = 1; i < 31; i += 2) mx[c] = fmax3(mx[c], __uint_as_float(s[c][i]), __uint_as_float(s[c][i + 1]));
      }
      float m_tile = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * mult;   // scale > 0
      if constexpr ((MODS & 1) != 0) m_tile += tile_add;

      const float m_new = fmaxf(m_run, m_tile);
      const bool grow = (m_new > m_run + kRescaleThreshold) || (m_run == kNegInf && m_new != kNegInf);
      const bool any_grow = __any_sync(0xffffffffu, grow);
      float alpha = 1.0f;
      if (grow) {
        alpha = (m_run == kNegInf) ? 0.f : ex2(m_run - m_new);
        m_run = m_new;
        l_run *= alpha;
      }
      if (n > 0 && any_grow) {
        // O of the previous tiles is complete (the S MMA just waited for was issued after their P V)
#pragma unroll 1
        for (int c = 0; c < DPAD / 32; ++c) {
          uint32_t r[32];
          tmem_ld32(t_o + c * 32, r);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
          tmem_st32(t_o + c * 32, r);
        }
      }
      float m_use = (m_run == kNegInf) ? 0.f : m_run;
      if constexpr ((MODS & 1) != 0) m_use -= tile_add;
      const uint64_t negm2 = f2_pack(-m_use, -m_use);
      if (!speculate || any_grow) {
#pragma unroll
        for (int i = 0; i < 4; ++i) l_part[i] = 0ull;
        exp_chunk(0, negm2, l_part, pk0);
      }
      tmem_st16(t_s, pk0);
      // 16-bit P goes back over the S buffer; the first half is handed to the MMA warp as soon as it is stored
      {
        uint32_t pk[16];
        exp_chunk(1, negm2, l_part, pk);
        tmem_st16(t_s + 16, pk);
        tmem_wait_st();
        tc_fence_before_sync();
        mbar_arrive(&sh.p_half[qt]);
      }
      {
        // the second half as one store: the exponentials of chunk 3 overlap the tail of chunk 2
        uint32_t pk2[16], pk3[16], pk[32];
        exp_chunk(2, negm2, l_part, pk2);
        exp_chunk(3, negm2, l_part, pk3);
#pragma unroll
        for (int i = 0; i < 16; ++i) { pk[i] = pk2[i]; pk[16 + i] = pk3[i]; }
        tmem_st32(t_s + 32, pk);
      }
      {
        float a0, a1;
        f2_unpack(f2_add(f2_add(l_part[0], l_part[1]), f2_add(l_part[2], l_part[3])), a0, a1);
        l_run += a0 + a1;
      }
      tmem_wait_st();
      tc_fence_before_sync();
      mbar_arrive(&sh.p_ready[qt]);
    }

    // epilogue: O / l through this group's (now dead) Q tile in shared memory and a TMA store, which
    // clips rows past S_q and columns past D; L = m + ln l straight to global memory
    if (qt < NQ && q_tile * kTile < p.S_q) {
      if (n > 0) {
        mbar_wait(&sh.o_done[qt], 0, abort_flag, p.status, DEV_TIMEOUT_MMA);
        tc_fence_after_sync();
      } else if (cta_hi >= cta_lo) {
        // no K/V tile for this Q tile, but its TMA load was issued: let it land before the tile is reused
        mbar_wait(&sh.q_full, 0, abort_flag, p.status, DEV_TIMEOUT_TMA);
      }
      const float inv_l = (n > 0 && l_run > 0.f) ? 1.0f / l_run : 0.f;
      uint8_t* stage = sQ + qt * kTileBytes;
#pragma unroll 1
      for (int c = 0; c < DPAD / 32; ++c) {
        uint32_t r[32];
        if (n > 0) { tmem_ld32(t_o + c * 32, r); tmem_wait_ld(); }
        else {
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = 0u;
        }
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i)
          pk[i] = pack2<BF16>(__uint_as_float(r[2 * i]) * inv_l, __uint_as_float(r[2 * i + 1]) * inv_l);
        uint8_t* blk = stage + (c >> 1) * 16384u;
#pragma unroll
        for (int g = 0; g < 4; ++g)
          *reinterpret_cast<uint4*>(blk + swz128(row_in_tile, (c & 1) * 4 + g)) =
              make_uint4(pk[4 * g], pk[4 * g + 1], pk[4 * g + 2], pk[4 * g + 3]);
      }
      fence_proxy_async_smem();
      named_barrier(1 + qt, 128);
      if (row_in_tile == 0) {
        for (int nb = 0; nb < NB; ++nb)
          if (nb * 64 < p.D) tma_store_4d(&p.map_o, stage + nb * 16384, nb * 64, q_tile * kTile, h, b);
        tma_store_commit();
        tma_store_wait_read();
      }
      if (q_row < p.S_q && p.lse != nullptr)
        p.lse[static_cast<int64_t>(bh) * p.S_q + q_row] =
            (n > 0 && l_run > 0.f) ? m_run * kLn2 + logf(l_run) : kNegInf;
    }
    tc_fence_before_sync();
  }

  linger_after_abort(abort_flag);
  __syncthreads();
  if (warp == 8) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, 512);
  }
}

// One thread per (unit, query, 16 keys): one generator call, 16 mask bytes.
__global__ void dropout_mask_kernel(unsigned char* mask, int units, int S_q, int S_k, DropoutRng rng) {
  const int groups = (S_k + 15) / 16;
  const int64_t total = static_cast<int64_t>(units) * S_q * groups;
  for (int64_t t = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; t < total;
       t += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int g = static_cast<int>(t % groups);
    const int64_t row = t / groups;               // unit * S_q + q
    const int q = static_cast<int>(row % S_q);
    const int unit = static_cast<int>(row / S_q);
    const uint32_t bits = dropout_keep16(rng, static_cast<uint32_t>(unit), static_cast<uint32_t>(q), static_cast<uint32_t>(g));
    unsigned char* dst = mask + row * S_k + g * 16;
    const int n = min(16, S_k - g * 16);
    for (int i = 0; i < n; ++i) dst[i] = (bits >> i) & 1u;
  }
}

cudaError_t launch_dropout_mask(unsigned char* mask, int units, int S_q, int S_k, unsigned int seed_lo, unsigned int seed_hi,
                                unsigned int offset, unsigned int threshold, cudaStream_t stream) {
  const int64_t total = static_cast<int64_t>(units) * S_q * ((S_k + 15) / 16);
  const int64_t blocks = (total + 255) / 256;
  const DropoutRng rng = {seed_lo, seed_hi, offset, threshold};
  dropout_mask_kernel<<<static_cast<unsigned>(blocks < 148 * 32 ? (blocks < 1 ? 1 : blocks) : 148 * 32), 256, 0, stream>>>(
      mask, units, S_q, S_k, rng);
  return cudaGetLastError();
}

// One thread per element pair of rows would be wasteful; a thread walks elements with a grid stride and flags the
// first difference from the causal mask (1 above the diagonal, 0 on and below it).
__global__ void mask_check_kernel(const void* mask, int dtype, int64_t total, int S_q, int S_k, unsigned int* mismatch) {
  unsigned int bad = 0;
  for (int64_t t = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; t < total;
       t += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int k = static_cast<int>(t % S_k);
    const int q = static_cast<int>((t / S_k) % S_q);
    const float want = k > q ? 1.0f : 0.0f;
    bad |= (load_mask_value(mask, dtype, t) != want) ? 1u : 0u;
  }
  if (__any_sync(0xffffffffu, bad != 0u) && (threadIdx.x & 31) == 0) atomicOr(mismatch, 1u);
}

cudaError_t launch_mask_check(const void* mask, int dtype, int batch, int S_q, int S_k, unsigned int* mismatch,
                              cudaStream_t stream) {
  const int64_t total = static_cast<int64_t>(batch) * S_q * S_k;
  const int64_t blocks = (total + 255) / 256;
  mask_check_kernel<<<static_cast<unsigned>(blocks < 148 * 16 ? (blocks < 1 ? 1 : blocks) : 148 * 16), 256, 0, stream>>>(
      mask, dtype, total, S_q, S_k, mismatch);
  return cudaGetLastError();
}

// One block per 128x128 tile of a [batch, S_q, S_k] mask: class 0 if every element of the tile is 0, 2 if every
// element is 1, else 1.  VEC: the tile's rows are whole 16-byte vectors (row length a multiple of 16 bytes, aligned
// base, tile not cut by the right edge): a thread compares four 32-bit words per load with the bit pattern of 0 and
// of 1 (-0.0 then counts as "not 0": the tile is read, which is always right).  Otherwise one element per load.
template <bool VEC>
__global__ void mask_classify_kernel(const void* mask, int dtype, int S_q, int S_k, uint8_t* tiles) {
  const int64_t base = static_cast<int64_t>(blockIdx.z) * S_q * S_k;
  int nonzero = 0, notone = 0;
  const bool full_width = blockIdx.x * kTile + kTile <= S_k;
  if (VEC && full_width) {
    const int esize = dtype == 2 ? 1 : 2;
    const int vecs = kTile * esize / 16;                 // 16-byte vectors per tile row: 8 (u8) or 16
    const uint32_t one = dtype == 2 ? 0x01010101u : (dtype == 1 ? 0x3f803f80u : 0x3c003c00u);
    const int v = threadIdx.x % vecs;
    const uint8_t* p0 = static_cast<const uint8_t*>(mask) + (base + static_cast<int64_t>(blockIdx.x) * kTile) * esize + v * 16;
    for (int r = threadIdx.x / vecs; r < kTile; r += 256 / vecs) {
      const int row = blockIdx.y * kTile + r;
      if (row >= S_q) break;
      const uint4 u = *reinterpret_cast<const uint4*>(p0 + static_cast<int64_t>(row) * S_k * esize);
      nonzero |= (u.x | u.y | u.z | u.w) != 0u;
      notone |= (u.x != one) | (u.y != one) | (u.z != one) | (u.w != one);
    }
  } else {
    // thread t reads column t % 128 of every second row: a warp reads 32 consecutive elements of a row
    const int col = blockIdx.x * kTile + (threadIdx.x & 127);
    if (col < S_k) {
      for (int r = threadIdx.x >> 7; r < kTile; r += 2) {
        const int row = blockIdx.y * kTile + r;
        if (row >= S_q) break;
        const float v = load_mask_value(mask, dtype, base + static_cast<int64_t>(row) * S_k + col);
        nonzero |= (v != 0.0f);
        notone |= (v != 1.0f);
      }
    }
  }
  nonzero = __syncthreads_or(nonzero);
  notone = __syncthreads_or(notone);
  if (threadIdx.x == 0)
    tiles[(static_cast<int64_t>(blockIdx.z) * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x] =
        static_cast<uint8_t>(!nonzero ? 0 : (!notone ? 2 : 1));
}

cudaError_t launch_mask_classify(const void* mask, int dtype, int batch, int S_q, int S_k, uint8_t* tiles,
                                 cudaStream_t stream) {
  dim3 grid((S_k + kTile - 1) / kTile, (S_q + kTile - 1) / kTile, batch);
  const int esize = dtype == 2 ? 1 : 2;
  const bool vec = (static_cast<int64_t>(S_k) * esize) % 16 == 0 && (reinterpret_cast<uintptr_t>(mask) & 15u) == 0;
  if (vec) mask_classify_kernel<true><<<grid, 256, 0, stream>>>(mask, dtype, S_q, S_k, tiles);
  else mask_classify_kernel<false><<<grid, 256, 0, stream>>>(mask, dtype, S_q, S_k, tiles);
  return cudaGetLastError();
}

cudaError_t launch_fa_fwd(const FwdParams& p, bool bf16, cudaStream_t stream) {
  const int dpad = p.D <= 64 ? 64 : (p.D <= 128 ? 128 : 256);
  const int nq = dpad > 128 ? 1 : 2, stages = dpad > 128 ? 1 : kStages;
  const size_t smem = static_cast<size_t>(nq + 2 * stages) * (dpad / 64) * 16384 + 1024;
  const int n_pairs = (p.S_q + nq * kTile - 1) / (nq * kTile);
  dim3 grid(static_cast<unsigned>(n_pairs) * static_cast<unsigned>(p.B * p.N));
  // Slices per group: 8 (measured best from 4 096 keys up: larger groups lose more in L2 than the order gains).  Short
  // sequences have so few tile pairs per slice that two groups of 8 do not even fill the SMs once; heaviest-first
  // then balances nothing, and the group is widened until it gives every SM two thread blocks (K and V of a group,
  // what its thread blocks share through L2, stay small at such lengths; bounded by 48 MB all the same).
  FwdParams pp = p;
  {
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    long long group = 8;
    if (16ll * n_pairs <= sms) {
      const long long unit_bytes = 4ll * p.S_k * p.D;                    // K and V of one slice, 16-bit
      const long long fit = (48ll << 20) / (unit_bytes > 0 ? unit_bytes : 1);
      group = (2ll * sms + n_pairs - 1) / n_pairs;
      if (group > fit) group = fit;
      if (group < 8) group = 8;
      if (group > 256) group = 256;
    }
    pp.unit_group = static_cast<int>(group);
  }
  int mods = (p.mods.mask_kind != 0 ? 1 : 0) | ((p.mods.alibi != nullptr || p.mods.alibi_slopes != nullptr) ? 2 : 0);
  const bool drop_u8 = p.mods.drop != nullptr && p.mods.drop_dtype == 2 /*U8*/ && p.S_k % 16 == 0 &&
                       (reinterpret_cast<uintptr_t>(p.mods.drop) & 15u) == 0;
  const int drop = p.mods.drop_philox != 0 ? 1 : (p.mods.drop != nullptr ? (drop_u8 ? 3 : 2) : 0);
  // head_dim 128 has every combination; the other two widths have "no mask, no alibi" and "both may be present"
  if (dpad != 128 && mods != 0) mods = 3;
  void (*kern)(const FwdParams) = nullptr;
#define ACCT_FWD_DROP(DP, BF, M)                                                                           \
  (drop == 0 ? fa_fwd_kernel<DP, BF, M, 0> : drop == 1 ? fa_fwd_kernel<DP, BF, M, 1>                       \
   : drop == 2 ? fa_fwd_kernel<DP, BF, M, 2> : fa_fwd_kernel<DP, BF, M, 3>)
#define ACCT_FWD_BF(DP, M) (bf16 ? ACCT_FWD_DROP(DP, true, M) : ACCT_FWD_DROP(DP, false, M))
  if (dpad == 128) {
    kern = mods == 0 ? ACCT_FWD_BF(128, 0) : mods == 1 ? ACCT_FWD_BF(128, 1) : mods == 2 ? ACCT_FWD_BF(128, 2) : ACCT_FWD_BF(128, 3);
  } else if (dpad == 64) {
    kern = mods == 0 ? ACCT_FWD_BF(64, 0) : ACCT_FWD_BF(64, 3);
  } else {
    kern = mods == 0 ? ACCT_FWD_BF(256, 0) : ACCT_FWD_BF(256, 3);
  }
#undef ACCT_FWD_BF
#undef ACCT_FWD_DROP
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  if (e != cudaSuccess) return e;
  kern<<<grid, kFwdThreads, smem, stream>>>(pp);
  return cudaGetLastError();
}

}  // namespace acct
