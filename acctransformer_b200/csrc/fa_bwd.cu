// FlashAttention-2 backward for sm_100a.
//
// A work item is one 128-row K/V tile of one (batch, head) slice together with the Q tiles that touch
// it; dK and dV accumulate in tensor memory for the whole walk, dQ tiles are added into an fp32
// global accumulator by TMA reduce.  The kernel is persistent: one CTA per SM takes work items from a
// global counter, heaviest tiles first (decode_item), and requests the next item's K and V while the
// current item's dK / dV are being written out.  Scores are recomputed TRANSPOSED (rows = keys, columns =
// queries) so that P^T and dS^T come out in the layout the dV / dK products need:
//   S^T  = K_j Q_i^T          (tcgen05, both operands K-major from shared memory)
//   dP^T = V_j dO_i^T
//   P^T  = exp2(S^T*scale*log2e - L_i*log2e);  dS^T = P^T * (dP^T * M - D_i)        (registers)
//   dK  += dS^T Q_i           (A = dS^T from tensor memory, written over dP^T; B = Q_i, MN-major)
//   dQ_i = dS K_j             (A = the same dS^T tile read MN-major; B = K_j, MN-major) -> over dP^T
//   dV  += (P^T*M) dO_i       (A from tensor memory, written over S^T; B = dO_i, MN-major)
// Warp roles (four warpgroups, registers re-split between them with setmaxnreg): warps 0-7 compute
// (thread = one key row x one half of the query columns), warps 8-11 drain dQ (thread = one query
// row), warp 12 = TMA producer (K/V once, Q in a two-stage ring, dO single-buffered), warp 13 = MMA
// issuer.  Tensor memory:
// S^T/P^T | dP^T/dQ | dK | dV, 128 columns each.  Per Q tile n the tensor pipe runs
// dP^T(n) | dV(n), S^T(n+1) | dK(n), dQ(n): dP^T starts as soon as the previous dQ has been pulled
// out of its columns, dV as soon as P^T is written (the compute warps go on to dS^T meanwhile), S^T
// of the next tile right behind it.  The compute warps never wait for dQ: the drain warpgroup takes
// it through a staging area in shared memory into the fp32 accumulator with TMA reduce-add.
// At the end of an item 16-bit dK and dV leave through shared memory and TMA stores, dK by the compute
// warps (through the dS^T tile) and dV by the drain warps (through their staging area) at the same
// time; fp32 gradients are stored directly.  The producer hands the items to the other roles decoded,
// through a two-slot mailbox, one step before the current item ends.
//
// Follows the reference's backward (train/acctransformer/flash_attention/ops/flash_attention/
// flash_attention_bwd.py:259-415): K/V tile outer, Q tile inner, P recomputed from L, D = rowsum(dO*O)
// (:138-159, here computed once by a separate kernel instead of per tile pair), dS with the
// un-dropped P (:161-181), fp32 accumulation of dQ/dK/dV (:183-257).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "fa_common.cuh"
#include "fa_kernels.cuh"
#include "fa_bwd_helpers.cuh"
#include "ptx.cuh"

namespace acct {

namespace {

constexpr int kBwdThreads = 512;        // four warpgroups: compute x2, drain, control
constexpr int kComputeThreads = 256;
constexpr int kDrainWarp0 = 8;
constexpr int kProducerWarp = 12;
constexpr int kMmaWarp = 13;
constexpr int kStages = 2;              // Q stages (dO has one)
constexpr int kBwdUnitGroup = 8;        // (batch, head) slices whose thread blocks are interleaved, heaviest tiles first
// Register budget per thread after the warpgroups re-split the register file (512 x 128 at launch):
// 256 x 152 + 128 x 152 + 128 x 56 = 65536.
constexpr int kRegsCompute = 152, kRegsDrain = 152, kRegsControl = 56;

// One work item: a 128-row K/V tile of one (batch, key/value head) slice and the Q tiles that touch it.
struct BwdItem {
  int b, h_kv, bh_kv, j;
  int i_lo, n_per, n_iter;     // first Q tile, Q tiles per query head, steps (n_per x query heads of the group)
  int kv_len;
};

struct BwdShared {
  uint64_t item_full[2];         // producer -> everyone: the number of the CTA's next work item is in item[]
  uint64_t item_empty[2];        // everyone -> producer: the slot has been read by the MMA, drain and compute threads
  uint64_t kv_full;
  uint64_t kv_empty;             // MMA -> producer: every product of the work item has finished, K and V may be replaced
  uint64_t acc_free;             // compute, drain -> MMA: dK and dV of the work item have been read out of tensor memory
  uint64_t q_full[kStages];
  uint64_t q_empty[kStages];     // drain (on dq_full) -> producer: the products reading this Q stage have finished
  uint64_t do_full;              // producer (dO of step n has landed) + drain (dQ of step n-1 is in registers, the dP^T
                                 // columns are free again) -> MMA: dP^T of step n may be issued.  One barrier for both:
                                 // every wait costs the issuing thread time in which the tensor pipe may idle
  uint64_t do_empty;             // MMA -> producer: the dV product reading dO has finished
  uint64_t st_full, dp_full;     // MMA -> compute: S^T / dP^T are in tensor memory
  uint64_t p_ready;              // compute -> MMA: P^T is in tensor memory
  uint64_t ds_ready;             // compute -> MMA: dS^T is in shared memory
  uint64_t dq_full;              // MMA -> drain: dV, dK and dQ products of this Q tile have finished
  uint64_t stats_ready;          // compute -> compute: lse2 / delta of this Q tile are in shared memory
  uint32_t tmem_base;
  volatile uint32_t abort_flag;
  int item[2];
  BwdItem decoded[2];            // the same two items, decoded by the producer (see next_item)
  alignas(16) float lse2[2][kTile];   // L * log2(e) per query of the tile (+inf for rows past S_q); read as float4
  alignas(16) float delta[2][kTile];
};

// P = exp2(s*scale + bias - L) for 32 consecutive queries of one key row; `bias` is -inf for key rows
// that do not exist, L is +inf for query rows that do not exist: both give exactly 0.
template <bool DIAG>
__device__ __forceinline__ void p_fast(const uint32_t (&s)[32], const float* lse2c, float scale_log2, float bias,
                                       int kv_idx, int q0, float (&pr)[32]) {
#pragma unroll
  for (int e4 = 0; e4 < 8; ++e4) {
    const float4 L = *reinterpret_cast<const float4*>(lse2c + 4 * e4);
    const float l[4] = {L.x, L.y, L.z, L.w};
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int e = 4 * e4 + u;
      float v = ex2(fmaf(__uint_as_float(s[e]), scale_log2, bias) - l[u]);
      if (DIAG) v = (kv_idx > q0 + e) ? 0.f : v;
      pr[e] = v;
    }
  }
}

// Pass over one half (64 query columns) of a thread's S^T row in tensor memory, for the tiles that need it: the
// mask term is added in score units (the common code multiplies by the scale afterwards) and (key, query) pairs
// outside the query's TriangleAttention row group become -inf.  Loads use clamped (always valid) addresses so
// that they carry no branches: what they fetch for a key or query that does not exist meets a P that is exactly 0
// there (bias = -inf / L = +inf).  Kept out of line: inlined, its registers disturb the allocation of the common
// path of every tile, taken or not.
__device__ __noinline__ void mask_prepass(const ScoreMods& mods, uint32_t t_st, int hf, int q_base, int kv_idx, int r,
                                          int b, int S_q, int S_k, float scale, bool use_mask, bool tri_partial) {
  const int kv_c = min(kv_idx, S_k - 1);
  const float mask_unit = -10000.0f / scale;
  // sixteen queries at a time: the lighter this function is in registers, the less its call site costs the tiles
  // that never come here
#pragma unroll 1
  for (int piece = 0; piece < 4; ++piece) {
    const int col = hf * 64 + piece * 16;           // first of the 16 S^T columns (queries) of this piece
    const int q0 = q_base + col;
    uint32_t sc[16];
    tmem_ld16(t_st + col, sc);
    uint32_t mraw[8];
    if (use_mask) {
      if (mods.mask_kind == 1)
        load_col_raw<8>(mods.mask, mods.mask_dtype, static_cast<int64_t>(mods.mask_batch > 1 ? b : 0) * S_q, q0, S_q - 1,
                        S_k, kv_c, mraw);
      else   // the 128 x 128 tile: element (query in tile, key in tile)
        load_col_raw<8>(mods.mask, mods.mask_dtype, 0, col, kTile - 1, kTile, r, mraw);
    }
    tmem_wait_ld();
    if (use_mask) {
#pragma unroll
      for (int e = 0; e < 16; ++e)
        sc[e] = __float_as_uint(fmaf(col_value(mraw[e >> 1], mods.mask_dtype, e & 1), mask_unit, __uint_as_float(sc[e])));
    }
    if (tri_partial) {
      // first key that does not exist for query q0 + e: end of its row group
#pragma unroll
      for (int e = 0; e < 16; ++e) {
        const int lim = ((q0 + e) / mods.tri_block + 1) * mods.tri_block;
        sc[e] = kv_idx >= lim ? __float_as_uint(kNegInf) : sc[e];
      }
    }
    tmem_st16(t_st + col, sc);
  }
  tmem_wait_st();
}


// Work item number -> item.  Items are numbered so that, inside a group of kBwdUnitGroup slices, the heaviest
// K/V tiles of ALL slices come first (under a causal mask tile 0 walks every Q tile, the last tile one): the CTAs take
// items in that order, so the SMs finish together, which matters most when a slice has few tiles, while the Q, dO
// and dQ tiles that the running CTAs share stay within L2.
// With an ordered dQ reduction the CTA of tile j waits for the CTAs of the later tiles (j' > j) that touch the same Q
// tile, so those must never be started after it: tiles are then handed out in descending order, and every wait
// points at an item that was taken earlier, i.e. is being worked on or finished, however many tiles a slice has.
__device__ __forceinline__ BwdItem decode_item(const BwdParams& p, int w) {
  const ScoreMods& mods = p.mods;
  BwdItem it;
  const int n_kv = p.N / p.kv_group;
  const int n_j = (p.S_k + kTile - 1) / kTile;
  const int n_units = p.B * n_kv;
  const int per_group = n_j * kBwdUnitGroup;
  const int grp = w / per_group, within = w % per_group;
  const int g_units = min(kBwdUnitGroup, n_units - grp * kBwdUnitGroup);
  const int jj = within / g_units;
  it.bh_kv = grp * kBwdUnitGroup + within % g_units;
  it.j = p.dq_order != nullptr ? n_j - 1 - jj : jj;
  it.b = it.bh_kv / n_kv;
  it.h_kv = it.bh_kv % n_kv;
  it.kv_len = p.S_k;
  if (mods.seq_lens != nullptr) it.kv_len = min(p.S_k, max(0, mods.seq_lens[it.b]));
  // Q tiles i that need K/V tile j:  j - next <= i <= j + prev, i >= j under the causal triangle
  int i_lo = 0, i_hi = (p.S_q + kTile - 1) / kTile - 1;
  if (mods.next_block_num < 65536) i_lo = max(i_lo, it.j - mods.next_block_num);
  if (mods.prev_block_num < 65536) i_hi = min(i_hi, it.j + mods.prev_block_num);
  if (mods.causal) i_lo = max(i_lo, it.j);
  if (mods.tri_block > 0) i_lo = max(i_lo, (((it.j * kTile) / mods.tri_block) * mods.tri_block) / kTile);
  if (it.j * kTile >= it.kv_len) i_hi = i_lo - 1;
  it.i_lo = i_lo;
  it.n_per = max(0, i_hi - i_lo + 1);
  it.n_iter = it.n_per * p.kv_group;
  return it;
}

// Every role learns its CTA's k-th work item here: its number and, decoded by the producer (the integer divisions of
// decode_item are not repeated by 400 threads between two items), what it stands for.  This wait does not look at the
// abort flag: the producer's own waits are all bounded, so it always gets to publish the next item (after a failure:
// the end marker), and all threads of a role must see the SAME item -- their loops, named barriers and
// warp-collective instructions depend on it.  Its own limit is generous and is not expected to be reached.
__device__ __forceinline__ int next_item(BwdShared& sh, int k, volatile uint32_t* abort_flag, unsigned int* status, BwdItem& out) {
  uint64_t* bar = &sh.item_full[k & 1];
  const uint32_t parity = (k >> 1) & 1;
  uint32_t polls = 0;
  while (!mbar_try_wait(bar, parity)) {
    if (++polls >= (kWaitPollLimit << 2)) {
      *abort_flag = 1u;
      atomicMax(status, DEV_TIMEOUT_SYNC);
      break;
    }
  }
  const int w = sh.item[k & 1];
  out = sh.decoded[k & 1];                // (stale behind the end marker: never looked at)
  mbar_arrive(&sh.item_empty[k & 1]);     // the slot may be reused once every consumer has read it
  return w;
}

}  // namespace

// MASKED = a mask tensor or TriangleAttention row groups may be present: tiles that need them get a pass over S^T
// in tensor memory before the common code.  DROP = 0 no dropout, 1 in-kernel generator, 2 dropout mask tensor of any
// type, 3 uint8 {0,1} mask tensor read as keep bits (4-byte aligned, S_k a multiple of 4).  The
// plain instantiation carries none of that code, so its register allocation is not disturbed by it.
template <int DPAD, bool BF16, bool MASKED, int DROP>
__global__ void __launch_bounds__(kBwdThreads, 1) fa_bwd_kernel(const __grid_constant__ BwdParams p) {
  constexpr int NB = DPAD / 64;
  constexpr uint32_t kTileBytes = NB * 16384u;   // 128 rows x DPAD 16-bit elements
  constexpr uint32_t kColST = 0, kColDP = 128, kColDK = 256, kColDV = 384;
  constexpr int kChunks = DPAD / 32;             // 32-column fp32 chunks of a dQ / dK / dV row

  // All shared memory is dynamic so that the tiles start at the (1024-byte aligned) base of the CTA's window.
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* sK = smem;
  uint8_t* sV = sK + kTileBytes;
  uint8_t* sQ = sV + kTileBytes;                   // kStages tiles
  uint8_t* sDO = sQ + kStages * kTileBytes;        // one tile
  uint8_t* sDS = sDO + kTileBytes;                 // dS^T: 2 blocks of 128 key rows x 64 queries
  uint8_t* sStage = sDS + 32768;                   // dQ staging: 2 chunks of 128 rows x 32 fp32
  BwdShared& sh = *reinterpret_cast<BwdShared*>(sStage + 32768);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  // The CTA is persistent: it takes work items (decode_item) one after the other from a global counter until none is
  // left.  Its tensor memory, barriers and warp roles live for the whole kernel; the K/V tiles of the next item are
  // requested as soon as the last product of the current one has finished, so that their latency falls under the
  // current item's dK / dV write-out.  `g0` counts the steps of the items done so far: every barrier that completes
  // once per step keeps one running phase across items.  `live` counts the items done so far that had any step.
  const ScoreMods& mods = p.mods;
  const int total_items = ((p.S_k + kTile - 1) / kTile) * p.B * (p.N / p.kv_group);

  if ((smem_u32(smem) & 1023u) != 0u) {          // the swizzled tiles need a 1024-byte aligned base
    if (tid == 0) atomicMax(p.status, DEV_BAD_SMEM_BASE);
    return;
  }

  if (tid == 0) {
    mbar_init(&sh.item_full[0], 1);
    mbar_init(&sh.item_full[1], 1);
    mbar_init(&sh.item_empty[0], 1 + kTile + kComputeThreads);
    mbar_init(&sh.item_empty[1], 1 + kTile + kComputeThreads);
    mbar_init(&sh.kv_full, 1);
    mbar_init(&sh.kv_empty, 1);
    mbar_init(&sh.acc_free, kComputeThreads + kTile);   // dK is written out by the compute warps, dV by the drain warps
    for (int s = 0; s < kStages; ++s) { mbar_init(&sh.q_full[s], 1); mbar_init(&sh.q_empty[s], 1); }
    mbar_init(&sh.do_full, 1 + kTile);
    mbar_init(&sh.do_empty, 1);
    mbar_init(&sh.st_full, 1);
    mbar_init(&sh.dp_full, 1);
    mbar_init(&sh.p_ready, kComputeThreads);
    mbar_init(&sh.ds_ready, kComputeThreads);
    mbar_init(&sh.dq_full, 1);
    mbar_init(&sh.stats_ready, kTile);
    sh.abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == kProducerWarp) { tmem_alloc(&sh.tmem_base, 512); tmem_relinquish(); }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = sh.tmem_base;
  volatile uint32_t* abort_flag = &sh.abort_flag;

  if (warp >= kProducerWarp) {
    // ------------------------------------------------------------------ control warpgroup
    reg_dealloc<kRegsControl>();
    if (warp == kProducerWarp) {
      // ---------------------------------------------------------------- TMA producer (and keeper of the work list)
      if (lane == 0) {
        prefetch_tmap(&p.map_q); prefetch_tmap(&p.map_k); prefetch_tmap(&p.map_v); prefetch_tmap(&p.map_do);
        prefetch_tmap(&p.map_dq);
        int g0 = 0, live = 0;
        // The item after the current one is claimed and published while the loads of the current item's last step but
        // one go out: late enough that no CTA sits on an unstarted item for long (that unbalances the end of the
        // kernel when a CTA has only a handful of items), early enough that the other roles know it before they
        // finish the current item (the compute warps request its first statistics at the end of the last step) and
        // that the counter's latency -- a global atomic next to 148 SMs' reduce traffic -- is not on their path.
        int w_cur = static_cast<int>(atomicAdd(p.work_counter, 1u));
        int w_nxt = total_items;
        auto publish = [&](int slot, int w) {
          sh.item[slot] = w;
          if (w < total_items) sh.decoded[slot] = decode_item(p, w);
          mbar_arrive(&sh.item_full[slot]);      // (release: the stores above are visible to whoever sees the phase)
        };
        publish(0, w_cur);
        for (int k = 0; w_cur < total_items; ++k) {
          const BwdItem it = sh.decoded[k & 1];  // (slot k & 1 is rewritten for item k + 2 at the earliest: next round)
          bool published = false;
          // the next item goes into the other slot once every consumer has read item k-1 out of it; after a failure
          // the end marker, so that every role leaves its loop at the same item
          auto publish_next = [&]() {
            if (k >= 1) mbar_wait(&sh.item_empty[(k + 1) & 1], ((k - 1) >> 1) & 1, abort_flag, p.status, DEV_TIMEOUT_SYNC);
            w_nxt = *abort_flag == 0u ? static_cast<int>(atomicAdd(p.work_counter, 1u)) : total_items;
            publish((k + 1) & 1, w_nxt);
            published = true;
          };
          if (it.n_iter > 0 && *abort_flag == 0u) {
            // K and V of the previous item are free once all of its products have finished
            if (live > 0) mbar_wait(&sh.kv_empty, (live - 1) & 1, abort_flag, p.status, DEV_TIMEOUT_SYNC);
            mbar_expect_tx(&sh.kv_full, 2 * kTileBytes);
            for (int nb = 0; nb < NB; ++nb) tma_load_4d(sK + nb * 16384, &p.map_k, &sh.kv_full, nb * 64, it.j * kTile, it.h_kv, it.b);
            for (int nb = 0; nb < NB; ++nb) tma_load_4d(sV + nb * 16384, &p.map_v, &sh.kv_full, nb * 64, it.j * kTile, it.h_kv, it.b);
            for (int n = 0; n < it.n_iter; ++n) {
              const int i = it.i_lo + n % it.n_per, h = it.h_kv * p.kv_group + n / it.n_per;
              const int gn = g0 + n;
              const int st = gn % kStages;
              // the Q stage is free once the dK product of two tiles ago has finished
              if (gn >= kStages) mbar_wait(&sh.q_empty[st], ((gn / kStages) - 1) & 1, abort_flag, p.status, DEV_TIMEOUT_SYNC);
              mbar_expect_tx(&sh.q_full[st], kTileBytes);
              for (int nb = 0; nb < NB; ++nb)
                tma_load_4d(sQ + st * kTileBytes + nb * 16384, &p.map_q, &sh.q_full[st], nb * 64, i * kTile, h, it.b);
              // dO has one buffer: it is free once the dV product of the previous tile has finished, and is not
              // needed again before the dP^T product of this tile, most of an iteration later
              if (gn >= 1) mbar_wait(&sh.do_empty, (gn - 1) & 1, abort_flag, p.status, DEV_TIMEOUT_SYNC);
              mbar_expect_tx(&sh.do_full, kTileBytes);
              for (int nb = 0; nb < NB; ++nb)
                tma_load_4d(sDO + nb * 16384, &p.map_do, &sh.do_full, nb * 64, i * kTile, h, it.b);
              if (n == (it.n_iter >= 2 ? it.n_iter - 2 : 0)) publish_next();
            }
            g0 += it.n_iter;
            ++live;
          }
          if (!published) publish_next();
          w_cur = w_nxt;
        }
      }
    } else if (warp == kMmaWarp) {
      // ---------------------------------------------------------------- MMA issuer
      // Tensor-pipe order per Q tile n:  dP^T(n) | dV(n), S^T(n+1) | dK(n), dQ(n).
      if (lane == 0) {
        const uint32_t idesc_s = make_idesc(BF16, 128, 128, false, false);     // S^T, dP^T
        const uint32_t idesc_kv = make_idesc(BF16, 128, DPAD, false, true);    // dV, dK
        const uint32_t idesc_dq = make_idesc(BF16, 128, DPAD, true, true);     // dQ
        const uint64_t kmajor = make_sdesc_base(16, 1024);
        const uint64_t mnmajor = make_sdesc_base(16384, 1024);
        // Descriptors as (low word, high word): the low word holds the start address in 16-byte units, so stepping
        // along a tile is one 32-bit add and the issuing thread spends next to nothing between two MMAs.
        const uint32_t k_hi = static_cast<uint32_t>(kmajor >> 32), k_lo = static_cast<uint32_t>(kmajor);
        const uint32_t mn_hi = static_cast<uint32_t>(mnmajor >> 32), mn_lo = static_cast<uint32_t>(mnmajor);
        auto lo_of = [](uint32_t base_lo, const uint8_t* ptr) { return base_lo | ((smem_u32(ptr) >> 4) & 0x3fffu); };
        const uint32_t kK = lo_of(k_lo, sK), kV = lo_of(k_lo, sV), kDO = lo_of(k_lo, sDO), kQ0 = lo_of(k_lo, sQ);
        const uint32_t mK = lo_of(mn_lo, sK), mDS = lo_of(mn_lo, sDS), mDO = lo_of(mn_lo, sDO), mQ0 = lo_of(mn_lo, sQ);
        constexpr uint32_t kTileUnits = kTileBytes >> 4;

        auto issue_st = [&](int st) {   // S^T = K Q^T
          const uint32_t kQ = kQ0 + st * kTileUnits;
#pragma unroll
          for (int kk = 0; kk < DPAD / 16; ++kk) {
            const uint32_t off = (kk >> 2) * 1024u + (kk & 3) * 2u;   // 16-byte units
            umma_ss_lohi(tmem + kColST, kK + off, k_hi, kQ + off, k_hi, idesc_s, kk > 0);
          }
          umma_commit(&sh.st_full);
        };

        int g0 = 0, live = 0;
        for (int k = 0;; ++k) {
          BwdItem it;
          const int w = next_item(sh, k, abort_flag, p.status, it);
          if (w >= total_items) break;
          if (it.n_iter == 0) continue;
          const int n_iter = it.n_iter;
          mbar_wait(&sh.kv_full, live & 1, abort_flag, p.status, DEV_TIMEOUT_TMA);
          mbar_wait(&sh.q_full[g0 % kStages], (g0 / kStages) & 1, abort_flag, p.status, DEV_TIMEOUT_TMA);
          tc_fence_after_sync();
          issue_st(g0 % kStages);
          for (int n = 0; n < n_iter; ++n) {
            const int gn = g0 + n;
            const int st = gn % kStages;
            const int stn = (gn + 1) % kStages;
            const uint32_t mQ = mQ0 + st * kTileUnits;
            // dP^T = V dO^T as early as possible: it only needs dO and the previous dQ out of its columns
            mbar_wait(&sh.do_full, gn & 1, abort_flag, p.status, DEV_TIMEOUT_TMA);
            tc_fence_after_sync();
#pragma unroll
            for (int kk = 0; kk < DPAD / 16; ++kk) {
              const uint32_t off = (kk >> 2) * 1024u + (kk & 3) * 2u;
              umma_ss_lohi(tmem + kColDP, kV + off, k_hi, kDO + off, k_hi, idesc_s, kk > 0);
            }
            umma_commit(&sh.dp_full);
            // dV += P^T dO as soon as P^T is in tensor memory (the compute warps go on to dS meanwhile);
            // P^T of query columns [64h, 64h+64) sits in S^T columns [64h, 64h+32)
            mbar_wait(&sh.p_ready, gn & 1, abort_flag, p.status, DEV_TIMEOUT_SYNC);
            // the first products of an item overwrite dK and dV: the previous item's must have been read out
            if (n == 0 && live > 0) mbar_wait(&sh.acc_free, (live - 1) & 1, abort_flag, p.status, DEV_TIMEOUT_SYNC);
            tc_fence_after_sync();
#pragma unroll
            for (int kk = 0; kk < kTile / 16; ++kk)
              umma_ts_lohi(tmem + kColDV, tmem + kColST + (kk >> 2) * 64 + (kk & 3) * 8, mDO + kk * 128u, mn_hi,
                           idesc_kv, n > 0 || kk > 0);
            umma_commit(&sh.do_empty);
            // S^T of the next Q tile right behind it (the tensor pipe runs in order, so P^T has been consumed)
            if (n + 1 < n_iter) {
              mbar_wait(&sh.q_full[stn], ((gn + 1) / kStages) & 1, abort_flag, p.status, DEV_TIMEOUT_TMA);
              tc_fence_after_sync();
              issue_st(stn);
            }
            // dK += dS^T Q and dQ = dS K once dS^T is in shared memory
            mbar_wait(&sh.ds_ready, gn & 1, abort_flag, p.status, DEV_TIMEOUT_SYNC);
            tc_fence_after_sync();
#pragma unroll
            for (int kk = 0; kk < kTile / 16; ++kk)   // dK: A = dS^T packed over the dP^T columns, like P^T over S^T
              umma_ts_lohi(tmem + kColDK, tmem + kColDP + (kk >> 2) * 64 + (kk & 3) * 8, mQ + kk * 128u, mn_hi,
                           idesc_kv, n > 0 || kk > 0);
#pragma unroll
            for (int kk = 0; kk < kTile / 16; ++kk)
              umma_ss_lohi(tmem + kColDP, mDS + kk * 128u, mn_hi, mK + kk * 128u, mn_hi, idesc_dq, kk > 0);
            umma_commit(&sh.dq_full);     // (the drain passes it on to the producer as q_empty[st]: one commit less here)
          }
          umma_commit(&sh.kv_empty);
          g0 += n_iter;
          ++live;
        }
      }
    }
  } else if (warp >= kDrainWarp0) {
    // ------------------------------------------------------------------ drain warpgroup: dQ_i out of tensor
    // memory, through a 32 KB swizzled staging area (two 32-column chunks at a time), into the fp32
    // accumulator by TMA reduce-add.  Thread t owns query row t of the tile.
    reg_alloc<kRegsDrain>();
    const int r = tid - kDrainWarp0 * 32;
    const uint32_t t_dq = tmem + (static_cast<uint32_t>((warp & 3) * 32) << 16) + kColDP;
    const bool elected = (r == 0);
    mbar_arrive(&sh.do_full);              // the first step of the kernel has no dQ before it to wait for
    int g0 = 0;
    for (int k = 0;; ++k) {
    BwdItem it;
    const int w = next_item(sh, k, abort_flag, p.status, it);
    if (w >= total_items) break;
    const int b = it.b, j = it.j, kv_len = it.kv_len;
    auto head_of = [&](int n) { return it.h_kv * p.kv_group + n / max(it.n_per, 1); };
    auto tile_of = [&](int n) { return it.i_lo + n % max(it.n_per, 1); };
    for (int n = 0; n < it.n_iter; ++n) {
      const int q_base = tile_of(n) * kTile;
      const int h = head_of(n);
      const int bh = b * p.N + h;
      mbar_wait(&sh.dq_full, (g0 + n) & 1, abort_flag, p.status, DEV_TIMEOUT_MMA);
      tc_fence_after_sync();
      // every product of this step has finished: its Q stage may be refilled (told to the producer from here, so that
      // the MMA-issuing thread, which issues nothing while it commits, has one commit less per step)
      if (elected) mbar_arrive(&sh.q_empty[(g0 + n) % kStages]);
      uint32_t dq[kChunks][32];
#pragma unroll
      for (int c = 0; c < kChunks; ++c) tmem_ld32(t_dq + c * 32, dq[c]);
      tmem_wait_ld();
      tc_fence_before_sync();
      mbar_arrive(&sh.do_full);          // (counts towards the NEXT step's phase: this step's has completed)
#pragma unroll
      for (int rd = 0; rd < kChunks / 2; ++rd) {
        // the staging area is free once the previous round's reduce has read it
        if (elected) tma_store_wait_read();
        named_barrier(3, kTile);
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
#pragma unroll
          for (int g = 0; g < 8; ++g)
            *reinterpret_cast<float4*>(sStage + cc * 16384u + swz128(r, g)) =
                make_float4(__uint_as_float(dq[rd * 2 + cc][4 * g]) * p.scale, __uint_as_float(dq[rd * 2 + cc][4 * g + 1]) * p.scale,
                            __uint_as_float(dq[rd * 2 + cc][4 * g + 2]) * p.scale, __uint_as_float(dq[rd * 2 + cc][4 * g + 3]) * p.scale);
        }
        fence_proxy_async_smem();
        named_barrier(3, kTile);
        if (elected) {
          if (p.dq_order != nullptr && rd == 0) {
            // Fixed summation order for dQ (opt-in): the K/V tiles that touch Q tile i add their parts in
            // descending tile order, which is the order in which they naturally reach tile i under a causal
            // mask.  j_top is the last K/V tile that touches tile i: it inverts the Q-tile range above.
            const int i = tile_of(n);
            int j_top = (kv_len + kTile - 1) / kTile - 1;
            if (mods.next_block_num < 65536) j_top = min(j_top, i + mods.next_block_num);
            if (mods.causal) j_top = min(j_top, i);
            if (mods.tri_block > 0) j_top = min(j_top, (((i * kTile + kTile - 1) / mods.tri_block + 1) * mods.tri_block - 1) / kTile);
            const unsigned int my_turn = static_cast<unsigned int>(j_top - j);
            const unsigned int* slot = p.dq_order + static_cast<int64_t>(bh) * ((p.S_q + kTile - 1) / kTile) + i;
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
            const int c = rd * 2 + cc;
            if (c * 32 < p.D) tma_reduce_add_4d(&p.map_dq, sStage + cc * 16384u, c * 32, q_base, h, b);
          }
          tma_store_commit();
          if (p.dq_order != nullptr && rd == kChunks / 2 - 1) {
            // pass the turn on once this tile's additions have been performed
            tma_store_wait_all();
            unsigned int* slot = p.dq_order + static_cast<int64_t>(bh) * ((p.S_q + kTile - 1) / kTile) + tile_of(n);
            asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(slot) : "memory");
          }
        }
      }
    }
    // dV of the item (16-bit gradients): out of tensor memory once the item's last products have finished (the last
    // dq_full above), through this warpgroup's staging area and one TMA store, while the compute warps write dK
    // through theirs.  Thread t owns key row t here.
    if (!p.grads_f32) {
      if (elected) tma_store_wait_read();        // the item's last dQ round has been read out of the staging area
      named_barrier(3, kTile);
      const uint32_t t_dv = tmem + (static_cast<uint32_t>((warp & 3) * 32) << 16) + kColDV;
      // (one 32-column chunk at a time, not unrolled: this runs once per item, and the drain's per-step code must keep
      // its place in the instruction cache)
#pragma unroll 1
      for (int c = 0; c < kChunks; ++c) {
        uint32_t dv[32];
        if (it.n_iter > 0) { tmem_ld32(t_dv + c * 32, dv); tmem_wait_ld(); }
        else {
#pragma unroll
          for (int e = 0; e < 32; ++e) dv[e] = 0u;
        }
        uint8_t* blk = sStage + (c >> 1) * 16384u;
#pragma unroll
        for (int g = 0; g < 4; ++g)
          *reinterpret_cast<uint4*>(blk + swz128(r, (c & 1) * 4 + g)) =
              make_uint4(pack2<BF16>(__uint_as_float(dv[8 * g]), __uint_as_float(dv[8 * g + 1])),
                         pack2<BF16>(__uint_as_float(dv[8 * g + 2]), __uint_as_float(dv[8 * g + 3])),
                         pack2<BF16>(__uint_as_float(dv[8 * g + 4]), __uint_as_float(dv[8 * g + 5])),
                         pack2<BF16>(__uint_as_float(dv[8 * g + 6]), __uint_as_float(dv[8 * g + 7])));
      }
      tc_fence_before_sync();
      if (it.n_iter > 0) mbar_arrive(&sh.acc_free);
      fence_proxy_async_smem();
      named_barrier(3, kTile);
      if (elected) {
        for (int nb = 0; nb < NB; ++nb)
          if (nb * 64 < p.D) tma_store_4d(&p.map_dv, sStage + nb * 16384, nb * 64, j * kTile, it.h_kv, b);
        tma_store_commit();
      }
    } else if (it.n_iter > 0) {
      mbar_arrive(&sh.acc_free);                  // fp32 gradients: the compute warps write both tiles out
    }
    g0 += it.n_iter;
    }
    if (elected) tma_store_wait_all();
  } else {
    // ------------------------------------------------------------------ compute warps
    reg_alloc<kRegsCompute>();
    const int hf = warp >> 2;                            // which half of the query columns / of head_dim
    const int r = (warp & 3) * 32 + lane;                // key row inside the tile (and dQ row when draining)
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t t_st = tmem + lane_base + kColST;
    const uint32_t t_dp = tmem + lane_base + kColDP;
    uint8_t* my_ds = sDS + hf * 16384u;                  // this half's dS^T block
    int g0 = 0;
    bool ds_stage_busy = false;     // a dK store may still be reading the dS^T tile (uniform over the compute threads)
    // What an item needs from global memory before its first step -- the statistics of its first Q tile and the key
    // row's alibi term -- is requested before the write-out of the item BEFORE it and left raw until then, so that
    // the latency of those loads does not sit between two items (it did: the compute warps came out of the
    // write-out, loaded, and only then looked at an S^T that had been waiting for them).
    float pre_lse = 0.f, pre_dlt = 0.f;
    uint32_t pre_bias = 0u;
    auto request_first = [&](const BwdItem& t) {
      if (t.n_iter <= 0) return;
      const int h0 = t.h_kv * p.kv_group;
      if (hf == 0) {
        const int64_t idx = (static_cast<int64_t>(t.b) * p.N + h0) * p.S_q + min(t.i_lo * kTile + r, p.S_q - 1);
        pre_lse = p.lse[idx];
        pre_dlt = p.delta[idx];
      }
      const int kv = t.j * kTile + r;
      if (kv < t.kv_len) {
        if (mods.alibi != nullptr)
          pre_bias = reinterpret_cast<const uint16_t*>(mods.alibi)[(static_cast<int64_t>(t.b) * p.N + h0) * p.S_k + kv];
        else if (mods.alibi_slopes != nullptr)
          pre_bias = __float_as_uint(mods.alibi_slopes[h0]);
      }
    };
    BwdItem it_next;
    int item_no = next_item(sh, 0, abort_flag, p.status, it_next);
    if (item_no < total_items) request_first(it_next);
    for (int k = 0; item_no < total_items; ++k) {
    const BwdItem it = it_next;
    int next_no = total_items;
    bool next_known = false;
    const int b = it.b, j = it.j, kv_len = it.kv_len, i_lo = it.i_lo, n_per = it.n_per, n_iter = it.n_iter;
    const int bh_kv = it.bh_kv;
    auto head_of = [&](int n) { return it.h_kv * p.kv_group + n / max(n_per, 1); };
    auto tile_of = [&](int n) { return i_lo + n % max(n_per, 1); };
    const int kv_idx = j * kTile + r;
    const bool kv_ok = kv_idx < kv_len;
    // alibi term of this key row in log2 units for query head h; -inf removes a key row that does not exist
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
    float bias_first = kNegInf;          // bias_of(head_of(0)), from the value requested ahead
    if (kv_ok) {
      bias_first = 0.f;
      if (mods.alibi != nullptr)
        bias_first = (BF16 ? __uint_as_float(pre_bias << 16) : __half2float(__ushort_as_half(static_cast<unsigned short>(pre_bias)))) * kLog2e;
      else if (mods.alibi_slopes != nullptr)
        bias_first = __uint_as_float(pre_bias) * static_cast<float>(kv_idx) * kLog2e;
    }

    // statistics of the first Q tile
    // The next tile's statistics are fetched one tile ahead and kept RAW until they are parked: any arithmetic on a
    // freshly loaded value would stall the warp (in-order issue) for the whole global-memory latency right there.
    float nxt_lse = 0.f, nxt_dlt = 0.f;
    bool nxt_ok = false;
    if (hf == 0 && n_iter > 0) {
      const int q_row = i_lo * kTile + r;
      const bool q_ok = q_row < p.S_q;
      // (buffer g0 & 1 was last read for the step before last, whose dS part every thread finished before the
      // products this thread has since waited for could be issued)
      sh.lse2[g0 & 1][r] = q_ok ? pre_lse * kLog2e : INFINITY;
      sh.delta[g0 & 1][r] = q_ok ? pre_dlt : 0.f;
      mbar_arrive(&sh.stats_ready);
    }

    // Optional per-tile summary of a full mask tensor: the class of tile (i, j) is fetched one tile ahead.
    const uint8_t* tile_class = nullptr;
    const int tiles_k = (p.S_k + kTile - 1) / kTile;
    if constexpr (MASKED) if (mods.mask_kind == 1 && mods.mask_tiles != nullptr)
      tile_class = mods.mask_tiles + static_cast<int64_t>(mods.mask_batch > 1 ? b : 0) * ((p.S_q + kTile - 1) / kTile) * tiles_k + j;
    int mask_class = 1, mask_class_next = 1;
    if (tile_class != nullptr && n_iter > 0) mask_class_next = tile_class[static_cast<int64_t>(tile_of(0)) * tiles_k];

    for (int n = 0; n < n_iter; ++n) {
      const int i = tile_of(n);
      const int q_base = i * kTile;
      const int bh = b * p.N + head_of(n);
      const int gn = g0 + n;                                    // running step number: the phase of the per-step barriers
      if (n % max(n_per, 1) == 0) bias = n == 0 ? bias_first : bias_of(head_of(n));   // first tile of a query head
      mask_class = mask_class_next;
      if (tile_class != nullptr && n + 1 < n_iter) mask_class_next = tile_class[static_cast<int64_t>(tile_of(n + 1)) * tiles_k];
      // ---- P part: needs S^T only
      mbar_wait(&sh.st_full, gn & 1, abort_flag, p.status, DEV_TIMEOUT_MMA);
      tc_fence_after_sync();
      // Park this tile's statistics (fetched during the previous tile).  S^T(n) was issued after all 256
      // compute threads arrived at p_ready(n-1), i.e. after they passed the previous stats_ready wait and
      // finished the dS part that read the buffer being overwritten.
      if (hf == 0 && n > 0) {
        sh.lse2[gn & 1][r] = nxt_ok ? nxt_lse * kLog2e : INFINITY;
        sh.delta[gn & 1][r] = nxt_ok ? nxt_dlt : 0.f;
        mbar_arrive(&sh.stats_ready);
      }
      // fetch the next tile's statistics now
      if (hf == 0 && n + 1 < n_iter) {
        const int q_row = tile_of(n + 1) * kTile + r;
        nxt_ok = q_row < p.S_q;
        const int64_t idx = (static_cast<int64_t>(b) * p.N + head_of(n + 1)) * p.S_q + min(q_row, p.S_q - 1);
        nxt_lse = p.lse[idx];      // (clamped, always valid address: no branch around the loads)
        nxt_dlt = p.delta[idx];
      }
      mbar_wait(&sh.stats_ready, gn & 1, abort_flag, p.status, DEV_TIMEOUT_SYNC);
      const float* lse2 = sh.lse2[gn & 1];
      const float* dlt = sh.delta[gn & 1];
      // A mask tile that is all 0 is not read; one that is all 1 adds one constant to every score of the tile,
      // which joins the key row's bias; any other tile is read.
      const bool mask_const = MASKED && mods.mask_kind == 1 && mask_class == 2;
      const bool use_mask = MASKED && ((mods.mask_kind == 1 && mask_class != 0 && !mask_const) || (mods.mask_kind == 2 && i == j));
      const float tile_bias = mask_const ? bias - 10000.0f * kLog2e : bias;
      const bool diag = mods.causal && (q_base < j * kTile + kTile - 1);
      // TriangleAttention row groups: the rows of this Q tile see keys below the end of their group; the smallest
      // such end is that of the tile's first row, and a K/V tile that lies wholly below it needs no per-element test
      const bool tri_partial = MASKED && mods.tri_block > 0 &&
                               (j * kTile + kTile > (q_base / mods.tri_block + 1) * mods.tri_block);

      if constexpr (MASKED) if (use_mask || tri_partial)
        mask_prepass(mods, t_st, hf, q_base, kv_idx, r, b, p.S_q, p.S_k, p.scale, use_mask, tri_partial);

      // P^T (dropped) goes over the first 32 of this half's own 64 S^T columns, which the half has
      // finished reading by then.
      float pr[2][32];
      uint32_t keep_bits[2] = {0xffffffffu, 0xffffffffu};   // in-kernel dropout: bit e = query q0 + e keeps this key
      {
        uint32_t s[2][32];
        tmem_ld32(t_st + (hf * 2) * 32, s[0]);
        tmem_ld32(t_st + (hf * 2 + 1) * 32, s[1]);
        tmem_wait_ld();
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
          const int c = hf * 2 + cc;
          uint32_t draw[16];       // dropout mask tensor: raw values of this chunk's queries, in flight under the exponentials
          if constexpr (DROP == 2)
            load_col32_raw(mods.drop, mods.drop_dtype, static_cast<int64_t>(bh) * p.S_q, q_base + c * 32, p.S_q - 1, p.S_k,
                           min(kv_idx, p.S_k - 1), draw);
          uint32_t raw8[8];        // uint8 mask as keep bits: eight words per lane, likewise in flight
          if constexpr (DROP == 3)
            u8_keep_load(mods.drop, static_cast<int64_t>(bh) * p.S_q, q_base + c * 32, p.S_q - 1, p.S_k, kv_idx - lane, lane, raw8);
          if (diag) p_fast<true>(s[cc], lse2 + c * 32, p.scale_log2, tile_bias, kv_idx, q_base + c * 32, pr[cc]);
          else p_fast<false>(s[cc], lse2 + c * 32, p.scale_log2, tile_bias, kv_idx, q_base + c * 32, pr[cc]);
          uint32_t pk[16];
          if constexpr (DROP == 1 || DROP == 3) {
            if constexpr (DROP == 1) keep_bits[cc] = philox_keep_column(mods, bh, q_base + c * 32, p.S_q - 1, kv_idx, lane);
            else keep_bits[cc] = u8_keep_bits(raw8, lane);
#pragma unroll
            for (int e = 0; e < 16; ++e)   // (explicit roundings: both dropout forms must give the same bits)
              pk[e] = pack2<BF16>(__fmul_rn(pr[cc][2 * e], ((keep_bits[cc] >> (2 * e)) & 1u) ? mods.drop_scale : 0.f),
                                  __fmul_rn(pr[cc][2 * e + 1], ((keep_bits[cc] >> (2 * e + 1)) & 1u) ? mods.drop_scale : 0.f));
          } else if constexpr (DROP == 2) {
#pragma unroll
            for (int e = 0; e < 16; ++e)
              pk[e] = pack2<BF16>(__fmul_rn(pr[cc][2 * e], __fmul_rn(col_value(draw[e], mods.drop_dtype, 0), mods.drop_scale)),
                                  __fmul_rn(pr[cc][2 * e + 1], __fmul_rn(col_value(draw[e], mods.drop_dtype, 1), mods.drop_scale)));
          } else {
#pragma unroll
            for (int e = 0; e < 16; ++e) pk[e] = pack2<BF16>(pr[cc][2 * e], pr[cc][2 * e + 1]);
          }
          tmem_st16(t_st + hf * 64 + cc * 16, pk);
        }
      }
      tmem_wait_st();
      tc_fence_before_sync();
      mbar_arrive(&sh.p_ready);

      // ---- dS part: dS^T = P^T * (dP^T * M - D) into this half's shared-memory block
      mbar_wait(&sh.dp_full, gn & 1, abort_flag, p.status, DEV_TIMEOUT_MMA);
      tc_fence_after_sync();
      if (ds_stage_busy) {       // first step after a write-out: the dK store has long read the tile by now
        if (tid == 0) tma_store_wait_read();
        named_barrier(4, kComputeThreads);
        ds_stage_busy = false;
      }
      {
        uint32_t dp[2][32];
        if constexpr (DROP == 0) {
          tmem_ld32(t_dp + (hf * 2) * 32, dp[0]);
          tmem_ld32(t_dp + (hf * 2 + 1) * 32, dp[1]);
          tmem_wait_ld();
        }
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
          const int c = hf * 2 + cc;
          uint32_t dk_[16];
          if constexpr (DROP == 0) {
#pragma unroll
            for (int e4 = 0; e4 < 8; ++e4) {
              const float4 Dl = *reinterpret_cast<const float4*>(dlt + c * 32 + 4 * e4);
              const float d0 = pr[cc][4 * e4 + 0] * (__uint_as_float(dp[cc][4 * e4 + 0]) - Dl.x);
              const float d1 = pr[cc][4 * e4 + 1] * (__uint_as_float(dp[cc][4 * e4 + 1]) - Dl.y);
              const float d2 = pr[cc][4 * e4 + 2] * (__uint_as_float(dp[cc][4 * e4 + 2]) - Dl.z);
              const float d3 = pr[cc][4 * e4 + 3] * (__uint_as_float(dp[cc][4 * e4 + 3]) - Dl.w);
              dk_[2 * e4] = pack2<BF16>(d0, d1);
              dk_[2 * e4 + 1] = pack2<BF16>(d2, d3);
            }
          } else {
            // With dropout dP is multiplied by the pair's dropout factor before D is subtracted.  One chunk of
            // dP^T at a time keeps the registers within the budget (the dS^T written below goes over columns of
            // chunk 0, which is in registers by then, never over chunk 1).
            tmem_ld32(t_dp + c * 32, dp[cc]);
            uint32_t draw[16];
            if constexpr (DROP == 2)
              load_col32_raw(mods.drop, mods.drop_dtype, static_cast<int64_t>(bh) * p.S_q, q_base + c * 32, p.S_q - 1,
                             p.S_k, min(kv_idx, p.S_k - 1), draw);
            tmem_wait_ld();
#pragma unroll
            for (int e4 = 0; e4 < 8; ++e4) {
              const float4 Dl = *reinterpret_cast<const float4*>(dlt + c * 32 + 4 * e4);
              const float dl[4] = {Dl.x, Dl.y, Dl.z, Dl.w};
              float d[4];
#pragma unroll
              for (int u = 0; u < 4; ++u) {
                const int e = 4 * e4 + u;
                float f;
                if constexpr (DROP == 1 || DROP == 3) f = ((keep_bits[cc] >> e) & 1u) ? mods.drop_scale : 0.f;
                else f = __fmul_rn(col_value(draw[e >> 1], mods.drop_dtype, e & 1), mods.drop_scale);
                d[u] = __fmul_rn(pr[cc][e], __fmaf_rn(__uint_as_float(dp[cc][e]), f, -dl[u]));
              }
              dk_[2 * e4] = pack2<BF16>(d[0], d[1]);
              dk_[2 * e4 + 1] = pack2<BF16>(d[2], d[3]);
            }
          }
          // dS^T goes to two places: over the first 32 of this half's own 64 dP^T columns (both chunks of which
          // are in registers by now), as the A operand of the dK product, and into shared memory, from where the
          // dQ product reads it transposed.  (An A operand in tensor memory runs about a third faster than one in
          // shared memory next to an MN-major B operand.)
          tmem_st16(t_dp + hf * 64 + cc * 16, dk_);
#pragma unroll
          for (int g = 0; g < 4; ++g)
            *reinterpret_cast<uint4*>(my_ds + swz128(r, cc * 4 + g)) =
                make_uint4(dk_[4 * g], dk_[4 * g + 1], dk_[4 * g + 2], dk_[4 * g + 3]);
        }
      }
      tmem_wait_st();
      fence_proxy_async_smem();
      tc_fence_before_sync();
      mbar_arrive(&sh.ds_ready);
      // The next item has been published since this item's first loads went out: learn it one step before the end and
      // request what its first step needs from global memory now, so that those loads return while the last products
      // of this item finish -- not behind the write-out, whose proxy fence would wait for them.
      if (n + 1 == n_iter) {
        next_no = next_item(sh, k + 1, abort_flag, p.status, it_next);
        next_known = true;
        if (next_no < total_items) request_first(it_next);
      }
    }

    // epilogue: dK (scaled) and dV rows of this tile; each half writes its half of head_dim.
    // (the tensor-memory loads are warp-collective: every lane runs them, only the stores are guarded)
    if (n_iter > 0) mbar_wait(&sh.dq_full, (g0 + n_iter - 1) & 1, abort_flag, p.status, DEV_TIMEOUT_MMA);
    tc_fence_after_sync();
    if (!next_known) {      // (an item without steps)
      next_no = next_item(sh, k + 1, abort_flag, p.status, it_next);
      if (next_no < total_items) request_first(it_next);
    }
    const bool row_ok = kv_idx < p.S_k;
    const int64_t row_off = (static_cast<int64_t>(bh_kv) * p.S_k + kv_idx) * p.D;
    if (!p.grads_f32) {
      // 16-bit gradients: dK goes through shared memory (swizzled, conflict-free 16-byte stores) and leaves by one TMA
      // store, which also drops the rows past S_k and the columns past head_dim; dV takes the same way through the
      // drain warps' staging area at the same time.  Direct stores -- one key row per lane, so every store
      // instruction touches 32 different 256-byte rows -- took the compute warps 10 000 to 12 000 clk per work item,
      // during which the next item's first scores sat waiting for them.
      // The staging area is this CTA's dS^T tile: the last dQ product has finished reading it, and the store's own
      // read of it is waited for right before the next dS^T is written (ds_stage_busy).
      {
        if (ds_stage_busy) {     // (an item without steps right after another write-out)
          if (tid == 0) tma_store_wait_read();
          named_barrier(4, kComputeThreads);
        }
        const uint32_t t_src = tmem + lane_base + kColDK;
#pragma unroll 1
        for (int cq = 0; cq < kChunks / 2; ++cq) {
          const int c = hf * (kChunks / 2) + cq;
          uint32_t v[32];
          if (n_iter > 0) { tmem_ld32(t_src + c * 32, v); tmem_wait_ld(); }
          else {
#pragma unroll
            for (int e = 0; e < 32; ++e) v[e] = 0u;
          }
          uint8_t* blk = sDS + (c >> 1) * 16384u;
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint32_t w[4];
#pragma unroll
            for (int e = 0; e < 4; ++e)
              w[e] = pack2<BF16>(__uint_as_float(v[8 * g + 2 * e]) * p.scale, __uint_as_float(v[8 * g + 2 * e + 1]) * p.scale);
            *reinterpret_cast<uint4*>(blk + swz128(r, (c & 1) * 4 + g)) = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
        tc_fence_before_sync();
        if (n_iter > 0) mbar_arrive(&sh.acc_free);      // dK is out of tensor memory (the drain warps answer for dV)
        fence_proxy_async_smem();
        named_barrier(4, kComputeThreads);
        if (tid == 0) {
          for (int nb = 0; nb < NB; ++nb)
            if (nb * 64 < p.D) tma_store_4d(&p.map_dk, sDS + nb * 16384, nb * 64, j * kTile, it.h_kv, b);
          tma_store_commit();
        }
        ds_stage_busy = true;
      }
    } else {
      // fp32 gradients (what the reference's grad primitive returns): each thread stores its key row's half of the
      // 128 x D fp32 tiles directly (a tile is 64 KB: it would take the staging area twice)
#pragma unroll 1
      for (int which = 0; which < 2; ++which) {
        const uint32_t t_src = tmem + lane_base + (which == 0 ? kColDK : kColDV);
        const float mul = which == 0 ? p.scale : 1.0f;
        float* dst = reinterpret_cast<float*>(which == 0 ? p.dk : p.dv) + row_off;
#pragma unroll 1
        for (int cq = 0; cq < kChunks / 2; ++cq) {
          const int c = hf * (kChunks / 2) + cq;
          uint32_t v[32];
          if (n_iter > 0) { tmem_ld32(t_src + c * 32, v); tmem_wait_ld(); }
          else {
#pragma unroll
            for (int e = 0; e < 32; ++e) v[e] = 0u;
          }
          if (!row_ok) continue;
#pragma unroll
          for (int g = 0; g < 8; ++g) {
            const int col = c * 32 + g * 4;
            if (col + 4 <= p.D)
              *reinterpret_cast<float4*>(dst + col) =
                  make_float4(__uint_as_float(v[4 * g]) * mul, __uint_as_float(v[4 * g + 1]) * mul,
                              __uint_as_float(v[4 * g + 2]) * mul, __uint_as_float(v[4 * g + 3]) * mul);
          }
        }
      }
      tc_fence_before_sync();
      // dK and dV are out of tensor memory: the next item's first products may overwrite them
      if (n_iter > 0) mbar_arrive(&sh.acc_free);
    }
    g0 += n_iter;
    item_no = next_no;
    }
    if (ds_stage_busy && tid == 0) tma_store_wait_read();   // shared memory must outlive the last store's read of it
  }

  linger_after_abort(abort_flag);
  __syncthreads();
  if (warp == kProducerWarp) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, 512);
  }
}

// D[row] = sum_d dO[row,d] * O[row,d]  (fp32).  LPR lanes x 16 bytes cover one row, so a warp takes 32 / LPR rows per
// step and every lane loads; a thread block walks rows with a grid stride.
// The same pass zero-fills what the main kernel adds into: row `row` of the packed fp32 dQ accumulator [rows, D] and
// the turn counters (the reference leaves that to its runtime, which zero-fills "atomic add" outputs before the
// launch: flash_attention_bwd.py:55-57).
template <bool BF16, int LPR>
__global__ void bwd_delta_kernel(const void* o, const void* d_o, float* delta, int64_t rows, int D, int64_t sb,
                                 int64_t sh_, int64_t ss, int N, int S_q, float* zero_acc, unsigned int* counters,
                                 int64_t n_counters) {
  constexpr int RPW = 32 / LPR;
  const int lane = threadIdx.x & 31;
  const int sub = lane % LPR, rsub = lane / LPR;
  const int64_t warp_global = static_cast<int64_t>(blockIdx.x) * (blockDim.x / 32) + (threadIdx.x >> 5);
  const int64_t warps_total = static_cast<int64_t>(gridDim.x) * (blockDim.x / 32);
  for (int64_t c = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; c < n_counters;
       c += static_cast<int64_t>(gridDim.x) * blockDim.x)
    counters[c] = 0u;
  for (int64_t row0 = warp_global * RPW; row0 < rows; row0 += warps_total * RPW) {
    const int64_t row = row0 + rsub;
    float acc = 0.f;
    if (row < rows && sub * 8 < D) {
      if (zero_acc != nullptr) {
        float4* z = reinterpret_cast<float4*>(zero_acc + row * D + sub * 8);
        z[0] = make_float4(0.f, 0.f, 0.f, 0.f);
        z[1] = make_float4(0.f, 0.f, 0.f, 0.f);
      }
      const int64_t bh = row / S_q;
      const int64_t off = (bh / N) * sb + (bh % N) * sh_ + (row % S_q) * ss;
      const uint4 a = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(o) + off + sub * 8);
      const uint4 g = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(d_o) + off + sub * 8);
      const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, gw[4] = {g.x, g.y, g.z, g.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float2 x, y;
        if constexpr (BF16) {
          x = make_float2(__uint_as_float(aw[e] << 16), __uint_as_float(aw[e] & 0xffff0000u));
          y = make_float2(__uint_as_float(gw[e] << 16), __uint_as_float(gw[e] & 0xffff0000u));
        } else {
          x = __half22float2(*reinterpret_cast<const __half2*>(&aw[e]));
          y = __half22float2(*reinterpret_cast<const __half2*>(&gw[e]));
        }
        acc = fmaf(x.x, y.x, acc);
        acc = fmaf(x.y, y.y, acc);
      }
    }
#pragma unroll
    for (int off2 = LPR / 2; off2 > 0; off2 >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off2);
    if (sub == 0 && row < rows) delta[row] = acc;
  }
}

template <bool BF16>
__global__ void bwd_convert_kernel(const float* __restrict__ src, void* __restrict__ dst, int64_t n, int f32_out) {
  const int64_t i = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) * 8;
  if (i >= n) return;   // n is a multiple of 8 (head_dim is)
  const float4 a = *reinterpret_cast<const float4*>(src + i);
  const float4 c = *reinterpret_cast<const float4*>(src + i + 4);
  if (f32_out) {
    *reinterpret_cast<float4*>(reinterpret_cast<float*>(dst) + i) = a;
    *reinterpret_cast<float4*>(reinterpret_cast<float*>(dst) + i + 4) = c;
  } else {
    *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(dst) + i) =
        make_uint4(pack2<BF16>(a.x, a.y), pack2<BF16>(a.z, a.w), pack2<BF16>(c.x, c.y), pack2<BF16>(c.z, c.w));
  }
}

cudaError_t launch_fa_bwd(const BwdParams& p, bool bf16, cudaStream_t stream) {
  const int dpad = p.D <= 64 ? 64 : 128;
  const size_t smem = static_cast<size_t>(3 + kStages) * (dpad / 64) * 16384 + 2 * 32768 + sizeof(BwdShared);
  // persistent CTAs, one per SM (tensor memory and shared memory admit no more), fewer if there is less work
  const long long items = static_cast<long long>((p.S_k + kTile - 1) / kTile) * p.B * (p.N / p.kv_group);
  int dev = 0, sms = 0;
  cudaError_t e0 = cudaGetDevice(&dev);
  if (e0 == cudaSuccess) e0 = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (e0 != cudaSuccess) return e0;
  dim3 grid(static_cast<unsigned>(items < sms ? items : sms));
  // (row groups of a multiple of 128 rows never cut a tile: the tile ranges alone take care of them)
  const bool masked = p.mods.mask_kind != 0 || (p.mods.tri_block > 0 && p.mods.tri_block % kTile != 0);
  const bool drop_u8_bits = p.mods.drop != nullptr && p.mods.drop_dtype == 2 /*U8*/ && p.S_k % 4 == 0 &&
                            (reinterpret_cast<uintptr_t>(p.mods.drop) & 3u) == 0;
  const int drop = p.mods.drop_philox != 0 ? 1 : (p.mods.drop != nullptr ? (drop_u8_bits ? 3 : 2) : 0);
  void (*kern)(const BwdParams) = nullptr;
#define ACCT_BWD_DROP(DP, BF, MK)                                                                      \
  (drop == 0 ? fa_bwd_kernel<DP, BF, MK, 0> : drop == 1 ? fa_bwd_kernel<DP, BF, MK, 1>                 \
   : drop == 2 ? fa_bwd_kernel<DP, BF, MK, 2> : fa_bwd_kernel<DP, BF, MK, 3>)
#define ACCT_BWD_PICK(DP, BF) (masked ? ACCT_BWD_DROP(DP, BF, true) : ACCT_BWD_DROP(DP, BF, false))
  if (dpad == 64) kern = bf16 ? ACCT_BWD_PICK(64, true) : ACCT_BWD_PICK(64, false);
  else kern = bf16 ? ACCT_BWD_PICK(128, true) : ACCT_BWD_PICK(128, false);
#undef ACCT_BWD_PICK
#undef ACCT_BWD_DROP
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  if (e != cudaSuccess) return e;
  kern<<<grid, kBwdThreads, smem, stream>>>(p);
  return cudaGetLastError();
}

template <int LPR>
static cudaError_t launch_bwd_delta_lpr(const void* o, const void* d_o, float* delta, int64_t rows, int D, int64_t sb,
                                        int64_t sh_, int64_t ss, int N, int S_q, bool bf16, cudaStream_t stream,
                                        float* zero_acc, unsigned int* counters, int64_t n_counters) {
  const int warps = 8;
  const int64_t rows_per_block = static_cast<int64_t>(warps) * (32 / LPR);
  int64_t blocks = (rows + rows_per_block - 1) / rows_per_block;
  const int64_t cap = 148 * 32;   // a few waves of blocks; the grid stride covers the rest
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  if (bf16) bwd_delta_kernel<true, LPR><<<static_cast<unsigned>(blocks), warps * 32, 0, stream>>>(o, d_o, delta, rows, D, sb, sh_, ss, N, S_q, zero_acc, counters, n_counters);
  else bwd_delta_kernel<false, LPR><<<static_cast<unsigned>(blocks), warps * 32, 0, stream>>>(o, d_o, delta, rows, D, sb, sh_, ss, N, S_q, zero_acc, counters, n_counters);
  return cudaGetLastError();
}

cudaError_t launch_bwd_delta(const void* o, const void* d_o, float* delta, int64_t rows, int D, int64_t o_stride_b,
                             int64_t o_stride_h, int64_t o_stride_s, int N, int S_q, bool bf16,
                             cudaStream_t stream, float* zero_acc, unsigned int* counters, int64_t n_counters) {
  if (D <= 64)
    return launch_bwd_delta_lpr<8>(o, d_o, delta, rows, D, o_stride_b, o_stride_h, o_stride_s, N, S_q, bf16, stream, zero_acc,
                                   counters, n_counters);
  if (D <= 128)
    return launch_bwd_delta_lpr<16>(o, d_o, delta, rows, D, o_stride_b, o_stride_h, o_stride_s, N, S_q, bf16, stream, zero_acc,
                                    counters, n_counters);
  return launch_bwd_delta_lpr<32>(o, d_o, delta, rows, D, o_stride_b, o_stride_h, o_stride_s, N, S_q, bf16, stream, zero_acc,
                                  counters, n_counters);
}

cudaError_t launch_bwd_convert_dq(const float* dq_acc, void* dq, int64_t n_elems, bool bf16, bool f32_out,
                                  cudaStream_t stream) {
  const int threads = 256;
  const unsigned blocks = static_cast<unsigned>((n_elems / 8 + threads - 1) / threads);
  if (bf16) bwd_convert_kernel<true><<<blocks, threads, 0, stream>>>(dq_acc, dq, n_elems, f32_out ? 1 : 0);
  else bwd_convert_kernel<false><<<blocks, threads, 0, stream>>>(dq_acc, dq, n_elems, f32_out ? 1 : 0);
  return cudaGetLastError();
}

}  // namespace acct
