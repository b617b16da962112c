// Parameter blocks and launchers of the attention kernels (internal to the library).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace acct {

constexpr int kTile = 128;          // rows of a Q tile and of a K/V tile; also the band block
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

// What the softmax stage must look at besides the raw scores.
struct ScoreMods {
  int causal;
  int prev_block_num, next_block_num;
  int mask_kind, mask_dtype, mask_batch;
  const void* mask;
  const uint8_t* mask_tiles;        // optional [mask_batch, ceil(S_q/128), ceil(S_k/128)]: 0 = tile all 0 (not read),
                                    // 2 = tile all 1 (fill value added, not read), 1 = read; null = read every tile
  const void* drop;
  int drop_dtype;
  float drop_scale;                 // 1/keep_prob for uint8 masks, 1 for pre-scaled 16-bit masks
  const void* alibi;                // [B,N,1,S_k] in the tensor dtype
  const float* alibi_slopes;        // [N]
  const int* seq_lens;              // [B]
  int tri_block;                    // > 0: query row r sees keys < (r / tri_block + 1) * tri_block only
  int drop_philox;                  // 1: dropout decided in the kernel (DropoutRng), `drop` is null, drop_scale = 256/threshold
  unsigned int drop_seed_lo, drop_seed_hi, drop_offset, drop_threshold;
};

struct alignas(64) FwdParams {
  CUtensorMap map_q, map_k, map_v, map_o;
  void* o;
  float* lse;
  int64_t o_stride_b, o_stride_h, o_stride_s;
  int B, N, S_q, S_k, D;
  int kv_group;                     // query heads per key/value head (1 unless grouped-query attention)
  int unit_group;                   // (batch, head) slices whose thread blocks are interleaved, heaviest tile pairs first
  float scale_log2;                 // scale * log2(e)
  ScoreMods mods;
  unsigned int* status;
};

struct alignas(64) BwdParams {
  CUtensorMap map_q, map_k, map_v, map_do;
  CUtensorMap map_dq;               // fp32 dQ accumulator [B,N,S_q,D], box 32 x 128
  CUtensorMap map_dk, map_dv;       // 16-bit dk, dv [B,N_kv,S_k,D], box 64 x 128 (unused with fp32 gradients and above head_dim 128)
  const float* lse;                 // [B,N,S_q]
  const float* delta;               // [B,N,S_q]  rowsum(dO * O)
  float* dq_acc;                    // [B,N,S_q,D] fp32, zeroed before launch
  unsigned int* dq_order;           // [B,N,ceil(S_q/128)] turn counters (x 2 for head_dim > 128), zeroed before launch;
                                    // nullptr = any order
  unsigned int* work_counter;       // one word, zeroed before launch: the next work item of the persistent CTAs
  void* dk;
  void* dv;
  int grads_f32;
  int B, N, S_q, S_k, D;
  int kv_group;                     // query heads per key/value head; dk, dv are [B, N / kv_group, S_k, D]
  float scale;                      // multiplies dS for dQ and dK
  float scale_log2;
  ScoreMods mods;
  unsigned int* status;
};

struct DecodeParams {
  const void* q;
  const void* k;
  const void* v;
  void* y;
  const int* seq_lens;
  float* part_acc;                  // [B*N, splits, D]
  float* part_ml;                   // [B*N, splits, 2]
  int64_t kv_stride_b, kv_stride_h, kv_stride_s;
  int B, N, S_max, D;
  int kv_group;                     // query heads per key/value head: 1..16 (head_dim <= 128), else 1, 2, 4 or 8
  const int* block_table;           // [B, max_pages] page numbers, or nullptr: contiguous caches
  int page_shift, max_pages;        // rows per page = 1 << page_shift; kv_stride_b is then the page stride
  int splits;
  float scale_log2;
};

// counts into *mismatch the elements of a [batch, S_q, S_k] mask that differ from the causal mask (key > query)
cudaError_t launch_mask_check(const void* mask, int dtype, int batch, int S_q, int S_k, unsigned int* mismatch,
                              cudaStream_t stream);

// writes one class byte per 128x128 tile of a [batch, S_q, S_k] mask into tiles[batch, ceil(S_q/128), ceil(S_k/128)]:
// 0 = all elements 0, 2 = all elements 1, 1 = anything else (ScoreMods::mask_tiles)
cudaError_t launch_mask_classify(const void* mask, int dtype, int batch, int S_q, int S_k, uint8_t* tiles,
                                 cudaStream_t stream);

// Launchers: return cudaGetLastError() of the launch.
cudaError_t launch_fa_fwd(const FwdParams& p, bool bf16, cudaStream_t stream);
cudaError_t launch_fa_bwd(const BwdParams& p, bool bf16, cudaStream_t stream);
// head_dim in (128, 256]: Q / dO maps with 64-row boxes, the dQ map with a 32 x 64 box, two turn counters per Q tile
cudaError_t launch_fa_bwd_wide(const BwdParams& p, bool bf16, cudaStream_t stream);
// writes the {0,1} mask the kernels' in-kernel dropout uses, [units, S_q, S_k] uint8 (units = B*N)
cudaError_t launch_dropout_mask(unsigned char* mask, int units, int S_q, int S_k, unsigned int seed_lo, unsigned int seed_hi,
                                unsigned int offset, unsigned int threshold, cudaStream_t stream);
// delta = rowsum(dO * O); the same pass zero-fills the packed fp32 dQ accumulator zero_acc[rows, D] and the counters
cudaError_t launch_bwd_delta(const void* o, const void* d_o, float* delta, int64_t rows, int D, int64_t o_stride_b,
                             int64_t o_stride_h, int64_t o_stride_s, int N, int S_q, bool bf16,
                             cudaStream_t stream, float* zero_acc, unsigned int* counters, int64_t n_counters);
cudaError_t launch_bwd_convert_dq(const float* dq_acc, void* dq, int64_t n_elems, bool bf16, bool f32_out,
                                  cudaStream_t stream);
cudaError_t launch_decode(const DecodeParams& p, bool bf16, cudaStream_t stream);
// split kernel for 2..16 query heads per cache head at head_dim <= 128 (tensor-core path, decode_gqa.cu)
cudaError_t launch_decode_gqa_split(const DecodeParams& p, bool bf16, cudaStream_t stream);
#ifndef ACCT_DECODE_GQA_MIN_GROUP
#define ACCT_DECODE_GQA_MIN_GROUP 2
#endif
constexpr int kDecodeGqaMinGroup = ACCT_DECODE_GQA_MIN_GROUP;   // groups of at least this many heads take that path

}  // namespace acct
