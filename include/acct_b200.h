/* acct_b200.h -- C ABI of libacct_b200.so: the attention hot path of acctransformer
 * (FlashAttention2 forward / backward, TriangleAttention's block-causal tiling, and the
 * inference prefill / decode op) as hand-written CUDA for NVIDIA B200 (sm_100a).
 *
 * Conventions
 *   - Plain C types only.  Every pointer named "device" is a CUDA device pointer owned by the
 *     caller; the library never allocates, frees or retains them.  `stream` is a cudaStream_t
 *     passed as void* (NULL = the legacy default stream).  Calls enqueue work and return; they do
 *     not synchronise the host.
 *   - Tensors are [B, N, S, D] ("batch, heads, sequence, head_dim"), D contiguous.  The element
 *     strides of B, N and S are given explicitly; 0 means "packed" (S stride D, N stride S*D,
 *     B stride N*S*D).  Every stride must be a multiple of 8 elements (16 bytes) and every base
 *     pointer 16-byte aligned.
 *   - The device that `stream` belongs to must be the calling thread's current device (per-device
 *     state, such as the status word and built-in scratch, is looked up through the current device).
 *   - Return value: 0 on success, otherwise one of the ACCT_ERR_* codes; acct_last_error() gives
 *     a message for the calling thread.  No C++ exception crosses this boundary.
 *   - Calls return before the kernels run.  A kernel that gives up on a bounded wait leaves garbage
 *     in its outputs and reports it ONLY through the device status word: call acct_device_status()
 *     wherever the host synchronises anyway (end of a step, before results are consumed).
 *   - There is no CPU fallback: without a usable sm_100 device the entry points fail.
 *
 * Paths below are relative to the reference project (mindspore-ai/acctransformer).
 */
#ifndef ACCT_B200_H_
#define ACCT_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ACCT_ABI_VERSION 3

#if defined(__GNUC__)
#define ACCT_API __attribute__((visibility("default")))
#else
#define ACCT_API
#endif

/* element types */
#define ACCT_F16 0
#define ACCT_BF16 1
#define ACCT_U8 2
#define ACCT_F32 3

/* status codes */
#define ACCT_OK 0
#define ACCT_ERR_NULL 1           /* a required pointer is NULL */
#define ACCT_ERR_SHAPE 2          /* a dimension is out of range or inconsistent */
#define ACCT_ERR_DTYPE 3          /* unsupported element type for this argument */
#define ACCT_ERR_UNSUPPORTED_D 4  /* head_dim not a multiple of 8 or larger than the kernels take */
#define ACCT_ERR_ALIGN 5          /* pointer or stride not 16-byte aligned */
#define ACCT_ERR_WORKSPACE 6      /* workspace missing or too small */
#define ACCT_ERR_CUDA 7           /* a CUDA call failed; acct_last_error() carries its text */
#define ACCT_ERR_DEVICE_TIMEOUT 8 /* a kernel gave up on a bounded wait (see acct_device_status) */
#define ACCT_ERR_NO_DEVICE 9      /* no sm_100 device / library built for another architecture */

/* attn_mask forms */
#define ACCT_MASK_NONE 0
#define ACCT_MASK_FULL 1    /* [mask_batch, S_q, S_k], mask_batch in {1, B}; 1 = masked */
#define ACCT_MASK_TILE128 2 /* [1,128,128], applied to diagonal 128x128 tiles only */

/* "no limit" for prev_block_num / next_block_num (the reference's default) */
#define ACCT_BAND_UNBOUNDED 65536
/* the band predicate is evaluated on 128x128 tiles */
#define ACCT_BAND_BLOCK 128
/* value added to a score per unit of attn_mask */
#define ACCT_MASK_FILL_VALUE (-10000.0f)

/* classes of a 128x128 mask tile (acct_fa_args.mask_tiles) */
#define ACCT_MASK_TILE_ZERO 0
#define ACCT_MASK_TILE_MIXED 1
#define ACCT_MASK_TILE_ONE 2

/* flags */
#define ACCT_FLAG_GRAD_F32 1u      /* acct_fa_bwd writes dq/dk/dv as fp32 (what the reference primitive returns) */
#define ACCT_FLAG_DETERMINISTIC 2u /* acct_fa_bwd adds the dq contributions of the K/V tiles in a fixed order, so that
                                      dq is bit-identical from run to run (dk, dv and the forward always are) */

#define ACCT_FLAG_DROPOUT_PHILOX 4u /* dropout decided inside the kernels from (dropout_seed, dropout_offset): no
                                      [B,N,S_q,S_k] mask tensor exists; dropout_mask must be NULL.  See acct_dropout_mask */

/* Arguments shared by the training forward and backward.
 *
 * Replaces the I/O contract of the reference's forward primitive
 *   train/acctransformer/flash_attention/ops/flash_attention/flash_attention_impl.py:30-56,129-154
 *   inputs  query, key, value, [attn_mask], [dropout_mask], [alibi_mask]; outputs output, rowsum;
 *   attrs   prev_block_num, next_block_num, tiling_stgy_name (tile sizes are internal here).
 * Semantics per (b, n) slice, all arithmetic in fp32 except the two matrix products, whose
 * operands are the 16-bit inputs / the 16-bit rounded probabilities:
 *   S = scale * Q K^T + alibi[b,n,0,:] + (-10000) * attn_mask[b or 0]     (flash_attention_fwd.py:308-392,
 *                                                                           attention.py:347-371)
 *   entries outside the block band  j - next <= i <= j + prev  (128-tiles i, j), above the diagonal
 *   when `causal`, or at key positions >= seq_lens[b] do not exist       (flash_attention_fwd.py:444-445)
 *   P = softmax(S);  O = (P * dropout_mask / keep_prob) V;  lse = rowmax(S) + log(rowsum(exp(S - rowmax)))
 *                                                                          (flash_attention_fwd.py:117-153,258-306)
 */
typedef struct acct_fa_args {
  int32_t dtype;            /* ACCT_F16 or ACCT_BF16: type of q, k, v, o, do, alibi */
  int32_t B, N, S_q, S_k, D;
  const void* q;            /* device [B,N,S_q,D] */
  const void* k;            /* device [B,N_kv,S_k,D] */
  const void* v;            /* device [B,N_kv,S_k,D] */
  void* o;                  /* device [B,N,S_q,D]; written by fwd, read by bwd */
  float* lse;               /* device [B,N,S_q] fp32, packed; written by fwd (may be NULL), read by bwd */
  int64_t q_stride[3];      /* element strides of B, N, S; 0 = packed */
  int64_t k_stride[3];
  int64_t v_stride[3];
  int64_t o_stride[3];
  int32_t mask_kind;        /* ACCT_MASK_* */
  int32_t mask_dtype;       /* ACCT_F16 / ACCT_BF16 / ACCT_U8 */
  int32_t mask_batch;       /* 1 or B (ACCT_MASK_FULL) */
  int32_t causal;           /* 1: key j > query i does not exist (no mask tensor is read for it) */
  const void* attn_mask;    /* device, see mask_kind */
  const void* dropout_mask; /* device [B,N,S_q,S_k] or NULL */
  int32_t dropout_dtype;    /* ACCT_U8: {0,1}, P is multiplied by mask/keep_prob;
                               ACCT_F16/ACCT_BF16: values {0, 1/keep_prob} as the reference cell builds them
                               (nn/layer/flash_attention.py:198-203), P is multiplied by the value */
  float keep_prob;          /* 1 - dropout_rate; used with ACCT_U8 */
  const void* alibi;        /* device [B,N,1,S_k] in `dtype`, packed, or NULL */
  const float* alibi_slopes;/* device [N] fp32 or NULL: bias = slope[n] * key_position (computed, not loaded) */
  int32_t prev_block_num;   /* >= ACCT_BAND_UNBOUNDED: no limit */
  int32_t next_block_num;
  float scale;              /* multiplies Q K^T; 1.0 = the raw primitive, head_dim^-1/2 = what the cell's two
                               fp16 multiplies by head_dim^-1/4 amount to (nn/layer/flash_attention.py:188-189) */
  const int32_t* seq_lens;  /* device [B] int32 or NULL: valid key count per batch entry */
  uint32_t flags;           /* ACCT_FLAG_* */
  int32_t tri_block;        /* 0 = off.  > 0: TriangleAttention row groups of this many query rows; a query row in
                               group g sees keys [0, min(S_k, (g+1)*tri_block)) only -- the keys the reference slices in
                               for that group (train/acctransformer/triangle_attention/triangle_attention.py:137-163) */
  uint64_t dropout_seed;    /* ACCT_FLAG_DROPOUT_PHILOX: key of the generator */
  uint64_t dropout_offset;  /* ACCT_FLAG_DROPOUT_PHILOX: below 2^32; a caller advances it from step to step */
  int32_t N_kv;             /* heads of k, v (and dk, dv): 0 or N = one per query head, as the reference requires
                               (nn/layer/flash_attention.py:193-196); a divisor of N = grouped-query attention, query
                               head n reads key/value head n / (N / N_kv); 1 = multi-query */
  const uint8_t* mask_tiles;/* device or NULL.  Summary of an ACCT_MASK_FULL attn_mask, one byte per 128x128 tile,
                               [mask_batch, ceil(S_q/128), ceil(S_k/128)], as acct_mask_classify_tiles writes it:
                               ACCT_MASK_TILE_ZERO = every element of the tile is 0 (the kernels read nothing for it),
                               ACCT_MASK_TILE_ONE = every element is 1 (the fill value is added without reading),
                               ACCT_MASK_TILE_MIXED = the tile is read.  Results are those of reading every tile; the
                               summary must describe the mask's current contents.  NULL = read every tile */
} acct_fa_args;

/* Extra I/O of the backward.
 *
 * Replaces the reference's grad primitive
 *   train/acctransformer/flash_attention/ops/flash_attention/flash_attention_impl.py:59-126
 *   inputs query, key, value, output, do, rowsum, [attn_mask], [dropout_mask], [alibi_mask] -> dq, dk, dv (fp32),
 * which `bprop` then casts to fp16 (:117-124).  dq/dk/dv here are written in `dtype` unless
 * ACCT_FLAG_GRAD_F32 is set; all three are packed [B,N,S,D].
 *   dV = (P*M)^T dO;  dP = (dO V^T)*M;  Dl = rowsum(dO*O);  dS = P*(dP - Dl);
 *   dQ = scale * dS K;  dK = scale * dS^T Q     (flash_attention_bwd.py:88-257, with M = dropout_mask/keep_prob)
 */
typedef struct acct_fa_bwd_io {
  const void* d_o;          /* device [B,N,S_q,D], strides = o_stride */
  void* dq;                 /* device [B,N,S_q,D] packed; with ACCT_FLAG_GRAD_F32 it is also the accumulator the
                               kernel adds into (zero-filled by the call), so no conversion pass follows */
  void* dk;                 /* device [B,N_kv,S_k,D] packed */
  void* dv;                 /* device [B,N_kv,S_k,D] packed */
  void* workspace;          /* device, >= acct_fa_bwd_workspace_bytes(); contents undefined on entry */
  size_t workspace_bytes;
  void* ev_kernel_start;    /* optional cudaEvent_t pair (or NULL): recorded on `stream` directly before and after the */
  void* ev_kernel_stop;     /* main backward kernel, so that a caller can time it apart from the row-sum, zero-fill and
                               dQ-conversion helpers of the same call */
} acct_fa_bwd_io;

/* In-kernel dropout (ACCT_FLAG_DROPOUT_PHILOX) replaces the mask tensor the reference cell generates and keeps in
 * memory for the backward (DropoutGenMask / DropoutDoMask, nn/layer/flash_attention.py:124-130,198-203; 4.3 GB at
 * B=2 N=32 S=8192).  The mask is a pure function of the position:
 *   r = Philox4x32-10(counter = (query, key >> 4, b*N + n, dropout_offset), key = (seed & 0xffffffff, seed >> 32))
 *   byte = byte (key & 15) of the 16 bytes r[0..3], little-endian;   kept  iff  byte < T,  T = round(keep_prob*256)
 * and kept probabilities are multiplied by 256/T, so the effective keep probability is T/256 (keep_prob is
 * quantised to 1/256; T is clamped to [1, 256]).  acct_dropout_mask writes exactly that mask as a packed uint8
 * {0,1} tensor [B,N,S_q,S_k] (reads B, N, S_q, S_k, keep_prob, dropout_seed, dropout_offset of `a` only): with it,
 * the tensor form (dropout_mask = that tensor, dropout_dtype = ACCT_U8, keep_prob = T/256) gives the same results. */
ACCT_API int acct_dropout_mask(const acct_fa_args* a, uint8_t* mask, void* stream);

/* Tells whether an attn_mask tensor [mask_batch, S_q, S_k] (ACCT_F16 / ACCT_BF16 / ACCT_U8, packed) is exactly the
 * causal mask: 1 where key > query, 0 elsewhere.  A caller that gets 1 can drop the tensor and set `causal` instead:
 * the kernels then read no mask at all (268 MB per step at B=8, S=4096) and skip the tiles above the diagonal, which
 * the reference cannot do because its mask is data (flash_attention_fwd.py:352-361 adds it tile by tile;
 * triangle_attention.py:126-135 slices it per row group).  Synchronises `stream`; meant to be called once per mask
 * tensor, not per step.  *is_causal receives 1 or 0. */
ACCT_API int acct_mask_is_causal(const void* mask, int32_t mask_dtype, int32_t mask_batch, int32_t S_q, int32_t S_k,
                                 int32_t* is_causal, void* stream);

/* Summarises an attn_mask tensor [mask_batch, S_q, S_k] (ACCT_F16 / ACCT_BF16 / ACCT_U8, packed) per 128x128 tile
 * into tiles[mask_batch, ceil(S_q/128), ceil(S_k/128)] (device, acct_mask_tiles_bytes() bytes) for
 * acct_fa_args.mask_tiles.  A mask that is not causal (padding, documents, prefixes) is still mostly made of
 * tiles that are all 0 or all 1; with the summary the kernels read only the mixed ones, where the reference reads
 * every tile of every head (flash_attention_fwd.py:352-361, flash_attention_bwd.py:359-372).  One pass over the
 * mask, enqueued on `stream` (no synchronisation); meant to be made once per mask tensor and reused by every
 * forward and backward call that takes that mask. */
ACCT_API size_t acct_mask_tiles_bytes(int32_t mask_batch, int32_t S_q, int32_t S_k);
ACCT_API int acct_mask_classify_tiles(const void* mask, int32_t mask_dtype, int32_t mask_batch, int32_t S_q, int32_t S_k,
                                      uint8_t* tiles, void* stream);

/* A device buffer of the library's own (1 MiB per GPU) for a summary of `bytes` bytes, or NULL if that does not fit:
 * for a caller that has nowhere to keep one between calls and therefore makes it anew before every forward / backward
 * (the entry points with MindSpore's calling convention do that).  One buffer per GPU: calls that use it must be
 * ordered on one stream. */
ACCT_API uint8_t* acct_mask_tiles_scratch(size_t bytes);

/* Forward: writes o and (if non-NULL) lse. */
ACCT_API int acct_fa_fwd(const acct_fa_args* a, void* stream);

/* Bytes of scratch acct_fa_bwd needs for `a` (row sums Dl, turn counters, the work counter of the kernel's persistent
 * thread blocks and, unless ACCT_FLAG_GRAD_F32 is set in a->flags, an fp32 dQ accumulator).  The call initialises
 * what it needs itself: the same workspace can be handed to call after call as it is.
 * The reference declares its fp32 gradient outputs "atomic add" buffers that the runtime zero-fills
 * (flash_attention_bwd.py:55-57); here the library zero-fills its own accumulator on `stream`. */
ACCT_API size_t acct_fa_bwd_workspace_bytes(const acct_fa_args* a);

/* Backward: reads q,k,v,o,lse,d_o (+ the same mask/dropout/alibi/band arguments as the forward). */
ACCT_API int acct_fa_bwd(const acct_fa_args* a, const acct_fa_bwd_io* g, void* stream);

/* Inference op  y = softmax(scale * q k^T) v.
 *
 * Replaces  FlashAttentionTik(q, k, v) -> y
 *   infer/flash_attention/tik/op_proto/flash_attention_tik.h:22-27 (registration),
 *   infer/flash_attention/tik/op_proto/flash_attention_tik.cpp:30-193 (shape checks: rank 3 or 4, k and v of
 *   equal shape, q/k/v agreeing on batch*heads and head_dim, y shaped like q),
 *   infer/flash_attention/tik/tbe/impl/flash_attention_fwd.py:19-748 (kernel).
 * The reference op has no scale, mask or lengths: scale = 1, causal = 0, seq_lens = NULL reproduce it;
 * the other settings are this library's extensions.  rank 3 ([B*N,S,D]) is expressed as B = 1.
 */
typedef struct acct_infer_args {
  int32_t dtype;
  int32_t rank;             /* 3 or 4, validated like the reference's InferShape; layout is the same memory */
  int32_t B, N, S_q, S_k, D;
  const void* q;
  const void* k;
  const void* v;
  void* y;
  int32_t causal;
  float scale;
  const int32_t* seq_lens;  /* device [B] or NULL */
  int32_t N_kv;             /* heads of k and v: 0 or N, or a divisor of N (grouped-query attention) */
} acct_infer_args;

ACCT_API int acct_infer_prefill(const acct_infer_args* a, void* stream);

/* Decode (one query token per sequence over a KV cache).  The reference has no decode path; this is the
 * q_len = 1 case of the op above with per-sequence valid lengths:
 *   y[b,n,0,:] = softmax(scale * q[b,n,0,:] K[b,n,0:len_b,:]^T) V[b,n,0:len_b,:]
 * Keys are split into `num_splits` ranges processed by separate thread blocks; partial (max, sum, acc)
 * triples go to `workspace` and a second kernel merges them. */
typedef struct acct_decode_args {
  int32_t dtype;
  int32_t B, N, S_max, D;
  const void* q;            /* device [B,N,1,D] packed */
  const void* k_cache;      /* device [B,N,S_max,D] */
  const void* v_cache;      /* device [B,N,S_max,D] */
  int64_t kv_stride[3];     /* element strides of B, N, S in the caches; 0 = packed */
  const int32_t* seq_lens;  /* device [B] int32, each in [1, S_max]; NULL = S_max everywhere */
  void* y;                  /* device [B,N,1,D] packed */
  float scale;
  int32_t num_splits;       /* 0 = chosen from the SM count, the number of (sequence, cache head) slices and S_max:
                               8 to 16 ranges of at least 512 keys, and no more than `workspace_bytes` holds */
  void* workspace;          /* device, >= acct_infer_decode_workspace_bytes() */
  size_t workspace_bytes;
  int32_t N_kv;             /* heads of the caches: 0 or N, or a divisor of N (grouped-query attention: the query heads
                               of a group share one pass over their key/value head): N / N_kv up to 16 at head_dim <= 128,
                               one of 2, 4, 8 above */
  /* Paged caches (block_table != NULL): k_cache / v_cache are page pools [num_pages, N_kv, page_size, D] (kv_stride =
   * element strides of page, head, row; 0 = packed), and key position s of sequence b lives in row s % page_size of
   * page block_table[b * max_pages + s / page_size].  S_max is then max_pages * page_size.  No counterpart in the
   * reference (it has no decode path); this is the cache layout serving stacks use. */
  const int32_t* block_table; /* device [B, max_pages] int32 page numbers, or NULL = contiguous caches */
  int32_t page_size;          /* rows per page: a power of two >= 16 */
  int32_t max_pages;          /* columns of block_table */
} acct_decode_args;

ACCT_API size_t acct_infer_decode_workspace_bytes(const acct_decode_args* a);
ACCT_API int acct_infer_decode(const acct_decode_args* a, void* stream);

/* The decode step for callers that cannot allocate device memory (a server whose pool is already carved up,
 * a plugin inside a framework that forbids allocation while a step is recorded or replayed, a latency-critical
 * thread that must stay off the allocator's lock).  No counterpart in the reference: it has no decode path and
 * its runtime hands every op its workspace.
 * Same arguments and results as acct_infer_decode, except that `workspace` / `workspace_bytes` are ignored: the
 * partial results go to an array of ACCT_DECODE_STATIC_SCRATCH_BYTES built into the library, which every GPU that
 * loads the library holds until the process exits.  Returns ACCT_ERR_WORKSPACE if the call needs more than that
 * (B*N*splits*(D+2)*4 bytes); with num_splits = 0 the split count is lowered to what the array holds instead (the
 * result then differs in rounding from a call that was given room for more ranges).  All calls on a GPU share the
 * array: calls that overlap on the GPU race, so keep
 * them ordered on one stream; nothing in the array needs clearing between calls.  The first call on each GPU
 * resolves the array's device address and should come before any stream capture.  Calls no cudaMalloc/cudaFree. */
#define ACCT_DECODE_STATIC_SCRATCH_BYTES (8 * 1024 * 1024)
ACCT_API int acct_infer_decode_static(const acct_decode_args* a, void* stream);

/* The same operators behind the calling convention MindSpore uses for ops.Custom(func_type="aot"):
 *   int f(int nparam, void** params, int* ndims, int64_t** shapes, const char** dtypes, void* stream, void* extra)
 * with params = the inputs followed by the outputs (device pointers), dtypes as MindSpore names them ("float16",
 * "bfloat16", "float32", "uint8", "bool").  They stand where the reference registers its TBE kernels:
 *   acct_ms_fa_fwd   ops.Custom(..., func_type="tbe") forward, flash_attention_impl.py:129-154
 *                    inputs query, key, value, [attn_mask], [dropout_mask], [alibi_mask]; outputs output, rowsum
 *   acct_ms_fa_grad  the grad primitive, flash_attention_impl.py:96-126
 *                    inputs query, key, value, output, do, rowsum, [attn_mask], [dropout_mask], [alibi_mask];
 *                    outputs dq, dk, dv (fp32) and a 1-D uint8 workspace of acct_fa_bwd_workspace_bytes() bytes,
 *                    declared as a fourth output so that the framework allocates it
 *   acct_ms_infer_fa FlashAttentionTik(q, k, v) -> y, flash_attention_tik.h:22-27 (rank 3 or 4)
 * Optional inputs are recognised by rank and shape (rank 3 / 128x128: attn_mask; [B,N,1,S_k]: alibi_mask;
 * [B,N,S_q,S_k]: dropout_mask; with S_q = 1 a lone [B,N,1,S_k] tensor is taken for the dropout mask).  Shapes are
 * checked against one another (k and v of one shape whose head count divides q's, masks and outputs of the sizes
 * that follow from q and k); a mismatch returns ACCT_ERR_SHAPE before anything is read.
 * The attributes the reference bakes into each primitive (flash_attention_impl.py:146-152: band limits; plus the keep
 * probability for uint8 dropout masks, a scale and an implicit causal mask, which are this library's additions) do
 * not travel with such a call.  A primitive is therefore bound to a numbered attribute slot through the NAME of the
 * entry point it is registered on: acct_ms_fa_attrs_slot() stores a tuple and returns its slot k in [0, 32) (an
 * identical tuple gets the slot it already has; -1 when all slots hold other tuples), and the operator pair is
 * registered on acct_ms_fa_fwd_s<k> / acct_ms_fa_grad_s<k>.  Layers of one graph with different band widths, dropout
 * rates or scales thus keep their own values.  The unnumbered entry points use one process-wide tuple, set with
 * acct_ms_set_fa_attrs; its defaults are "no band, keep_prob 1, scale 1, not causal".
 * acct_ms_fa_attrs_slot_ex() also records WHICH optional inputs the primitive passes (ACCT_MS_HAS_* bits, in the
 * reference's order attn_mask, dropout_mask, alibi_mask): the call then takes exactly those, by position, and checks
 * each against the shape its name demands, instead of guessing from shapes (-1 = guess, as the other two do). */
#define ACCT_MS_HAS_ATTN_MASK 1
#define ACCT_MS_HAS_DROPOUT_MASK 2
#define ACCT_MS_HAS_ALIBI_MASK 4
ACCT_API void acct_ms_set_fa_attrs(int prev_block_num, int next_block_num, float keep_prob, float scale, int causal);
ACCT_API int acct_ms_fa_attrs_slot(int prev_block_num, int next_block_num, float keep_prob, float scale, int causal);
ACCT_API int acct_ms_fa_attrs_slot_ex(int prev_block_num, int next_block_num, float keep_prob, float scale, int causal,
                                      int optional_inputs);
#define ACCT_MS_SLOT_ENTRY(k)                                                                                       \
  ACCT_API int acct_ms_fa_fwd_s##k(int nparam, void** params, int* ndims, int64_t** shapes, const char** dtypes,    \
                                   void* stream, void* extra);                                                      \
  ACCT_API int acct_ms_fa_grad_s##k(int nparam, void** params, int* ndims, int64_t** shapes, const char** dtypes,   \
                                    void* stream, void* extra);
ACCT_MS_SLOT_ENTRY(0) ACCT_MS_SLOT_ENTRY(1) ACCT_MS_SLOT_ENTRY(2) ACCT_MS_SLOT_ENTRY(3) ACCT_MS_SLOT_ENTRY(4)
ACCT_MS_SLOT_ENTRY(5) ACCT_MS_SLOT_ENTRY(6) ACCT_MS_SLOT_ENTRY(7) ACCT_MS_SLOT_ENTRY(8) ACCT_MS_SLOT_ENTRY(9)
ACCT_MS_SLOT_ENTRY(10) ACCT_MS_SLOT_ENTRY(11) ACCT_MS_SLOT_ENTRY(12) ACCT_MS_SLOT_ENTRY(13) ACCT_MS_SLOT_ENTRY(14)
ACCT_MS_SLOT_ENTRY(15) ACCT_MS_SLOT_ENTRY(16) ACCT_MS_SLOT_ENTRY(17) ACCT_MS_SLOT_ENTRY(18) ACCT_MS_SLOT_ENTRY(19)
ACCT_MS_SLOT_ENTRY(20) ACCT_MS_SLOT_ENTRY(21) ACCT_MS_SLOT_ENTRY(22) ACCT_MS_SLOT_ENTRY(23) ACCT_MS_SLOT_ENTRY(24)
ACCT_MS_SLOT_ENTRY(25) ACCT_MS_SLOT_ENTRY(26) ACCT_MS_SLOT_ENTRY(27) ACCT_MS_SLOT_ENTRY(28) ACCT_MS_SLOT_ENTRY(29)
ACCT_MS_SLOT_ENTRY(30) ACCT_MS_SLOT_ENTRY(31)
#undef ACCT_MS_SLOT_ENTRY
ACCT_API int acct_ms_fa_fwd(int nparam, void** params, int* ndims, int64_t** shapes, const char** dtypes, void* stream,
                            void* extra);
ACCT_API int acct_ms_fa_grad(int nparam, void** params, int* ndims, int64_t** shapes, const char** dtypes, void* stream,
                             void* extra);
ACCT_API int acct_ms_infer_fa(int nparam, void** params, int* ndims, int64_t** shapes, const char** dtypes, void* stream,
                              void* extra);

/* Reads and clears the device-side status word of the current device (synchronises `stream`).
 * Returns ACCT_OK, or ACCT_ERR_DEVICE_TIMEOUT if some kernel gave up on a bounded wait since the last call. */
ACCT_API int acct_device_status(void* stream);

/* Failure-reporting self-test: enqueues a one-thread kernel whose bounded wait is certain to run out (it waits, with
 * a small poll limit, on a barrier nothing arrives at), so that the next acct_device_status() returns
 * ACCT_ERR_DEVICE_TIMEOUT.  The kernel returns normally; the context stays usable and later calls are unaffected.
 * No counterpart in the reference (its kernels have no waits that can be observed from the host). */
ACCT_API int acct_selftest_wait_timeout(void* stream);

/* Message for the last non-zero return on the calling thread ("" if none). */
ACCT_API const char* acct_last_error(void);

/* ACCT_ABI_VERSION the library was built with. */
ACCT_API int acct_abi_version(void);

#ifdef __cplusplus
}
#endif
#endif /* ACCT_B200_H_ */
