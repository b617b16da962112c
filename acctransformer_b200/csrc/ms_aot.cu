// Entry points with the signature MindSpore gives a custom operator of func_type "aot":
//   int f(int nparam, void** params, int* ndims, int64_t** shapes, const char** dtypes, void* stream, void* extra)
// (params: the inputs followed by the outputs, all device pointers).  They unpack that call into the argument
// structs of the library's own entry points, so that the reference's two primitives
//   train/acctransformer/flash_attention/ops/flash_attention/flash_attention_impl.py:96-126  (grad)
//   train/acctransformer/flash_attention/ops/flash_attention/flash_attention_impl.py:129-154 (forward)
// and its inference op (infer/flash_attention/tik/op_proto/flash_attention_tik.h:22-27) can be registered as
// ops.Custom("libacct_b200.so:acct_ms_fa_fwd", ..., func_type="aot").  Host code only.
//
// The optional inputs carry no names in this calling convention; they are told apart by rank and shape, in the
// reference's order attn_mask, dropout_mask, alibi_mask:
//   rank 3 (or rank 2 128x128)            attn_mask  [1 or B, S_q, S_k] / [1,128,128]
//   rank 4 with shape [B,N,1,S_k]         alibi_mask (when S_q != 1)
//   rank 4 with shape [B,N,S_q,S_k]       dropout_mask
// Operator attributes (band limits, keep probability for uint8 masks, the scale) are not part of the call either.  The
// reference bakes them into each primitive when it is built (flash_attention_impl.py:146-152), so that two layers of
// one graph can differ; here a primitive is bound to one of kSlots numbered attribute slots by the NAME of the entry
// point it calls: acct_ms_fa_attrs_slot() stores a tuple of attributes and returns its slot k, and the operator is
// registered on acct_ms_fa_fwd_s<k> / acct_ms_fa_grad_s<k>.  The unnumbered entry points use the process-wide default
// that acct_ms_set_fa_attrs() sets.
#include <cstring>
#include <mutex>

#include "../../include/acct_b200.h"

namespace {

struct FaAttrs {
  int prev_block_num = ACCT_BAND_UNBOUNDED;
  int next_block_num = ACCT_BAND_UNBOUNDED;
  float keep_prob = 1.0f;
  float scale = 1.0f;   // the raw primitive does not scale (the cell pre-multiplies q and k)
  int causal = 0;
  int optional_inputs = -1;   // which optional inputs the primitive passes (ACCT_MS_HAS_* bits); -1 = tell by shape
};
constexpr int kSlots = 32;
FaAttrs g_attrs;                     // the process-wide default (slot -1)
FaAttrs g_slot[kSlots];
int g_slots_used = 0;
std::mutex g_attrs_mutex;            // set while a graph is built, copied by every call

int dtype_code(const char* s) {
  if (s == nullptr) return -1;
  if (std::strcmp(s, "float16") == 0) return ACCT_F16;
  if (std::strcmp(s, "bfloat16") == 0) return ACCT_BF16;
  if (std::strcmp(s, "uint8") == 0 || std::strcmp(s, "bool") == 0) return ACCT_U8;
  if (std::strcmp(s, "float32") == 0) return ACCT_F32;
  return -1;
}

// Fills the tensor part of `a` from q, k, v at params[0..2]; false if they are not rank-4 [B,N,S,D] tensors of one
// 16-bit type that agree with one another: k and v of one shape [B, N_kv, S_k, D] with N_kv dividing N (the head
// count of k and v is taken from THEIR shape, so a tensor with fewer heads is never read as if it had q's).
bool fill_qkv(acct_fa_args& a, void** params, const int* ndims, int64_t** shapes, const char** dtypes) {
  if (ndims[0] != 4 || ndims[1] != 4 || ndims[2] != 4) return false;
  const int dt = dtype_code(dtypes[0]);
  if (dt != ACCT_F16 && dt != ACCT_BF16) return false;
  if (dtype_code(dtypes[1]) != dt || dtype_code(dtypes[2]) != dt) return false;
  const int64_t* q = shapes[0];
  const int64_t* k = shapes[1];
  const int64_t* v = shapes[2];
  for (int i = 0; i < 4; ++i)
    if (q[i] <= 0 || k[i] <= 0 || q[i] > 0x7fffffff || k[i] > 0x7fffffff || v[i] != k[i]) return false;
  if (k[0] != q[0] || k[3] != q[3] || q[1] % k[1] != 0) return false;
  a.dtype = dt;
  a.B = static_cast<int32_t>(q[0]);
  a.N = static_cast<int32_t>(q[1]);
  a.S_q = static_cast<int32_t>(q[2]);
  a.D = static_cast<int32_t>(q[3]);
  a.S_k = static_cast<int32_t>(k[2]);
  a.N_kv = static_cast<int32_t>(k[1]);
  a.q = params[0];
  a.k = params[1];
  a.v = params[2];
  return true;
}

// true iff tensor i has exactly the given rank-4 shape and type
bool is_shape4(int i, const int* ndims, int64_t** shapes, const char** dtypes, int64_t d0, int64_t d1, int64_t d2, int64_t d3,
               int dt) {
  return ndims[i] == 4 && shapes[i][0] == d0 && shapes[i][1] == d1 && shapes[i][2] == d2 && shapes[i][3] == d3 &&
         dtype_code(dtypes[i]) == dt;
}

// One optional input, known (by declaration) or found (by shape) to be the attn_mask; false if its shape or type
// would make the kernels read out of bounds.
bool place_attn_mask(acct_fa_args& a, int i, void** params, const int* ndims, int64_t** shapes, const char** dtypes) {
  const int r = ndims[i];
  const int64_t* s = shapes[i];
  const int dt = dtype_code(dtypes[i]);
  if ((r != 3 && r != 2) || a.attn_mask != nullptr || dt < 0 || dt == ACCT_F32) return false;
  const bool tile = (r == 3 && s[0] == 1 && s[1] == 128 && s[2] == 128 && !(a.S_q == 128 && a.S_k == 128)) ||
                    (r == 2 && s[0] == 128 && s[1] == 128);
  if (!tile) {   // a full mask is [1 or B, S_q, S_k] (or [S_q, S_k]): anything else would be read out of bounds
    const int64_t mq = r == 3 ? s[1] : s[0], mk = r == 3 ? s[2] : s[1];
    if (mq != a.S_q || mk != a.S_k) return false;
    if (r == 3 && s[0] != 1 && s[0] != a.B) return false;
  }
  a.attn_mask = params[i];
  a.mask_dtype = dt;
  a.mask_kind = tile ? ACCT_MASK_TILE128 : ACCT_MASK_FULL;   // attention.py:279-285
  a.mask_batch = (tile || r == 2) ? 1 : static_cast<int32_t>(s[0]);
  return true;
}
bool place_alibi(acct_fa_args& a, int i, void** params, const int* ndims, int64_t** shapes, const char** dtypes) {
  const int64_t* s = shapes[i];
  if (ndims[i] != 4 || s[0] != a.B || s[1] != a.N || s[2] != 1 || s[3] != a.S_k) return false;
  if (a.alibi != nullptr || dtype_code(dtypes[i]) != a.dtype) return false;
  a.alibi = params[i];
  return true;
}
bool place_dropout(acct_fa_args& a, int i, void** params, const int* ndims, int64_t** shapes, const char** dtypes) {
  const int64_t* s = shapes[i];
  const int dt = dtype_code(dtypes[i]);
  if (ndims[i] != 4 || s[0] != a.B || s[1] != a.N || s[2] != a.S_q || s[3] != a.S_k) return false;
  if (a.dropout_mask != nullptr || dt < 0 || dt == ACCT_F32) return false;
  a.dropout_mask = params[i];
  a.dropout_dtype = dt;
  return true;
}

// Places params[first .. last) as attn_mask / dropout_mask / alibi_mask; false on an input it cannot place.
// `declared` >= 0 (ACCT_MS_HAS_* bits, from the primitive's attribute slot): exactly those inputs, in the reference's
// order (flash_attention_impl.py:146-152), each checked against the shape its name demands.  `declared` < 0: by rank
// and shape, which cannot tell an alibi_mask from a dropout_mask when S_q = 1 (taken for the dropout mask).
bool fill_optionals(acct_fa_args& a, int first, int last, void** params, const int* ndims, int64_t** shapes,
                    const char** dtypes, int declared) {
  if (declared >= 0) {
    int i = first;
    if (declared & ACCT_MS_HAS_ATTN_MASK) { if (i >= last || !place_attn_mask(a, i, params, ndims, shapes, dtypes)) return false; ++i; }
    if (declared & ACCT_MS_HAS_DROPOUT_MASK) { if (i >= last || !place_dropout(a, i, params, ndims, shapes, dtypes)) return false; ++i; }
    if (declared & ACCT_MS_HAS_ALIBI_MASK) { if (i >= last || !place_alibi(a, i, params, ndims, shapes, dtypes)) return false; ++i; }
    return i == last;
  }
  for (int i = first; i < last; ++i) {
    const int r = ndims[i];
    const int64_t* s = shapes[i];
    if (r == 3 || r == 2) {
      if (!place_attn_mask(a, i, params, ndims, shapes, dtypes)) return false;
    } else if (r == 4 && s[2] == 1 && a.S_q != 1) {
      if (!place_alibi(a, i, params, ndims, shapes, dtypes)) return false;
    } else if (!place_dropout(a, i, params, ndims, shapes, dtypes)) {
      return false;
    }
  }
  return true;
}

// A full attn_mask is summarised per 128x128 tile into the library's scratch buffer right before the call that reads
// it (same stream), so that only the mask's mixed tiles are read; a mask too large for the buffer is read in full.
int summarise_mask(acct_fa_args& a, void* stream) {
  if (a.mask_kind != ACCT_MASK_FULL || a.attn_mask == nullptr) return ACCT_OK;
  uint8_t* tiles = acct_mask_tiles_scratch(acct_mask_tiles_bytes(a.mask_batch, a.S_q, a.S_k));
  if (tiles == nullptr) return ACCT_OK;
  const int rc = acct_mask_classify_tiles(a.attn_mask, a.mask_dtype, a.mask_batch, a.S_q, a.S_k, tiles, stream);
  if (rc == ACCT_OK) a.mask_tiles = tiles;
  return rc;
}

// copies the slot's attributes into `a`; returns its declaration of the optional inputs
int apply_attrs(acct_fa_args& a, int slot) {
  FaAttrs at;
  {
    std::lock_guard<std::mutex> lock(g_attrs_mutex);
    at = (slot >= 0 && slot < kSlots) ? g_slot[slot] : g_attrs;
  }
  a.prev_block_num = at.prev_block_num;
  a.next_block_num = at.next_block_num;
  a.keep_prob = at.keep_prob;
  a.scale = at.scale;
  a.causal = at.causal;
  return at.optional_inputs;
}

}  // namespace

extern "C" {

// Process-wide operator attributes for the two training entry points below (set while the graph is built).
ACCT_API void acct_ms_set_fa_attrs(int prev_block_num, int next_block_num, float keep_prob, float scale, int causal) {
  std::lock_guard<std::mutex> lock(g_attrs_mutex);
  g_attrs.prev_block_num = prev_block_num;
  g_attrs.next_block_num = next_block_num;
  g_attrs.keep_prob = keep_prob;
  g_attrs.scale = scale;
  g_attrs.causal = causal;
}

}  // extern "C"

namespace {

// inputs query, key, value, [attn_mask], [dropout_mask], [alibi_mask]; outputs output, rowsum
int ms_fa_fwd(int slot, int nparam, void** params, int* ndims, int64_t** shapes, const char** dtypes, void* stream) {
  if (nparam < 5 || nparam > 8 || params == nullptr || ndims == nullptr || shapes == nullptr || dtypes == nullptr)
    return ACCT_ERR_SHAPE;
  acct_fa_args a;
  std::memset(&a, 0, sizeof a);
  if (!fill_qkv(a, params, ndims, shapes, dtypes)) return ACCT_ERR_SHAPE;
  const int declared = apply_attrs(a, slot);
  if (!fill_optionals(a, 3, nparam - 2, params, ndims, shapes, dtypes, declared)) return ACCT_ERR_SHAPE;
  if (dtype_code(dtypes[nparam - 1]) != ACCT_F32) return ACCT_ERR_DTYPE;   // rowsum is fp32 (impl.py:134-136)
  // output is shaped and typed like q, rowsum is [B, N, S_q]
  if (!is_shape4(nparam - 2, ndims, shapes, dtypes, a.B, a.N, a.S_q, a.D, a.dtype)) return ACCT_ERR_SHAPE;
  if (ndims[nparam - 1] != 3 || shapes[nparam - 1][0] != a.B || shapes[nparam - 1][1] != a.N || shapes[nparam - 1][2] != a.S_q)
    return ACCT_ERR_SHAPE;
  a.o = params[nparam - 2];
  a.lse = static_cast<float*>(params[nparam - 1]);
  if (const int rc = summarise_mask(a, stream)) return rc;
  return acct_fa_fwd(&a, stream);
}

// inputs query, key, value, output, do, rowsum, [attn_mask], [dropout_mask], [alibi_mask];
// outputs dq, dk, dv (fp32, as the reference's grad primitive returns them) and a uint8 workspace tensor of
// acct_fa_bwd_workspace_bytes() bytes, declared as a fourth output so that the framework allocates it.
int ms_fa_grad(int slot, int nparam, void** params, int* ndims, int64_t** shapes, const char** dtypes, void* stream) {
  if (nparam < 10 || nparam > 13 || params == nullptr || ndims == nullptr || shapes == nullptr || dtypes == nullptr)
    return ACCT_ERR_SHAPE;
  acct_fa_args a;
  std::memset(&a, 0, sizeof a);
  if (!fill_qkv(a, params, ndims, shapes, dtypes)) return ACCT_ERR_SHAPE;
  const int first_out = nparam - 4;
  const int declared = apply_attrs(a, slot);
  if (!fill_optionals(a, 6, first_out, params, ndims, shapes, dtypes, declared)) return ACCT_ERR_SHAPE;
  for (int i = first_out; i < first_out + 3; ++i)
    if (dtype_code(dtypes[i]) != ACCT_F32) return ACCT_ERR_DTYPE;
  if (ndims[nparam - 1] != 1) return ACCT_ERR_WORKSPACE;
  // output and do are shaped and typed like q; dq like q, dk and dv like k (fp32)
  for (int i = 3; i <= 4; ++i)
    if (!is_shape4(i, ndims, shapes, dtypes, a.B, a.N, a.S_q, a.D, a.dtype)) return ACCT_ERR_SHAPE;
  if (!is_shape4(first_out, ndims, shapes, dtypes, a.B, a.N, a.S_q, a.D, ACCT_F32)) return ACCT_ERR_SHAPE;
  for (int i = first_out + 1; i < first_out + 3; ++i)
    if (!is_shape4(i, ndims, shapes, dtypes, a.B, a.N_kv, a.S_k, a.D, ACCT_F32)) return ACCT_ERR_SHAPE;
  a.o = params[3];
  a.lse = static_cast<float*>(params[5]);
  if (const int rc = summarise_mask(a, stream)) return rc;
  a.flags |= ACCT_FLAG_GRAD_F32;
  acct_fa_bwd_io g;
  std::memset(&g, 0, sizeof g);
  g.d_o = params[4];
  g.dq = params[first_out];
  g.dk = params[first_out + 1];
  g.dv = params[first_out + 2];
  g.workspace = params[nparam - 1];
  g.workspace_bytes = static_cast<size_t>(shapes[nparam - 1][0]);
  return acct_fa_bwd(&a, &g, stream);
}

}  // namespace

extern "C" {

ACCT_API int acct_ms_fa_fwd(int nparam, void** params, int* ndims, int64_t** shapes, const char** dtypes, void* stream,
                            void* /*extra*/) {
  return ms_fa_fwd(-1, nparam, params, ndims, shapes, dtypes, stream);
}
ACCT_API int acct_ms_fa_grad(int nparam, void** params, int* ndims, int64_t** shapes, const char** dtypes, void* stream,
                             void* /*extra*/) {
  return ms_fa_grad(-1, nparam, params, ndims, shapes, dtypes, stream);
}

// Stores a tuple of attributes and returns the number k of its slot (an identical tuple gets the slot it already
// has); -1 when all slots hold other tuples.  Operators registered on acct_ms_fa_fwd_s<k> / acct_ms_fa_grad_s<k> use it.
ACCT_API int acct_ms_fa_attrs_slot_ex(int prev_block_num, int next_block_num, float keep_prob, float scale, int causal,
                                      int optional_inputs) {
  if (optional_inputs < -1 || optional_inputs > 7) return -1;
  std::lock_guard<std::mutex> lock(g_attrs_mutex);
  for (int i = 0; i < g_slots_used; ++i) {
    const FaAttrs& t = g_slot[i];
    if (t.prev_block_num == prev_block_num && t.next_block_num == next_block_num && t.keep_prob == keep_prob &&
        t.scale == scale && t.causal == causal && t.optional_inputs == optional_inputs)
      return i;
  }
  if (g_slots_used >= kSlots) return -1;
  FaAttrs& t = g_slot[g_slots_used];
  t.prev_block_num = prev_block_num;
  t.next_block_num = next_block_num;
  t.keep_prob = keep_prob;
  t.scale = scale;
  t.causal = causal;
  t.optional_inputs = optional_inputs;
  return g_slots_used++;
}
ACCT_API int acct_ms_fa_attrs_slot(int prev_block_num, int next_block_num, float keep_prob, float scale, int causal) {
  return acct_ms_fa_attrs_slot_ex(prev_block_num, next_block_num, keep_prob, scale, causal, -1);
}

#define ACCT_MS_SLOT(k)                                                                                               \
  ACCT_API int acct_ms_fa_fwd_s##k(int nparam, void** params, int* ndims, int64_t** shapes, const char** dtypes,      \
                                   void* stream, void*) {                                                             \
    return ms_fa_fwd(k, nparam, params, ndims, shapes, dtypes, stream);                                               \
  }                                                                                                                   \
  ACCT_API int acct_ms_fa_grad_s##k(int nparam, void** params, int* ndims, int64_t** shapes, const char** dtypes,     \
                                    void* stream, void*) {                                                            \
    return ms_fa_grad(k, nparam, params, ndims, shapes, dtypes, stream);                                              \
  }
ACCT_MS_SLOT(0) ACCT_MS_SLOT(1) ACCT_MS_SLOT(2) ACCT_MS_SLOT(3) ACCT_MS_SLOT(4) ACCT_MS_SLOT(5) ACCT_MS_SLOT(6) ACCT_MS_SLOT(7)
ACCT_MS_SLOT(8) ACCT_MS_SLOT(9) ACCT_MS_SLOT(10) ACCT_MS_SLOT(11) ACCT_MS_SLOT(12) ACCT_MS_SLOT(13) ACCT_MS_SLOT(14) ACCT_MS_SLOT(15)
ACCT_MS_SLOT(16) ACCT_MS_SLOT(17) ACCT_MS_SLOT(18) ACCT_MS_SLOT(19) ACCT_MS_SLOT(20) ACCT_MS_SLOT(21) ACCT_MS_SLOT(22) ACCT_MS_SLOT(23)
ACCT_MS_SLOT(24) ACCT_MS_SLOT(25) ACCT_MS_SLOT(26) ACCT_MS_SLOT(27) ACCT_MS_SLOT(28) ACCT_MS_SLOT(29) ACCT_MS_SLOT(30) ACCT_MS_SLOT(31)
#undef ACCT_MS_SLOT

// inputs q, k, v (rank 3 [B*N,S,D] or rank 4 [B,N,S,D]); output y shaped like q
// (infer/flash_attention/tik/op_proto/flash_attention_tik.cpp:163-191)
ACCT_API int acct_ms_infer_fa(int nparam, void** params, int* ndims, int64_t** shapes, const char** dtypes, void* stream,
                              void* /*extra*/) {
  if (nparam != 4 || params == nullptr || ndims == nullptr || shapes == nullptr || dtypes == nullptr)
    return ACCT_ERR_SHAPE;
  const int r = ndims[0];
  if ((r != 3 && r != 4) || ndims[1] != r || ndims[2] != r) return ACCT_ERR_SHAPE;
  acct_infer_args a;
  std::memset(&a, 0, sizeof a);
  const int dt = dtype_code(dtypes[0]);
  if (dt != ACCT_F16 && dt != ACCT_BF16) return ACCT_ERR_DTYPE;
  a.dtype = dt;
  a.rank = r;
  const int o = r - 3;   // index of the heads (rank 3: batch*heads) dimension
  a.B = r == 4 ? static_cast<int32_t>(shapes[0][0]) : 1;
  a.N = static_cast<int32_t>(shapes[0][o]);
  a.S_q = static_cast<int32_t>(shapes[0][o + 1]);
  a.D = static_cast<int32_t>(shapes[0][o + 2]);
  a.S_k = static_cast<int32_t>(shapes[1][o + 1]);
  if (shapes[1][o] != shapes[0][o] || shapes[2][o] != shapes[0][o] || shapes[1][o + 2] != a.D ||
      shapes[2][o + 2] != a.D || shapes[2][o + 1] != a.S_k)
    return ACCT_ERR_SHAPE;
  a.q = params[0];
  a.k = params[1];
  a.v = params[2];
  a.y = params[3];
  a.causal = 0;
  a.scale = 1.0f;   // the reference op applies no scale
  return acct_infer_prefill(&a, stream);
}

}  // extern "C"
