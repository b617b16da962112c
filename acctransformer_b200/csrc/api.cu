// C-ABI entry points of libacct_b200.so: argument validation (the role the reference's Python
// checks and its C++ InferShape play), tensor-map construction and kernel launches.
#include <mutex>
#include <stdarg.h>

#include "common.cuh"
#include "fa_kernels.cuh"
#include "ptx.cuh"

namespace acct {

// ---------------------------------------------------------------------------------------------
// errors
// ---------------------------------------------------------------------------------------------
char* last_error_buf() {
  static thread_local char buf[512] = {0};
  return buf;
}

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(last_error_buf(), 512, fmt, ap);
  va_end(ap);
  return code;
}

int fail_cuda(cudaError_t e, const char* what) {
  return fail(ACCT_ERR_CUDA, "%s: %s (%s)", what, cudaGetErrorString(e), cudaGetErrorName(e));
}

// ---------------------------------------------------------------------------------------------
// per-device state
// ---------------------------------------------------------------------------------------------
__device__ unsigned int g_status_word = 0;
// Scratch for a mask's per-tile summary, for callers that have nowhere to keep one (acct_mask_tiles_scratch).
constexpr size_t kTilesScratchBytes = 1u << 20;
__device__ uint8_t g_tiles_scratch[kTilesScratchBytes];
__device__ unsigned int g_mask_mismatch;   // scratch of acct_mask_is_causal (calls are serialised by g_mask_mutex)

// One thread waits, with the same bounded wait the attention kernels use (poll limit 2^10 instead of 2^24), on a
// barrier at which nothing ever arrives.  The wait runs out, the status word receives DEV_TIMEOUT_SYNC and the
// kernel returns normally: what a real kernel does when a hand-off never comes, without any of its work.
__global__ void wait_timeout_selftest_kernel(unsigned int* status) {
  __shared__ uint64_t bar;
  __shared__ volatile uint32_t abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    abort_flag = 0;
    mbar_fence_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) mbar_wait<(1u << 10)>(&bar, 0, &abort_flag, status, DEV_TIMEOUT_SYNC);
  __syncthreads();
  linger_after_abort(&abort_flag);
}

namespace {
constexpr int kMaxDevices = 64;
std::mutex g_mutex;
std::mutex g_mask_mutex;
struct PerDevice {
  bool ready = false;
  int rc = 0;
  DeviceInfo info{};
  unsigned int* status = nullptr;
};
PerDevice g_dev[kMaxDevices];

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;

int init_device(PerDevice** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(ACCT_ERR_NO_DEVICE, "no CUDA device: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices) return fail(ACCT_ERR_NO_DEVICE, "device index %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_mutex);
  PerDevice& d = g_dev[dev];
  if (!d.ready) {
    cudaDeviceProp prop;
    e = cudaGetDeviceProperties(&prop, dev);
    if (e != cudaSuccess) return fail_cuda(e, "cudaGetDeviceProperties");
    d.info.sm_count = prop.multiProcessorCount;
    d.info.cc_major = prop.major;
    d.info.cc_minor = prop.minor;
    d.info.max_smem_optin = static_cast<int>(prop.sharedMemPerBlockOptin);
    if (prop.major != 10) {
      d.rc = ACCT_ERR_NO_DEVICE;
    } else {
      e = cudaGetSymbolAddress(reinterpret_cast<void**>(&d.status), g_status_word);
      if (e != cudaSuccess) return fail_cuda(e, "cudaGetSymbolAddress(status)");
      if (g_encode == nullptr) {
        cudaDriverEntryPointQueryResult q;
        void* fn = nullptr;
        e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
        if (e != cudaSuccess || fn == nullptr) return fail(ACCT_ERR_CUDA, "cuTensorMapEncodeTiled unavailable");
        g_encode = reinterpret_cast<EncodeTiledFn>(fn);
      }
    }
    d.ready = true;
  }
  if (d.rc != 0)
    return fail(d.rc, "device %d is sm_%d%d; this library is built for sm_100a only", dev, d.info.cc_major,
                d.info.cc_minor);
  *out = &d;
  return 0;
}
}  // namespace

int device_info(DeviceInfo* out) {
  PerDevice* d = nullptr;
  int rc = init_device(&d);
  if (rc) return rc;
  *out = d->info;
  return 0;
}

unsigned int* device_status_ptr() {
  PerDevice* d = nullptr;
  if (init_device(&d)) return nullptr;
  return d->status;
}

int make_tmap_4d(CUtensorMap* out, const TensorDesc4& t, int box_rows) {
  cuuint64_t dims[4] = {(cuuint64_t)t.dims[0], (cuuint64_t)t.dims[1], (cuuint64_t)t.dims[2], (cuuint64_t)t.dims[3]};
  // rows of the box are 128 bytes: 64 sixteen-bit elements, or 32 fp32 elements (the dQ accumulator)
  const cuuint64_t esz = t.dtype == ACCT_F32 ? 4 : 2;
  cuuint64_t strides[3] = {(cuuint64_t)t.strides[0] * esz, (cuuint64_t)t.strides[1] * esz, (cuuint64_t)t.strides[2] * esz};
  cuuint32_t box[4] = {(cuuint32_t)(128 / esz), (cuuint32_t)box_rows, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  const CUtensorMapDataType dt = t.dtype == ACCT_F32    ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                 : t.dtype == ACCT_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                        : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  CUresult r = g_encode(out, dt, 4, const_cast<void*>(t.ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(ACCT_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return 0;
}

// ---------------------------------------------------------------------------------------------
// validation
// ---------------------------------------------------------------------------------------------
namespace {

constexpr int kMaxHeadDimCell = 256;   // the reference cell's limit (nn/layer/flash_attention.py:26,105-106)
constexpr int kMaxHeadDimFwd = 256;    // forward / prefill kernels: tiles padded to 64, 128 or 256 columns
constexpr int kMaxHeadDimBwd = 256;    // backward: one kernel up to 128, the split-width kernel above that

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int check_strides(const char* name, const int64_t s[3], int64_t S, int64_t N, int64_t D, int64_t out[3]) {
  out[2] = packed_or(s[2], D);
  out[1] = packed_or(s[1], S * D);
  out[0] = packed_or(s[0], N * S * D);
  for (int i = 0; i < 3; ++i) {
    if (out[i] <= 0) return fail(ACCT_ERR_SHAPE, "%s stride %d must be positive", name, i);
    if (out[i] % 8 != 0) return fail(ACCT_ERR_ALIGN, "%s stride %d (%lld elements) is not a multiple of 8", name, i, (long long)out[i]);
  }
  if (out[2] < D) return fail(ACCT_ERR_SHAPE, "%s sequence stride smaller than head_dim", name);
  return 0;
}

int check_head_dim(int D, int kernel_max, const char* what) {
  if (D <= 0 || D > kMaxHeadDimCell) return fail(ACCT_ERR_UNSUPPORTED_D, "head_dim %d outside (0, %d]", D, kMaxHeadDimCell);
  if (D % 8 != 0) return fail(ACCT_ERR_UNSUPPORTED_D, "head_dim %d is not a multiple of 8", D);
  if (D > kernel_max) return fail(ACCT_ERR_UNSUPPORTED_D, "head_dim %d > %d is not built for the %s", D, kernel_max, what);
  return 0;
}

struct Strides {
  int64_t q[3], k[3], v[3], o[3];
};

// heads of k / v: one per query head unless the caller groups them
int kv_heads(const acct_fa_args* a) { return a->N_kv > 0 ? a->N_kv : a->N; }

int validate_fa(const acct_fa_args* a, Strides* st, bool backward = false) {
  if (a == nullptr) return fail(ACCT_ERR_NULL, "args is NULL");
  if (a->dtype != ACCT_F16 && a->dtype != ACCT_BF16) return fail(ACCT_ERR_DTYPE, "dtype must be ACCT_F16 or ACCT_BF16");
  if (a->B <= 0 || a->N <= 0 || a->S_q <= 0 || a->S_k <= 0) return fail(ACCT_ERR_SHAPE, "B, N, S_q, S_k must be positive");
  if (static_cast<int64_t>(a->B) * a->N > 65535) return fail(ACCT_ERR_SHAPE, "B*N = %lld exceeds 65535", (long long)a->B * a->N);
  int rc = backward ? check_head_dim(a->D, kMaxHeadDimBwd, "backward") : check_head_dim(a->D, kMaxHeadDimFwd, "forward");
  if (rc) return rc;
  if (!a->q || !a->k || !a->v || !a->o) return fail(ACCT_ERR_NULL, "q, k, v, o must be non-NULL");
  if (!aligned16(a->q) || !aligned16(a->k) || !aligned16(a->v) || !aligned16(a->o))
    return fail(ACCT_ERR_ALIGN, "q, k, v, o must be 16-byte aligned");
  if ((rc = check_strides("q", a->q_stride, a->S_q, a->N, a->D, st->q))) return rc;
  if (a->N_kv < 0 || (a->N_kv > 0 && a->N % a->N_kv != 0))
    return fail(ACCT_ERR_SHAPE, "N_kv = %d must be 0 or a divisor of N = %d", a->N_kv, a->N);
  const int n_kv = kv_heads(a);
  if ((rc = check_strides("k", a->k_stride, a->S_k, n_kv, a->D, st->k))) return rc;
  if ((rc = check_strides("v", a->v_stride, a->S_k, n_kv, a->D, st->v))) return rc;
  if ((rc = check_strides("o", a->o_stride, a->S_q, a->N, a->D, st->o))) return rc;
  if (!(a->scale > 0.f) || !(a->scale < 1e30f)) return fail(ACCT_ERR_SHAPE, "scale must be a positive finite number");
  if (a->prev_block_num < 0 || a->next_block_num < 0) return fail(ACCT_ERR_SHAPE, "prev/next_block_num must be >= 0");
  switch (a->mask_kind) {
    case ACCT_MASK_NONE: break;
    case ACCT_MASK_FULL:
      if (!a->attn_mask) return fail(ACCT_ERR_NULL, "attn_mask is NULL for ACCT_MASK_FULL");
      if (a->mask_batch != 1 && a->mask_batch != a->B) return fail(ACCT_ERR_SHAPE, "mask_batch must be 1 or B");
      break;
    case ACCT_MASK_TILE128:
      if (!a->attn_mask) return fail(ACCT_ERR_NULL, "attn_mask is NULL for ACCT_MASK_TILE128");
      break;
    default: return fail(ACCT_ERR_SHAPE, "unknown mask_kind %d", a->mask_kind);
  }
  if (a->mask_tiles != nullptr && a->mask_kind != ACCT_MASK_FULL)
    return fail(ACCT_ERR_SHAPE, "mask_tiles describes an ACCT_MASK_FULL attn_mask only");
  if (a->mask_kind != ACCT_MASK_NONE && a->mask_dtype != ACCT_F16 && a->mask_dtype != ACCT_BF16 && a->mask_dtype != ACCT_U8)
    return fail(ACCT_ERR_DTYPE, "attn_mask dtype must be F16, BF16 or U8");
  if (a->dropout_mask) {
    if (a->dropout_dtype != ACCT_F16 && a->dropout_dtype != ACCT_BF16 && a->dropout_dtype != ACCT_U8)
      return fail(ACCT_ERR_DTYPE, "dropout_mask dtype must be U8, F16 or BF16");
    if (a->dropout_dtype == ACCT_U8 && !(a->keep_prob > 0.f && a->keep_prob <= 1.f))
      return fail(ACCT_ERR_SHAPE, "keep_prob must be in (0, 1]");
  }
  if (a->flags & ACCT_FLAG_DROPOUT_PHILOX) {
    if (a->dropout_mask) return fail(ACCT_ERR_SHAPE, "ACCT_FLAG_DROPOUT_PHILOX excludes a dropout_mask tensor");
    if (!(a->keep_prob > 0.f && a->keep_prob <= 1.f)) return fail(ACCT_ERR_SHAPE, "keep_prob must be in (0, 1]");
    if (a->dropout_offset >> 32) return fail(ACCT_ERR_SHAPE, "dropout_offset must be below 2^32");
  }
  if (a->tri_block < 0) return fail(ACCT_ERR_SHAPE, "tri_block must be >= 0");
  if (a->alibi && a->alibi_slopes) return fail(ACCT_ERR_SHAPE, "give either alibi or alibi_slopes, not both");
  return 0;
}

// round(keep_prob * 256) clamped to [1, 256]: positions whose random byte is below it are kept
unsigned int dropout_threshold(float keep_prob) {
  const long t = lroundf(keep_prob * 256.0f);
  return static_cast<unsigned int>(t < 1 ? 1 : (t > 256 ? 256 : t));
}

ScoreMods make_mods(const acct_fa_args* a) {
  ScoreMods m;
  m.causal = a->causal ? 1 : 0;
  m.prev_block_num = a->prev_block_num >= ACCT_BAND_UNBOUNDED ? ACCT_BAND_UNBOUNDED : a->prev_block_num;
  m.next_block_num = a->next_block_num >= ACCT_BAND_UNBOUNDED ? ACCT_BAND_UNBOUNDED : a->next_block_num;
  m.mask_kind = a->mask_kind;
  m.mask_dtype = a->mask_dtype;
  m.mask_batch = a->mask_batch;
  m.mask = a->mask_kind == ACCT_MASK_NONE ? nullptr : a->attn_mask;
  m.mask_tiles = a->mask_kind == ACCT_MASK_FULL ? a->mask_tiles : nullptr;
  m.drop = a->dropout_mask;
  m.drop_dtype = a->dropout_dtype;
  m.drop_scale = (a->dropout_mask && a->dropout_dtype == ACCT_U8) ? 1.0f / a->keep_prob : 1.0f;
  m.alibi = a->alibi;
  m.alibi_slopes = a->alibi_slopes;
  m.seq_lens = a->seq_lens;
  m.tri_block = a->tri_block;
  m.drop_philox = 0;
  m.drop_seed_lo = m.drop_seed_hi = m.drop_offset = 0;
  m.drop_threshold = 256;
  if ((a->flags & ACCT_FLAG_DROPOUT_PHILOX) && dropout_threshold(a->keep_prob) < 256u) {
    m.drop_philox = 1;
    m.drop_seed_lo = static_cast<unsigned int>(a->dropout_seed & 0xffffffffull);
    m.drop_seed_hi = static_cast<unsigned int>(a->dropout_seed >> 32);
    m.drop_offset = static_cast<unsigned int>(a->dropout_offset);
    m.drop_threshold = dropout_threshold(a->keep_prob);
    m.drop_scale = 256.0f / static_cast<float>(m.drop_threshold);
  }
  return m;
}

int make_qkv_maps(const acct_fa_args* a, const Strides& st, CUtensorMap* mq, CUtensorMap* mk, CUtensorMap* mv,
                  int q_box_rows = kTile) {
  TensorDesc4 t;
  t.dtype = a->dtype;
  int rc;
  t.ptr = a->q; t.dims[0] = a->D; t.dims[1] = a->S_q; t.dims[2] = a->N; t.dims[3] = a->B;
  t.strides[0] = st.q[2]; t.strides[1] = st.q[1]; t.strides[2] = st.q[0];
  if ((rc = make_tmap_4d(mq, t, q_box_rows))) return rc;
  t.ptr = a->k; t.dims[1] = a->S_k; t.dims[2] = kv_heads(a);
  t.strides[0] = st.k[2]; t.strides[1] = st.k[1]; t.strides[2] = st.k[0];
  if ((rc = make_tmap_4d(mk, t, kTile))) return rc;
  t.ptr = a->v;
  t.strides[0] = st.v[2]; t.strides[1] = st.v[1]; t.strides[2] = st.v[0];
  return make_tmap_4d(mv, t, kTile);
}

}  // namespace
}  // namespace acct

using namespace acct;

extern "C" {

int acct_abi_version(void) { return ACCT_ABI_VERSION; }

const char* acct_last_error(void) { return last_error_buf(); }

int acct_device_status(void* stream) {
  unsigned int* st = device_status_ptr();
  if (st == nullptr) return ACCT_ERR_NO_DEVICE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  unsigned int host = 0;
  cudaError_t e = cudaMemcpyAsync(&host, st, sizeof(host), cudaMemcpyDeviceToHost, s);
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  if (e != cudaSuccess) return fail_cuda(e, "reading the device status word");
  if (host != 0) {
    e = cudaMemsetAsync(st, 0, sizeof(host), s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    return fail(ACCT_ERR_DEVICE_TIMEOUT, "a kernel gave up on a bounded wait (code %u: 1=TMA load, 2=MMA completion, 3=hand-off, 4=shared-memory base misaligned)", host);
  }
  return ACCT_OK;
}

int acct_selftest_wait_timeout(void* stream) {
  unsigned int* st = device_status_ptr();
  if (st == nullptr) return ACCT_ERR_NO_DEVICE;
  wait_timeout_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(st);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail_cuda(e, "launching the wait self-test kernel");
  return ACCT_OK;
}

int acct_dropout_mask(const acct_fa_args* a, uint8_t* mask, void* stream) {
  if (a == nullptr || mask == nullptr) return fail(ACCT_ERR_NULL, "acct_dropout_mask: NULL argument");
  if (a->B <= 0 || a->N <= 0 || a->S_q <= 0 || a->S_k <= 0) return fail(ACCT_ERR_SHAPE, "B, N, S_q, S_k must be positive");
  if (!(a->keep_prob > 0.f && a->keep_prob <= 1.f)) return fail(ACCT_ERR_SHAPE, "keep_prob must be in (0, 1]");
  if (a->dropout_offset >> 32) return fail(ACCT_ERR_SHAPE, "dropout_offset must be below 2^32");
  if (device_status_ptr() == nullptr) return ACCT_ERR_NO_DEVICE;
  cudaError_t e = launch_dropout_mask(mask, a->B * a->N, a->S_q, a->S_k, static_cast<unsigned int>(a->dropout_seed & 0xffffffffull),
                                      static_cast<unsigned int>(a->dropout_seed >> 32),
                                      static_cast<unsigned int>(a->dropout_offset), dropout_threshold(a->keep_prob),
                                      static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return fail_cuda(e, "launching the dropout mask kernel");
  return ACCT_OK;
}

int acct_mask_is_causal(const void* mask, int32_t mask_dtype, int32_t mask_batch, int32_t S_q, int32_t S_k,
                        int32_t* is_causal, void* stream) {
  if (mask == nullptr || is_causal == nullptr) return fail(ACCT_ERR_NULL, "acct_mask_is_causal: NULL argument");
  if (mask_dtype != ACCT_F16 && mask_dtype != ACCT_BF16 && mask_dtype != ACCT_U8)
    return fail(ACCT_ERR_DTYPE, "attn_mask dtype must be F16, BF16 or U8");
  if (mask_batch <= 0 || S_q <= 0 || S_k <= 0) return fail(ACCT_ERR_SHAPE, "mask_batch, S_q, S_k must be positive");
  if (device_status_ptr() == nullptr) return ACCT_ERR_NO_DEVICE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // the scratch word is one per device: hold the lock until the answer has been read back
  std::lock_guard<std::mutex> lock(g_mask_mutex);
  unsigned int* flag = nullptr;
  cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&flag), g_mask_mismatch);
  if (e == cudaSuccess) e = cudaMemsetAsync(flag, 0, sizeof(unsigned int), s);
  if (e == cudaSuccess) e = launch_mask_check(mask, mask_dtype, mask_batch, S_q, S_k, flag, s);
  unsigned int host = 1;
  if (e == cudaSuccess) e = cudaMemcpyAsync(&host, flag, sizeof(host), cudaMemcpyDeviceToHost, s);
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  if (e != cudaSuccess) return fail_cuda(e, "checking the mask");
  *is_causal = host == 0 ? 1 : 0;
  return ACCT_OK;
}

uint8_t* acct_mask_tiles_scratch(size_t bytes) {
  if (bytes == 0 || bytes > kTilesScratchBytes || device_status_ptr() == nullptr) return nullptr;
  uint8_t* ptr = nullptr;
  if (cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_tiles_scratch) != cudaSuccess) return nullptr;
  return ptr;
}

size_t acct_mask_tiles_bytes(int32_t mask_batch, int32_t S_q, int32_t S_k) {
  if (mask_batch <= 0 || S_q <= 0 || S_k <= 0) return 0;
  return static_cast<size_t>(mask_batch) * ((S_q + kTile - 1) / kTile) * ((S_k + kTile - 1) / kTile);
}

int acct_mask_classify_tiles(const void* mask, int32_t mask_dtype, int32_t mask_batch, int32_t S_q, int32_t S_k,
                             uint8_t* tiles, void* stream) {
  if (mask == nullptr || tiles == nullptr) return fail(ACCT_ERR_NULL, "acct_mask_classify_tiles: NULL argument");
  if (mask_dtype != ACCT_F16 && mask_dtype != ACCT_BF16 && mask_dtype != ACCT_U8)
    return fail(ACCT_ERR_DTYPE, "attn_mask dtype must be F16, BF16 or U8");
  if (mask_batch <= 0 || S_q <= 0 || S_k <= 0) return fail(ACCT_ERR_SHAPE, "mask_batch, S_q, S_k must be positive");
  if (mask_batch > 65535 || (S_q + kTile - 1) / kTile > 65535)
    return fail(ACCT_ERR_SHAPE, "mask_batch and S_q / 128 must not exceed 65535");
  if (device_status_ptr() == nullptr) return ACCT_ERR_NO_DEVICE;
  cudaError_t e = launch_mask_classify(mask, mask_dtype, mask_batch, S_q, S_k, tiles, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return fail_cuda(e, "launching the mask classification kernel");
  return ACCT_OK;
}

int acct_fa_fwd(const acct_fa_args* a, void* stream) {
  Strides st;
  int rc = validate_fa(a, &st);
  if (rc) return rc;
  unsigned int* status = device_status_ptr();
  if (status == nullptr) return ACCT_ERR_NO_DEVICE;
  FwdParams p;
  memset(&p, 0, sizeof(p));
  if ((rc = make_qkv_maps(a, st, &p.map_q, &p.map_k, &p.map_v))) return rc;
  {
    TensorDesc4 t;
    t.dtype = a->dtype; t.ptr = a->o;
    t.dims[0] = a->D; t.dims[1] = a->S_q; t.dims[2] = a->N; t.dims[3] = a->B;
    t.strides[0] = st.o[2]; t.strides[1] = st.o[1]; t.strides[2] = st.o[0];
    if ((rc = make_tmap_4d(&p.map_o, t, kTile))) return rc;
  }
  p.o = a->o;
  p.lse = a->lse;
  p.o_stride_b = st.o[0]; p.o_stride_h = st.o[1]; p.o_stride_s = st.o[2];
  p.B = a->B; p.N = a->N; p.S_q = a->S_q; p.S_k = a->S_k; p.D = a->D;
  p.kv_group = a->N / kv_heads(a);
  p.scale_log2 = a->scale * kLog2e;
  p.mods = make_mods(a);
  p.status = status;
  cudaError_t e = launch_fa_fwd(p, a->dtype == ACCT_BF16, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return fail_cuda(e, "launching the forward kernel");
  return ACCT_OK;
}

size_t acct_fa_bwd_workspace_bytes(const acct_fa_args* a) {
  if (a == nullptr || a->B <= 0 || a->N <= 0 || a->S_q <= 0 || a->D <= 0) return 0;
  const size_t rows = static_cast<size_t>(a->B) * a->N * a->S_q;
  // (two counters per Q tile above head_dim 128, where two CTAs share a K/V tile by halves of head_dim)
  const size_t q_tiles = static_cast<size_t>(a->B) * a->N * ((a->S_q + kTile - 1) / kTile) * (a->D > 128 ? 2 : 1) + 1;
  // (+ 1: the work counter of the persistent thread blocks)
  // delta [rows] fp32 | turn counters of the ordered dQ reduction [B*N*ceil(S_q/128)] u32 | dQ accumulator
  // [rows, D] fp32; the first two padded to 256 bytes.  With fp32 gradients dq itself is the accumulator.
  const size_t acc = (a->flags & ACCT_FLAG_GRAD_F32) ? 0 : rows * static_cast<size_t>(a->D) * 4;
  return ((rows * 4 + 255) / 256) * 256 + ((q_tiles * 4 + 255) / 256) * 256 + acc;
}

int acct_fa_bwd(const acct_fa_args* a, const acct_fa_bwd_io* g, void* stream) {
  Strides st;
  int rc = validate_fa(a, &st, true);
  if (rc) return rc;
  if (g == nullptr) return fail(ACCT_ERR_NULL, "backward io is NULL");
  if (!g->d_o || !g->dq || !g->dk || !g->dv || !a->lse) return fail(ACCT_ERR_NULL, "d_o, dq, dk, dv and lse must be non-NULL");
  if (!aligned16(g->d_o) || !aligned16(g->dq) || !aligned16(g->dk) || !aligned16(g->dv))
    return fail(ACCT_ERR_ALIGN, "d_o, dq, dk, dv must be 16-byte aligned");
  const size_t need = acct_fa_bwd_workspace_bytes(a);
  if (g->workspace == nullptr || g->workspace_bytes < need)
    return fail(ACCT_ERR_WORKSPACE, "backward workspace: need %zu bytes, got %zu", need, g->workspace ? g->workspace_bytes : (size_t)0);
  if ((reinterpret_cast<uintptr_t>(g->workspace) & 255u) != 0) return fail(ACCT_ERR_ALIGN, "workspace must be 256-byte aligned");
  unsigned int* status = device_status_ptr();
  if (status == nullptr) return ACCT_ERR_NO_DEVICE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool bf16 = a->dtype == ACCT_BF16;
  const size_t rows = static_cast<size_t>(a->B) * a->N * a->S_q;
  float* delta = static_cast<float*>(g->workspace);
  const bool wide = a->D > 128;      // the split-width kernel: 64-row Q / dO boxes, 64-row dQ box, 2 counters per tile
  const size_t q_tiles = static_cast<size_t>(a->B) * a->N * ((a->S_q + kTile - 1) / kTile) * (wide ? 2 : 1) + 1;   // + work counter
  const size_t order_bytes = ((q_tiles * 4 + 255) / 256) * 256;
  unsigned int* dq_order = reinterpret_cast<unsigned int*>(static_cast<uint8_t*>(g->workspace) + ((rows * 4 + 255) / 256) * 256);
  // fp32 gradients: the kernel's reduce-add lands in the caller's dq directly, no copy afterwards
  const bool dq_in_place = (a->flags & ACCT_FLAG_GRAD_F32) != 0;
  float* dq_acc = dq_in_place ? static_cast<float*>(g->dq)
                              : reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(dq_order) + order_bytes);

  BwdParams p;
  memset(&p, 0, sizeof(p));
  if ((rc = make_qkv_maps(a, st, &p.map_q, &p.map_k, &p.map_v, wide ? 64 : kTile))) return rc;
  TensorDesc4 t;
  t.dtype = a->dtype; t.ptr = g->d_o;
  t.dims[0] = a->D; t.dims[1] = a->S_q; t.dims[2] = a->N; t.dims[3] = a->B;
  t.strides[0] = st.o[2]; t.strides[1] = st.o[1]; t.strides[2] = st.o[0];
  if ((rc = make_tmap_4d(&p.map_do, t, wide ? 64 : kTile))) return rc;
  // the fp32 dQ accumulator, packed [B,N,S_q,D]: target of the kernel's TMA reduce-add
  t.dtype = ACCT_F32; t.ptr = dq_acc;
  t.strides[0] = a->D; t.strides[1] = static_cast<int64_t>(a->S_q) * a->D;
  t.strides[2] = static_cast<int64_t>(a->N) * a->S_q * a->D;
  if ((rc = make_tmap_4d(&p.map_dq, t, wide ? 64 : kTile))) return rc;
  if (!wide && !(a->flags & ACCT_FLAG_GRAD_F32)) {
    // 16-bit dk, dv, packed [B,N_kv,S_k,D]: the kernel writes a tile through shared memory and one TMA store
    const int n_kv = kv_heads(a);
    t.dtype = a->dtype;
    t.dims[0] = a->D; t.dims[1] = a->S_k; t.dims[2] = n_kv; t.dims[3] = a->B;
    t.strides[0] = a->D; t.strides[1] = static_cast<int64_t>(a->S_k) * a->D;
    t.strides[2] = static_cast<int64_t>(n_kv) * a->S_k * a->D;
    t.ptr = g->dk;
    if ((rc = make_tmap_4d(&p.map_dk, t, kTile))) return rc;
    t.ptr = g->dv;
    if ((rc = make_tmap_4d(&p.map_dv, t, kTile))) return rc;
  }

  // one helper pass before the main kernel: row sums, and the zero-fill of the accumulator and the turn counters
  cudaError_t e = launch_bwd_delta(a->o, g->d_o, delta, static_cast<int64_t>(rows), a->D, st.o[0], st.o[1], st.o[2], a->N,
                                   a->S_q, bf16, s, dq_acc, dq_order, static_cast<int64_t>(q_tiles));
  if (e != cudaSuccess) return fail_cuda(e, "launching the row-sum kernel");
  p.lse = a->lse; p.delta = delta; p.dq_acc = dq_acc;
  p.dq_order = (a->flags & ACCT_FLAG_DETERMINISTIC) ? dq_order : nullptr;
  p.dk = g->dk; p.dv = g->dv;
  p.work_counter = dq_order + (q_tiles - 1);
  p.grads_f32 = (a->flags & ACCT_FLAG_GRAD_F32) ? 1 : 0;
  p.B = a->B; p.N = a->N; p.S_q = a->S_q; p.S_k = a->S_k; p.D = a->D;
  p.kv_group = a->N / kv_heads(a);
  p.scale = a->scale; p.scale_log2 = a->scale * kLog2e;
  p.mods = make_mods(a);
  p.status = status;
  if (g->ev_kernel_start != nullptr) {
    e = cudaEventRecord(static_cast<cudaEvent_t>(g->ev_kernel_start), s);
    if (e != cudaSuccess) return fail_cuda(e, "recording the kernel-start event");
  }
  e = wide ? launch_fa_bwd_wide(p, bf16, s) : launch_fa_bwd(p, bf16, s);
  if (e != cudaSuccess) return fail_cuda(e, "launching the backward kernel");
  if (g->ev_kernel_stop != nullptr) {
    e = cudaEventRecord(static_cast<cudaEvent_t>(g->ev_kernel_stop), s);
    if (e != cudaSuccess) return fail_cuda(e, "recording the kernel-stop event");
  }
  if (dq_in_place) return ACCT_OK;
  e = launch_bwd_convert_dq(dq_acc, g->dq, static_cast<int64_t>(rows) * a->D, bf16, false, s);
  if (e != cudaSuccess) return fail_cuda(e, "launching the dQ conversion kernel");
  return ACCT_OK;
}

// The reference's InferShape accepts rank 3 or 4, requires k and v of one shape, q/k/v agreeing on
// batch*heads and head_dim, and bounds every dimension (op_proto/flash_attention_tik.cpp:30-193;
// tbe/impl/flash_attention_fwd.py:34-40,89-119).  Its numeric limits are properties of the Ascend
// kernels; the limits enforced here are this library's own.
int acct_infer_prefill(const acct_infer_args* a, void* stream) {
  if (a == nullptr) return fail(ACCT_ERR_NULL, "args is NULL");
  if (a->rank != 3 && a->rank != 4) return fail(ACCT_ERR_SHAPE, "rank must be 3 or 4, got %d", a->rank);
  if (a->rank == 3 && a->B != 1) return fail(ACCT_ERR_SHAPE, "rank-3 input is [B*N, S, D]: pass B = 1");
  if (!a->y) return fail(ACCT_ERR_NULL, "y is NULL");
  acct_fa_args f;
  memset(&f, 0, sizeof(f));
  f.dtype = a->dtype;
  f.B = a->B; f.N = a->N; f.S_q = a->S_q; f.S_k = a->S_k; f.D = a->D;
  f.q = a->q; f.k = a->k; f.v = a->v; f.o = a->y; f.lse = nullptr;
  f.mask_kind = ACCT_MASK_NONE;
  f.causal = a->causal;
  f.prev_block_num = ACCT_BAND_UNBOUNDED; f.next_block_num = ACCT_BAND_UNBOUNDED;
  f.scale = a->scale;
  f.seq_lens = a->seq_lens;
  f.keep_prob = 1.0f;
  f.N_kv = a->N_kv;
  return acct_fa_fwd(&f, stream);
}

size_t acct_infer_decode_workspace_bytes(const acct_decode_args* a) {
  if (a == nullptr || a->B <= 0 || a->N <= 0 || a->D <= 0) return 0;
  int splits = a->num_splits;
  if (splits <= 0) splits = 64;   // upper bound of what the automatic choice may pick
  return static_cast<size_t>(a->B) * a->N * splits * (static_cast<size_t>(a->D) + 2) * 4;
}

int acct_infer_decode(const acct_decode_args* a, void* stream) {
  if (a == nullptr) return fail(ACCT_ERR_NULL, "args is NULL");
  if (a->dtype != ACCT_F16 && a->dtype != ACCT_BF16) return fail(ACCT_ERR_DTYPE, "dtype must be ACCT_F16 or ACCT_BF16");
  if (a->B <= 0 || a->N <= 0 || a->S_max <= 0) return fail(ACCT_ERR_SHAPE, "B, N, S_max must be positive");
  if (a->D <= 0 || a->D % 8 != 0 || a->D > 256) return fail(ACCT_ERR_UNSUPPORTED_D, "decode head_dim %d must be a multiple of 8 in (0, 256]", a->D);
  if (!a->q || !a->k_cache || !a->v_cache || !a->y) return fail(ACCT_ERR_NULL, "q, k_cache, v_cache, y must be non-NULL");
  if (!aligned16(a->q) || !aligned16(a->k_cache) || !aligned16(a->v_cache) || !aligned16(a->y))
    return fail(ACCT_ERR_ALIGN, "q, k_cache, v_cache, y must be 16-byte aligned");
  if (!(a->scale > 0.f)) return fail(ACCT_ERR_SHAPE, "scale must be positive");
  if (a->N_kv < 0 || (a->N_kv > 0 && a->N % a->N_kv != 0))
    return fail(ACCT_ERR_SHAPE, "N_kv = %d must be 0 or a divisor of N = %d", a->N_kv, a->N);
  const int n_kv = a->N_kv > 0 ? a->N_kv : a->N;
  const int group = a->N / n_kv;
  if (!((a->D <= 128 && group <= 16) || group == 1 || group == 2 || group == 4 || group == 8))
    return fail(ACCT_ERR_SHAPE, "decode takes N / N_kv up to 16 at head_dim <= 128 and in {1, 2, 4, 8} above, got %d at head_dim %d",
                group, a->D);
  int page_shift = 0;
  if (a->block_table != nullptr) {
    if (a->page_size < 16 || (a->page_size & (a->page_size - 1)) != 0)
      return fail(ACCT_ERR_SHAPE, "page_size = %d must be a power of two >= 16", a->page_size);
    if (a->max_pages <= 0 || static_cast<int64_t>(a->max_pages) * a->page_size < a->S_max)
      return fail(ACCT_ERR_SHAPE, "block_table with %d pages of %d rows cannot hold S_max = %d", a->max_pages, a->page_size, a->S_max);
    while ((1 << page_shift) < a->page_size) ++page_shift;
  }
  int64_t kvs[3];
  // paged: the strides are those of a [num_pages, N_kv, page_size, D] pool
  int rc = check_strides("kv", a->kv_stride, a->block_table ? a->page_size : a->S_max, n_kv, a->D, kvs);
  if (rc) return rc;
  int splits = a->num_splits;
  if (splits < 0 || splits > 64) return fail(ACCT_ERR_SHAPE, "num_splits must be in [0, 64]");
  if (static_cast<int64_t>(a->B) * a->N > 65535) return fail(ACCT_ERR_SHAPE, "B*N = %lld exceeds 65535", (long long)a->B * a->N);
  DeviceInfo info;
  if ((rc = device_info(&info))) return rc;
  if (splits == 0) {
    // Automatic choice.  Sequence lengths differ between the sequences of a batch (1 024 .. 16 384 keys in the
    // benchmark configuration), and a (sequence, cache head) slice cut into few parts leaves the SMs unevenly
    // loaded at the end.  Measured on B200 at head_dim 128 with 32 .. 1 024 slices: one query head per cache head is
    // within 2 % of its best with 8 parts per slice for 512 slices or more, rising to 16 parts for 128 slices or
    // fewer (2 parts, the earlier choice at 1 024 slices, was 7-18 % below); grouped heads, whose parts each carry
    // the partial results of the whole group, do best with 8 to 12 parts.  Never parts shorter than 512 keys, and
    // never more parts than the caller's workspace holds.
    const int64_t units = static_cast<int64_t>(a->B) * n_kv;
    const int64_t per_sm = group > 1 ? 4 : 24, most = group > 1 ? 12 : 16;
    int64_t want = (static_cast<int64_t>(info.sm_count) * per_sm + units - 1) / units;
    if (want < 8) want = 8;
    if (want > most) want = most;
    const int64_t cap = (a->S_max + 511) / 512;
    if (want > cap) want = cap;
    const int64_t fit = static_cast<int64_t>(a->workspace_bytes / (static_cast<size_t>(a->B) * a->N * (static_cast<size_t>(a->D) + 2) * 4));
    if (want > fit) want = fit;
    splits = static_cast<int>(want < 1 ? 1 : want);
  }
  const size_t need = static_cast<size_t>(a->B) * a->N * splits * (static_cast<size_t>(a->D) + 2) * 4;
  if (a->workspace == nullptr || a->workspace_bytes < need)
    return fail(ACCT_ERR_WORKSPACE, "decode workspace: need %zu bytes, got %zu", need, a->workspace ? a->workspace_bytes : (size_t)0);
  if (!aligned16(a->workspace)) return fail(ACCT_ERR_ALIGN, "workspace must be 16-byte aligned");
  DecodeParams p;
  p.q = a->q; p.k = a->k_cache; p.v = a->v_cache; p.y = a->y; p.seq_lens = a->seq_lens;
  p.part_acc = static_cast<float*>(a->workspace);
  p.part_ml = p.part_acc + static_cast<size_t>(a->B) * a->N * splits * a->D;
  p.kv_stride_b = kvs[0]; p.kv_stride_h = kvs[1]; p.kv_stride_s = kvs[2];
  p.B = a->B; p.N = a->N; p.S_max = a->S_max; p.D = a->D;
  p.kv_group = group;
  p.block_table = a->block_table; p.page_shift = page_shift; p.max_pages = a->max_pages;
  p.splits = splits;
  p.scale_log2 = a->scale * kLog2e;
  cudaError_t e = launch_decode(p, a->dtype == ACCT_BF16, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return fail_cuda(e, "launching the decode kernels");
  return ACCT_OK;
}

}  // extern "C"
