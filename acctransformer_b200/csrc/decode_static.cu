// acct_infer_decode_static: the decode step for callers that cannot allocate device memory.
//
// Some hosts of this library have no way to call cudaMalloc at the moment they need a decode step:
// a serving loop whose memory pool was carved up at start-up and is now full, a plugin running inside
// a framework that forbids allocation while it records or replays a step, a real-time thread that
// must not take the allocator's lock.  The regular entry point makes them bring a workspace for the
// per-split partial results; this variant keeps that scratch inside the library instead, in a
// fixed-size array that is part of the loaded module.
//
// Cost and limits, stated plainly:
//   * the array occupies ACCT_DECODE_STATIC_SCRATCH_BYTES (8 MiB) on every GPU that loads the library,
//     from load until the process exits, whether or not this entry point is ever called;
//   * a call whose partial results do not fit is refused with ACCT_ERR_WORKSPACE (use fewer splits, or
//     the regular entry point with a workspace of your own);
//   * all calls on one GPU share the one array.  Nothing in it has to start at zero -- every slot that
//     the merge kernel reads is first written by the split kernel of the same call -- so left-over
//     contents of an earlier call are harmless, but two calls that overlap on the GPU (different
//     streams, or different host threads without ordering) overwrite each other's partial results
//     and race.  Order them on one stream.
//   * the first call on each GPU looks up the array's device address (cudaGetSymbolAddress) with that
//     GPU current.  That first call should therefore happen before any stream capture begins.
// No cudaMalloc, cudaFree or allocating library routine is called from here.
#include <mutex>

#include "common.cuh"

namespace acct {
namespace {

// Inside host code this name is only a handle for the runtime, not a device address: handing it to
// a kernel would make the kernel read whatever host memory the handle happens to be.  The address a
// kernel may use comes from cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_decode_static_scratch[ACCT_DECODE_STATIC_SCRATCH_BYTES];

constexpr int kMaxDevicesStatic = 64;
std::mutex g_static_mutex;
void* g_static_ptr[kMaxDevicesStatic] = {nullptr};

// Device address of the scratch array on the current device (looked up once per device).
int static_scratch_address(void** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(ACCT_ERR_NO_DEVICE, "no CUDA device: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevicesStatic) return fail(ACCT_ERR_NO_DEVICE, "device index %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_static_mutex);
  if (g_static_ptr[dev] == nullptr) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_decode_static_scratch);
    if (e != cudaSuccess) return fail_cuda(e, "cudaGetSymbolAddress(static decode scratch)");
    if (ptr == nullptr) return fail(ACCT_ERR_CUDA, "static decode scratch has no device address");
    g_static_ptr[dev] = ptr;
  }
  *out = g_static_ptr[dev];
  return 0;
}

}  // namespace
}  // namespace acct

using namespace acct;

extern "C" ACCT_API int acct_infer_decode_static(const acct_decode_args* a, void* stream) {
  if (a == nullptr) return fail(ACCT_ERR_NULL, "args is NULL");
  void* scratch = nullptr;
  int rc = static_scratch_address(&scratch);
  if (rc) return rc;
  acct_decode_args with_scratch = *a;          // the caller's workspace fields are ignored
  with_scratch.workspace = scratch;
  with_scratch.workspace_bytes = ACCT_DECODE_STATIC_SCRATCH_BYTES;
  rc = acct_infer_decode(&with_scratch, stream);
  if (rc == ACCT_ERR_WORKSPACE) {
    const size_t bound = acct_infer_decode_workspace_bytes(a);
    return fail(ACCT_ERR_WORKSPACE,
                "acct_infer_decode_static: the built-in scratch holds %d bytes and this call needs more "
                "(up to %zu for B=%d N=%d D=%d num_splits=%d); pass a smaller num_splits or use "
                "acct_infer_decode with your own workspace",
                (int)ACCT_DECODE_STATIC_SCRATCH_BYTES, bound, a->B, a->N, a->D, a->num_splits);
  }
  return rc;
}
