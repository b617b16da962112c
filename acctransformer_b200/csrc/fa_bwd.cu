#include "fa_kernels.cuh"
namespace acct {
cudaError_t launch_fa_bwd(const BwdParams&, bool, cudaStream_t) { return cudaErrorNotSupported; }
cudaError_t launch_bwd_delta(const void*, const void*, float*, int64_t, int, int64_t, int64_t, int64_t, int, int, bool, cudaStream_t) { return cudaErrorNotSupported; }
cudaError_t launch_bwd_convert_dq(const float*, void*, int64_t, bool, bool, cudaStream_t) { return cudaErrorNotSupported; }
}
