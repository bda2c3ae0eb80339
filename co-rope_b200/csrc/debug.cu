// Diagnostics declared in include/corope_b200_debug.h that need a kernel of their own.
#include "common.cuh"
#include "../../include/corope_b200_debug.h"

namespace corope {
namespace {

// One warp waits on a barrier that expects one arrival and never gets it, with the same bounded-wait helper the production
// kernels use (only the poll limit differs), then leaves through the normal exit.
__global__ void expire_wait_kernel(int* status, unsigned max_polls) {
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        mbar_init(&bar, 1);
        fence_mbar_init();
    }
    __syncthreads();
    const bool ok = mbar_wait_limited(&bar, 0, status, 0x7e, &abort_flag, max_polls);
    (void)ok;   // false: the phase never completes
}

}  // namespace
}  // namespace corope

extern "C" int corope_debug_expire_wait(int* status_word, unsigned max_polls, void* stream) {
    if (max_polls == 0 || max_polls > (1u << 16)) max_polls = 1u << 10;
    corope::expire_wait_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(status_word, max_polls);
    corope::count_launch();
    return (int)cudaGetLastError();
}

extern "C" int corope_debug_synth_tables(const float* inv_freq, float* cos_out, float* sin_out, int N, int half_d, void* stream) {
    if (!inv_freq || !cos_out || !sin_out || N <= 0 || half_d <= 0) return COROPE_ERR_NULL_POINTER;
    return corope::launch_synth_tables(inv_freq, cos_out, sin_out, N, half_d, (cudaStream_t)stream);
}
