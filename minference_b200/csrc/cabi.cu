// Library-wide entry points of the C ABI: version string, per-thread error text, and a self-test
// of the bounded device wait every kernel of the library relies on.
#include "common.h"
#include "sm100_ptx.cuh"

namespace minf {
char* last_error_buffer() {
    static thread_local char buf[512] = {0};
    return buf;
}
}  // namespace minf

extern "C" const char* minf_version(void) { return "minfer_b200 0.1 (sm_100a)"; }
extern "C" const char* minf_last_error(void) { return minf::last_error_buffer(); }

namespace minf {
// One CTA waits on an mbarrier that nothing arrives on.  The wait must give up after `limit_ns`,
// raise the CTA's abort flag and let the kernel leave through its normal exit with status bit 0
// set -- the path a protocol fault in the attention or estimator kernels would take.
__global__ void bounded_wait_probe_kernel(unsigned long long limit_ns, int32_t* status) {
    __shared__ unsigned long long never;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&never), 1);
        abort_flag = 0;
        fence_mbar_init();
    }
    __syncthreads();
    const bool ok = mbar_wait_for(smem_u32(&never), 0, &abort_flag, limit_ns);
    __syncthreads();
    if (threadIdx.x == 0 && (!ok || abort_flag)) atomicOr(status + MINF_ST_ERROR, 1);
}
}  // namespace minf

extern "C" int minf_selftest_bounded_wait(int limit_us, int32_t* status, void* stream) {
    if (!status) return minf::fail(MINF_E_ARG, "null pointer argument");
    if (limit_us < 1 || limit_us > 1000000) return minf::fail(MINF_E_ARG, "limit_us must be between 1 and 1000000");
    minf::bounded_wait_probe_kernel<<<1, 64, 0, static_cast<cudaStream_t>(stream)>>>((unsigned long long)limit_us * 1000ull, status);
    MINF_LAUNCH_OK("bounded_wait_probe_kernel");
    return MINF_OK;
}
