// convnn_b200_selftest_wait_timeout: lets a test watch the bounded mbarrier wait of the
// tensor-core kernels give up, without putting any copy, MMA or second CTA at risk.  The
// kernel is one CTA; thread 0 waits on a barrier that expects one arrival which never comes.
#include "common.cuh"
#include "sm100.cuh"

namespace convnn {
namespace {

__global__ void wait_timeout_kernel(int* status, unsigned long long* waited_ns, unsigned long long budget_ns) {
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        sm100::mbar_init(&bar, 1);
        abort_flag = 0;
        sm100::fence_barrier_init();
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned long long t0 = sm100::global_timer_ns();
        const bool ok = sm100::mbar_wait(&bar, 0, &abort_flag, budget_ns);
        *waited_ns = sm100::global_timer_ns() - t0;
        *status = ok ? 0 : 41;
    }
}

}  // namespace
}  // namespace convnn

extern "C" int convnn_b200_selftest_wait_timeout(uint32_t budget_us, int* status_dev, uint64_t* waited_ns_dev,
                                                 void* stream) {
    using namespace convnn;
    if (!status_dev || !waited_ns_dev)
        return set_error(CONVNN_E_NULL, "convnn_b200_selftest_wait_timeout: NULL output pointer");
    if (budget_us < 1 || budget_us > 100000)
        return set_error(CONVNN_E_INVALID, "convnn_b200_selftest_wait_timeout: budget_us must be in 1 .. 100000");
    wait_timeout_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(
        status_dev, reinterpret_cast<unsigned long long*>(waited_ns_dev), (unsigned long long)budget_us * 1000ull);
    CONVNN_CHECK_LAUNCH("selftest_wait_timeout");
    return CONVNN_OK;
}
