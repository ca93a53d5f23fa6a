// Self-test of the bounded device waits.  Every mbarrier wait in this library gives up after a time
// limit, records a code in StepCounters::error and lets its kernel drain, so a lost signal becomes a
// host-side error instead of a hung GPU (the reference's waits spin without a limit,
// cuda/pipeline.cuh:24-25,32-33).  This kernel makes one such wait run out on purpose in the only
// harmless way: one CTA, a barrier that nothing ever arms, no copy or tensor-core operation in
// flight, a limit of about a millisecond.
#include "sm100.cuh"

using namespace sm100;

namespace {
__global__ void __launch_bounds__(32) starved_wait_kernel(StepCounters *counters, unsigned long long limit_ns,
                                                          int code, int *gave_up) {
    __shared__ uint64_t barrier;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        mbarrier_init(smem_address(&barrier), 1);
        abort_flag = 0;
        fence_barrier_init();
    }
    __syncwarp();
    if (threadIdx.x == 0) {
        const bool completed = mbarrier_wait(smem_address(&barrier), 0, &abort_flag, counters, code, limit_ns);
        *gave_up = completed ? 0 : 1;
    }
}
} // namespace

// Returns 1 when the wait gave up (the expected outcome), 0 when it reported completion.
int launch_starved_wait(StepCounters *counters, double limit_ms, int code, cudaStream_t s) {
    if (!(limit_ms > 0.0) || limit_ms > 100.0)
        throw std::runtime_error("wait limit must be in (0, 100] milliseconds");
    int *flag = nullptr;
    CHECK_CUDA(cudaMallocAsync(&flag, sizeof(int), s));
    starved_wait_kernel<<<1, 32, 0, s>>>(counters, (unsigned long long)(limit_ms * 1e6), code, flag);
    CHECK_CUDA(cudaGetLastError());
    int host = -1;
    CHECK_CUDA(cudaMemcpyAsync(&host, flag, sizeof(int), cudaMemcpyDeviceToHost, s));
    CHECK_CUDA(cudaStreamSynchronize(s));
    CHECK_CUDA(cudaFreeAsync(flag, s));
    return host;
}
