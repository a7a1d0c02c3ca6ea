// A one-block launch that shows what a bounded wait does when nothing arrives:
// it waits on a barrier that no one signals, for at most `limit_ns`, then
// records its code in the error word and returns.  The launch cannot hang (the
// limit is clamped to one second) and leaves the context usable; the host reads
// the word as it does after any kernel with bounded waits.
#include "common.cuh"
#include "sm100.cuh"

namespace {

constexpr int WAIT_PROBE_CODE = 9;

__global__ void wait_probe_kernel(unsigned long long limit_ns, int* err) {
    __shared__ __align__(8) uint64_t bar;
    rfx::pdl_wait();
    if (threadIdx.x == 0) {
        sm100::mbar_init(&bar, 1);
        sm100::fence_barrier_init();
        if (!sm100::mbar_wait_for(&bar, 0, limit_ns)) atomicExch(err, WAIT_PROBE_CODE);
    }
}

}  // namespace

extern "C" int rfx_wait_probe(long long limit_ns, int* err, void* stream) {
    if (limit_ns < 0 || err == nullptr) return RFX_ERR_BAD_ARG;
    if (limit_ns > 1000000000ll) limit_ns = 1000000000ll;
    wait_probe_kernel<<<1, 32, 0, (cudaStream_t)stream>>>((unsigned long long)limit_ns, err);
    return (int)cudaGetLastError();
}
