// Self-test of the failure path every tensor-core kernel of this library shares: a bounded
// mbarrier wait (tc::mbar_wait) that runs out.  The kernel below waits on a barrier nobody
// arrives at, with a caller-chosen limit; the wait gives up, the kernel records which wait it
// was in the GPU's status word and returns by itself -- no trap, no endless loop, the context
// stays usable.  The host side then sees exactly what it sees after a production kernel gave
// up: PARAS_E_TIMEOUT from the next status check, reported once.
#include "common.cuh"
#include "tc_prims.cuh"

namespace pb {
namespace {

constexpr int kSelftestTag = 27;  // bit of the status word this wait reports

__global__ void bounded_wait_selftest_kernel(int* status, uint64_t limit_ns) {
    __shared__ __align__(8) uint64_t barrier_word;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        tc::mbar_init(tc::smem_u32(&barrier_word), 1);
        tc::mbar_fence_init();
    }
    __syncthreads();
    bool ok = true;
    if (threadIdx.x == 0)  // phase 0 never completes: there is no arrival
        ok = tc::mbar_wait(tc::smem_u32(&barrier_word), 0, &abort_flag, kSelftestTag, limit_ns);
    __syncthreads();
    if (threadIdx.x == 0 && !ok) {
        *status = abort_flag;
        __threadfence_system();
    }
}

}  // namespace
}  // namespace pb

extern "C" int paras_b200_selftest_bounded_wait(int gpu, uint32_t limit_us, int* status_word) {
    int st;
    pb::Gpu* g = pb::use_gpu(gpu, &st);
    if (!g) return st;
    if (limit_us == 0 || limit_us > 1000000u)
        return pb::fail(PARAS_E_INVALID, "paras selftest: limit must be 1..1000000 microseconds");
    PB_CUDA(cudaStreamSynchronize(g->stream));
    if ((st = pb::check_status_word(g)) != PARAS_OK) return st;  // an earlier, real failure
    pb::bounded_wait_selftest_kernel<<<1, 32, 0, g->stream>>>(g->status_dev, uint64_t(limit_us) * 1000u);
    PB_LAUNCH_CHECK("bounded_wait_selftest_kernel");
    PB_CUDA(cudaStreamSynchronize(g->stream));
    if (status_word) *status_word = *static_cast<volatile int*>(g->status_host);
    return pb::check_status_word(g);  // PARAS_E_TIMEOUT, and the word is cleared
}
