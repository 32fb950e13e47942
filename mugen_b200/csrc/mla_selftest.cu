// Self-test of the bounded-wait path: a one-block kernel whose threads wait on an mbarrier that
// nothing will ever complete.  It exercises, on purpose and in isolation, what every tcgen05 kernel
// of this library does when a wait runs out (a lost TMA completion, a twin block that never
// signals): the waiter gives up after `limit_cycles`, raises ST_WAIT_TIMEOUT in the status word,
// tells the rest of the block through the abort flag, the block frees the tensor memory it holds
// and returns normally.  The context stays usable; the host sees the failure through mla_status.
// The product kernels' own barriers are never starved to test this.
#include "../../include/mugen_mla.h"
#include "mla_launch.h"
#include "mla_tc5.cuh"

namespace mla {

namespace {

using namespace tc5;

__global__ void __launch_bounds__(128)
wait_timeout_selftest_kernel(long long limit_cycles, uint32_t* __restrict__ status, uint32_t* __restrict__ report)
{
    __shared__ __align__(8) uint64_t bar_storage;
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;
    const uint32_t bar = smem_u32(&bar_storage);
    const uint32_t tid = threadIdx.x, warp = tid / 32;
    if (tid == 0) {
        abort_flag = 0;
        mbar_init(bar, 1);                 // one arrival expected; none will come
        mbar_init_fence();
    }
    if (warp == 0) tc_alloc<32>(&tmem_slot);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_slot;

    // warp 1 sleeps in the barrier unit, the others poll: both flavours of the wait must give up
    const long long t0 = clock64();
    const bool ok = warp == 1 ? mbar_wait<kSleep>(bar, 0, &abort_flag, status, limit_cycles)
                              : mbar_wait<kPoll>(bar, 0, &abort_flag, status, limit_cycles);
    const long long waited = clock64() - t0;

    tc_fence_before();
    __syncthreads();
    if (warp == 0) {                       // what the block holds is given back on the failure path too
        tc_fence_after();
        tc_dealloc<32>(tmem);
    }
    if (tid == 0) {
        report[0] = ok ? 1u : 0u;          // 0: the wait gave up, as it must
        report[1] = uint32_t(waited > 0x7fffffffLL ? 0x7fffffffLL : waited);
    }
}

}  // namespace

void launch_wait_timeout_selftest(long long limit_cycles, uint32_t* status, uint32_t* report, cudaStream_t st)
{
    wait_timeout_selftest_kernel<<<1, 128, 0, st>>>(limit_cycles, status, report);
}

}  // namespace mla
