// A probe of the bounded wait that every tcgen05 kernel of this library is built on.
//
// The kernels wait on mbarriers with `tc::mbar_wait`, which gives up after a limit, and then
// `tc::report` a code into a host-visible status word and wind down.  In a healthy run no wait
// ever runs out, so that path would never be exercised.  This probe runs exactly those two
// functions on a barrier at which nothing arrives, with a small limit given by the caller: the
// wait runs out after `limit` polls (microseconds), the code lands in the status word, and the
// kernel returns normally.  Nothing faults, traps or spins without a bound; the context stays
// usable, which the test shows by running ordinary work afterwards.
#include "tcgen05_common.cuh"

namespace {

__global__ void wait_probe_kernel(int* status, uint32_t limit, int code, int arrive_first) {
    __shared__ __align__(8) uint64_t bar;
    const uint32_t b = ri::tc::smem_u32(&bar);
    if (threadIdx.x == 0) {
        ri::tc::mbar_init(b, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        if (arrive_first) ri::tc::mbar_arrive(b);        // the healthy case: the wait succeeds at once
        if (!ri::tc::mbar_wait(b, 0, limit)) ri::tc::report(status, code);
    }
}

}  // namespace

RI_DEFINE_LAST_ERROR()

// Launches one thread that waits (at most `limit` polls, 1 <= limit <= 1,000,000) on a barrier that
// nothing arrives at (or, with arrive_first != 0, that has been arrived at already) and stores
// `code` in *status if the wait ran out.  `status` must be host-visible memory the device can write.
RI_API int ri_wait_probe(int limit, int code, int arrive_first, int* status, cudaStream_t stream) {
    if (limit < 1 || limit > 1000000) return ri::fail("ri_wait_probe: limit %d outside 1..1,000,000", limit);
    if (!status) return ri::fail("ri_wait_probe: no status word");
    wait_probe_kernel<<<1, 32, 0, stream>>>(status, (uint32_t)limit, code, arrive_first);
    return ri::check_launch("ri_wait_probe");
}
