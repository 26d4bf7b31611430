// A kernel that does nothing but run out of patience: it proves, on the device, that a bounded wait of
// the TMA/tcgen05 kernels ends by itself when its bytes never arrive.
//
// One block arms a shared-memory barrier for more bytes than anyone sends, waits on it through the same
// mbar_wait the product kernels use (tc_utils.cuh) with the limit it is given, and returns.  The wait
// raises SB_STATUS_TIMEOUT in the status word and sets the block's abort flag, which ends the second
// thread's wait at once; out[0] = 1 when the first wait gave up, out[1] = 1 when the second did, out[2] =
// clock cycles the first wait lasted.  Nothing faults, traps or hangs: the kernel ends in about `limit`
// cycles and the context stays usable.  The reference has no counterpart (its kernels have no waits).
#include "tc_utils.cuh"

__global__ void wait_probe_kernel(int* status, long long* out, long long limit) {
    __shared__ __align__(8) uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        mbar_init(&bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        mbar_expect_tx(&bar, 1024);   // one arrival with 1024 bytes still to come: the phase cannot complete
        const long long t0 = clock64();
        const bool ok = mbar_wait(&bar, 0, &abort_flag, status, limit);
        out[0] = ok ? 0 : 1;
        out[2] = clock64() - t0;
    } else if (threadIdx.x == 32) {
        // waits far longer on its own; the first thread's time-out must end it through the flag
        const bool ok = mbar_wait<true>(&bar, 0, &abort_flag, status, SB_WAIT_LIMIT);
        out[1] = ok ? 0 : 1;
    }
}

extern "C" int sb_wait_probe(int* status, long long* out, long long limit_cycles, cudaStream_t stream) {
    if (limit_cycles < 0 || limit_cycles > (1ll << 28)) return (int)cudaErrorInvalidValue;   // a probe stays short
    wait_probe_kernel<<<1, 64, 0, stream>>>(status, out, limit_cycles);
    SB_LAUNCH_CHECK();
}
