// Self-test entry points for the library's failure reporting. No counterpart in the reference
// (its kernels have no waits that can expire and no status word).
//
// Every kernel of this library bounds its waits and, when one gives up, writes
// {code, role, block, detail} to the caller's status word and returns instead of hanging the GPU.
// The production limit is about two seconds, so nothing can exercise that path cheaply; the
// kernel here has exactly one wait, on an mbarrier that nobody ever arrives at, with the limit
// given by the caller in SM cycles. It lets a test watch the whole chain: wait expires, kernel
// returns normally, host reads the status word. Nothing traps, faults or waits without a limit.
#include "host_common.cuh"
#include "ptx.cuh"

namespace wb {

constexpr int SELFTEST_CODE_WAIT = 7;   // status[0] written by the wait self-test
constexpr int SELFTEST_ROLE = 77;       // status[1]

__global__ void __launch_bounds__(32) selftest_wait_kernel(int* status, long long limit_cycles, int detail) {
    __shared__ __align__(8) unsigned long long bar_mem;
    const uint32_t bar = smem_u32(&bar_mem);
    if (threadIdx.x == 0) {
        mbar_init(bar, 1);  // one arrival expected; none will come
        fence_barrier_init();
    }
    __syncwarp();
    if (threadIdx.x == 0) {
        if (!mbar_wait_limit(bar, 0u, limit_cycles)) {
            if (status != nullptr && atomicCAS(status, 0, SELFTEST_CODE_WAIT) == 0) {
                status[1] = SELFTEST_ROLE;
                status[2] = static_cast<int>(blockIdx.x);
                status[3] = detail;
            }
        }
    }
    __syncwarp();
}

// One thread evaluates the debug-build index check with an index that is out of range. The check
// records the fault and the access it guards (a store to out[index]) is skipped, so the kernel
// touches no memory outside `out` in either build.
__global__ void __launch_bounds__(32) selftest_index_kernel(int* status, int* out, int n, int index) {
    if (threadIdx.x == 0) {
        const bool in_range = index >= 0 && index < n;
        if (in_range && WB_DEBUG_INDEX(in_range, status, 104, index)) out[index] = 1;
        if (!in_range) (void)WB_DEBUG_INDEX(in_range, status, 104, index);
    }
}

}  // namespace wb

extern "C" int wmma_ops_selftest_wait_expiry(long long limit_cycles, int detail, int* status, void* stream) {
    using namespace wb;
    WB_REQUIRE(status != nullptr, WMMA_OPS_ERR_INVALID, "selftest_wait_expiry: status is null");
    WB_REQUIRE(limit_cycles >= 1000 && limit_cycles <= 4000000000ll, WMMA_OPS_ERR_INVALID,
               "selftest_wait_expiry: limit must be between 1e3 and 4e9 cycles (got %lld)", limit_cycles);
    selftest_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(status, limit_cycles, detail);
    WB_CHECK_CUDA(cudaGetLastError());
    return WMMA_OPS_OK;
}

extern "C" int wmma_ops_selftest_debug_index(int index, int n, int* out, int* status, void* stream) {
    using namespace wb;
    WB_REQUIRE(status != nullptr && out != nullptr && n >= 1, WMMA_OPS_ERR_INVALID,
               "selftest_debug_index: null pointer or empty buffer");
    selftest_index_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(status, out, n, index);
    WB_CHECK_CUDA(cudaGetLastError());
    return WMMA_OPS_OK;
}

extern "C" int wmma_ops_debug_checks_enabled(void) {
#ifdef WMMA_OPS_DEBUG_CHECKS
    return 1;
#else
    return 0;
#endif
}
