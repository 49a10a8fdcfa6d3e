// All-reduce (sum) of an fp16 buffer that every rank holds in symmetric memory, done through the
// NVSwitch: one launch per rank, no staging copies.
//
// The sharded layer's row-parallel GEMMs end in the project's only exchange step, the sum of the
// ranks' partial outputs (the reference is single-GPU and has none). Each rank writes its partial
// product straight into a buffer that is mapped on all ranks and bound to an NVLink multicast
// object. Rank r then owns the r-th slice of the buffer:
//   multimem.ld_reduce  reads the slice from all ranks at once; the switch adds the eight copies
//                       (fp32 accumulation) and delivers one 16-byte result,
//   multimem.st         writes the sum back to all ranks' copies.
// Per GPU the links carry the buffer once out and once in, which is the two-shot minimum; the
// ring all-reduce of a communication library moves the same bytes in 2 (n - 1) latency-bound steps.
//
// The caller synchronises the ranks before (all partial products written) and after (all slices
// stored) with the symmetric-memory barrier; this kernel itself waits on nobody.
#include <cuda_runtime.h>

#include "host_common.cuh"

namespace wb {

__device__ __forceinline__ uint4 multimem_ld_reduce_f16(const uint4* p) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p)
                 : "memory");
    return v;
}

__device__ __forceinline__ void multimem_st(uint4* p, const uint4& v) {
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z),
                 "r"(v.w)
                 : "memory");
}

constexpr int AR_UNROLL = 8;  // reductions in flight per thread: a trip through the switch takes microseconds

__global__ void __launch_bounds__(512) multimem_allreduce_f16_kernel(uint4* mc, size_t first_vec, size_t n_vec) {
    // mc: multicast address of the buffer; this rank reduces the 16-byte vectors [first_vec, first_vec + n_vec)
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    uint4* base = mc + first_vec;
    size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    for (; i + (AR_UNROLL - 1) * stride < n_vec; i += AR_UNROLL * stride) {
        uint4 v[AR_UNROLL];
#pragma unroll
        for (int u = 0; u < AR_UNROLL; ++u) v[u] = multimem_ld_reduce_f16(base + i + u * stride);
#pragma unroll
        for (int u = 0; u < AR_UNROLL; ++u) multimem_st(base + i + u * stride, v[u]);
    }
    for (; i < n_vec; i += stride) multimem_st(base + i, multimem_ld_reduce_f16(base + i));
    __threadfence_system();
}

}  // namespace wb

extern "C" int wmma_ops_multimem_allreduce_f16(void* multicast_ptr, size_t n_halves, int rank, int world,
                                               int max_ctas, void* stream) {
    using namespace wb;
    WB_REQUIRE(multicast_ptr != nullptr, WMMA_OPS_ERR_INVALID, "multimem_allreduce: null multicast pointer");
    WB_REQUIRE(world >= 1 && rank >= 0 && rank < world, WMMA_OPS_ERR_INVALID,
               "multimem_allreduce: rank %d out of range for world size %d", rank, world);
    WB_REQUIRE(reinterpret_cast<uintptr_t>(multicast_ptr) % 16 == 0 && n_halves % 8 == 0, WMMA_OPS_ERR_INVALID,
               "multimem_allreduce: the buffer must be 16-byte aligned and a multiple of 8 halves long");
    const size_t total_vec = n_halves / 8;
    // slices in 16-byte vectors, as even as they can be
    const size_t base = total_vec / world, extra = total_vec % world;
    const size_t first = static_cast<size_t>(rank) * base + (static_cast<size_t>(rank) < extra ? rank : extra);
    const size_t n_vec = base + (static_cast<size_t>(rank) < extra ? 1 : 0);
    if (n_vec == 0) return WMMA_OPS_OK;
    int ctas = max_ctas > 0 ? max_ctas : sm_count();
    const size_t want = (n_vec + 511) / 512;
    if (static_cast<size_t>(ctas) > want) ctas = static_cast<int>(want);
    multimem_allreduce_f16_kernel<<<ctas, 512, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<uint4*>(multicast_ptr), first, n_vec);
    WB_CHECK_CUDA(cudaGetLastError());
    return WMMA_OPS_OK;
}
