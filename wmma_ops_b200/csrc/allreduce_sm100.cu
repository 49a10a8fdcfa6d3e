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
#include <cuda_fp16.h>
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

// ---------------------------------------------------------------------------------------------
// The same sum as one self-contained launch: the two rank barriers that bracket the reduction
// (every rank's partial output is written / every rank's slice is stored everywhere) are made
// inside the kernel with flags in symmetric memory, instead of two extra barrier launches per sum.
// Two input forms: fp16 partials summed in place, or fp32 partials summed into a separate fp16
// buffer (twice the bytes on the way in, no fp16 rounding of the partial outputs).
//
// Flags. Every rank holds, per channel, SW_MAX_CTAS x SW_MAX_WORLD arrival words and SW_MAX_CTAS
// epoch words. CTA b of rank r announces step e by writing e to word [b][r] of every rank's flags
// (peer stores, release at system scope) and waits until its own words [b][0..world) have all
// reached e (acquire loads). The epoch of a CTA lives in device memory and advances by two per
// launch, so nothing is ever reset and a launch replayed from a CUDA graph keeps working. A CTA
// only ever waits for the same CTA of the other ranks; the kernel as a whole completes when all of
// its CTAs have, which is when every rank has stored every part of its slice.
// Every wait is bounded (about a second); on expiry the CTA records {code 5, rank, block, peer} in
// the status word and carries on, so a rank that never arrives costs a wrong result, not a hang.
namespace wb {

constexpr int SW_MAX_CTAS = 128;
constexpr int SW_THREADS = 192;
constexpr int SW_MAX_WORLD = 16;
constexpr int SW_CHANNEL_WORDS = SW_MAX_CTAS * SW_MAX_WORLD + SW_MAX_CTAS;
constexpr int SW_CHANNELS = 4;
constexpr long long SW_WAIT_CYCLES = 2000000000ll;

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ uint4 multimem_ld_reduce_f32(const uint4* p) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p)
                 : "memory");
    return v;
}

__device__ __forceinline__ uint32_t pack_h2(uint32_t a_bits, uint32_t b_bits) {
    const __half2 h = __floats2half2_rn(__uint_as_float(a_bits), __uint_as_float(b_bits));
    return *reinterpret_cast<const uint32_t*>(&h);
}

// Step `e` of CTA blockIdx.x: threads 0..world-1 each tell one peer and wait for that peer.
__device__ __forceinline__ void sw_rank_barrier(uint32_t* const* flag_ptrs, int channel, int rank, int world, uint32_t e,
                                                int* status) {
    __syncthreads();  // this CTA's earlier stores are ordered before the fence of the signalling threads
    const int r = threadIdx.x;
    if (r < world) {
        const size_t word = static_cast<size_t>(channel) * SW_CHANNEL_WORDS + static_cast<size_t>(blockIdx.x) * SW_MAX_WORLD;
        __threadfence_system();
        st_release_sys(flag_ptrs[r] + word + rank, e);
        const uint32_t* mine = flag_ptrs[rank] + word + r;
        const long long t0 = clock64();
        uint32_t spins = 0;
        while (static_cast<int>(ld_acquire_sys(mine) - e) < 0) {
            __nanosleep(64);
            if ((++spins & 0xff) == 0 && clock64() - t0 > SW_WAIT_CYCLES) {
                if (status != nullptr && atomicCAS(status, 0, 5) == 0) {
                    status[1] = rank;
                    status[2] = static_cast<int>(blockIdx.x);
                    status[3] = r;
                }
                break;
            }
        }
    }
    __syncthreads();
}

// F32_IN: partials are fp32 at mc_in and the sums go, as fp16, to mc_out (16 bytes of output per two
// 16-byte input vectors); otherwise fp16 partials at mc_in are summed in place (mc_out == mc_in).
// first / count are in units of 16 bytes of output.
//
// CTAs of SW_THREADS threads at no more than 64 registers: 12 K registers, a few bytes of shared memory. That is
// what the persistent W4A16 prefill kernel leaves free on an SM, so the CTAs of this kernel run beside it on
// SMs that it fills, and a GEMM on another stream need not leave SMs idle for the sum.
template <bool F32_IN>
__global__ void __maxnreg__(64) switch_allreduce_kernel(const uint4* mc_in, uint4* mc_out, size_t first, size_t count,
                                                               uint32_t* const* flag_ptrs, int channel, int rank, int world,
                                                               int* status) {
    __shared__ uint32_t epoch_s;
    uint32_t* epoch_word = flag_ptrs[rank] + static_cast<size_t>(channel) * SW_CHANNEL_WORDS + SW_MAX_CTAS * SW_MAX_WORLD +
                           blockIdx.x;
    if (threadIdx.x == 0) epoch_s = *epoch_word;
    __syncthreads();
    const uint32_t e = epoch_s;
    sw_rank_barrier(flag_ptrs, channel, rank, world, e + 1, status);  // every rank's partial output is written

    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (F32_IN) {
        constexpr int U = AR_UNROLL / 2;
        const uint4* in = mc_in + 2 * first;
        uint4* out = mc_out + first;
        for (; i < count; i += U * stride) {
            uint4 a[U], b[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const size_t k = i + u * stride;
                if (k < count) {
                    a[u] = multimem_ld_reduce_f32(in + 2 * k);
                    b[u] = multimem_ld_reduce_f32(in + 2 * k + 1);
                }
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const size_t k = i + u * stride;
                if (k < count) {
                    uint4 o;
                    o.x = pack_h2(a[u].x, a[u].y);
                    o.y = pack_h2(a[u].z, a[u].w);
                    o.z = pack_h2(b[u].x, b[u].y);
                    o.w = pack_h2(b[u].z, b[u].w);
                    multimem_st(out + k, o);
                }
            }
        }
    } else {
        uint4* base = mc_out + first;
        for (; i < count; i += AR_UNROLL * stride) {
            uint4 v[AR_UNROLL];
#pragma unroll
            for (int u = 0; u < AR_UNROLL; ++u)
                if (i + u * stride < count) v[u] = multimem_ld_reduce_f16(base + i + u * stride);
#pragma unroll
            for (int u = 0; u < AR_UNROLL; ++u)
                if (i + u * stride < count) multimem_st(base + i + u * stride, v[u]);
        }
    }
    sw_rank_barrier(flag_ptrs, channel, rank, world, e + 2, status);  // every rank's slice is stored everywhere
    if (threadIdx.x == 0) *epoch_word = e + 2;
}

// The same sum, following a GEMM of this rank that is still running. The W4A16 kernel can produce its output
// token block by token block and count the finished 128-column tiles of each block in block_done[]; this kernel
// runs beside it on another stream. `parts` CTAs share a token block: each waits (bounded) until its own rank
// has finished the block, meets the same CTA of the other ranks (which have waited for their rank's block), and
// sums its part of this rank's slice of the block through the switch, while the GEMM works on later blocks.
// What remains after the GEMM's last tile is the sum of the last block or two instead of the whole buffer.
// One closing barrier per CTA: every rank's slices are stored everywhere when the kernel completes.
// The counters return to zero for the next product: the last of a block's `parts` CTAs to have seen the block
// complete resets block_done[b] and the arrival count seen[b].
// A CTA of this kernel waits for CTAs of the GEMM, never the other way round, and the GEMM's CTAs must all be
// resident for it to finish its blocks: launch the GEMM first and leave it room (as many SMs free as this kernel
// has CTAs, or the prefill tile, beside which one CTA of this kernel fits on an SM).
template <bool F32_IN>
__global__ void __maxnreg__(64) switch_allreduce_following_kernel(const uint4* mc_in, uint4* mc_out, int n_blocks, int parts,
                                                                  size_t block_vecs, size_t total_vecs, int* block_done,
                                                                  int* seen, int tiles_per_block, uint32_t* const* flag_ptrs,
                                                                  int channel, int rank, int world, int* status) {
    __shared__ uint32_t epoch_s;
    uint32_t* epoch_word = flag_ptrs[rank] + static_cast<size_t>(channel) * SW_CHANNEL_WORDS + SW_MAX_CTAS * SW_MAX_WORLD +
                           blockIdx.x;
    if (threadIdx.x == 0) epoch_s = *epoch_word;
    __syncthreads();
    uint32_t step = epoch_s;
    const int part = static_cast<int>(blockIdx.x) % parts;
    const int groups = static_cast<int>(gridDim.x) / parts;  // token blocks in flight
    for (int b = static_cast<int>(blockIdx.x) / parts; b < n_blocks; b += groups) {
        if (threadIdx.x == 0) {
            const long long t0 = clock64();
            uint32_t spins = 0;
            int have;
            while (true) {
                asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(have) : "l"(block_done + b) : "memory");
                if (have >= tiles_per_block) break;
                __nanosleep(128);
                if ((++spins & 0xff) == 0 && clock64() - t0 > SW_WAIT_CYCLES) {
                    if (status != nullptr && atomicCAS(status, 0, 6) == 0) {
                        status[1] = rank;
                        status[2] = static_cast<int>(blockIdx.x);
                        status[3] = b;
                    }
                    break;
                }
            }
            if (atomicAdd(seen + b, 1) == parts - 1) {  // all of the block's CTAs have seen it complete
                seen[b] = 0;
                block_done[b] = 0;
            }
        }
        ++step;
        sw_rank_barrier(flag_ptrs, channel, rank, world, step, status);  // every rank has finished block b

        // this rank's slice of block b, and this CTA's part of the slice (16-byte units of output)
        const size_t b_first = static_cast<size_t>(b) * block_vecs;
        const size_t b_count = (b_first + block_vecs <= total_vecs) ? block_vecs : total_vecs - b_first;
        const size_t per_rank = b_count / world, extra_r = b_count % world;
        const size_t s_first = b_first + rank * per_rank + (static_cast<size_t>(rank) < extra_r ? rank : extra_r);
        const size_t s_count = per_rank + (static_cast<size_t>(rank) < extra_r ? 1 : 0);
        const size_t per_part = (s_count + parts - 1) / parts;
        const size_t first = s_first + part * per_part;
        const size_t p_end = (part + 1) * per_part < s_count ? (part + 1) * per_part : s_count;
        const size_t count = part * per_part < p_end ? p_end - part * per_part : 0;
        const size_t stride = blockDim.x;
        size_t i = threadIdx.x;
        if (F32_IN) {
            constexpr int U = AR_UNROLL / 2;
            const uint4* in = mc_in + 2 * first;
            uint4* out = mc_out + first;
            for (; i < count; i += U * stride) {
                uint4 a[U], c[U];
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const size_t k = i + u * stride;
                    if (k < count) {
                        a[u] = multimem_ld_reduce_f32(in + 2 * k);
                        c[u] = multimem_ld_reduce_f32(in + 2 * k + 1);
                    }
                }
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const size_t k = i + u * stride;
                    if (k < count) {
                        uint4 o;
                        o.x = pack_h2(a[u].x, a[u].y);
                        o.y = pack_h2(a[u].z, a[u].w);
                        o.z = pack_h2(c[u].x, c[u].y);
                        o.w = pack_h2(c[u].z, c[u].w);
                        multimem_st(out + k, o);
                    }
                }
            }
        } else {
            uint4* base = mc_out + first;
            for (; i < count; i += AR_UNROLL * stride) {
                uint4 v[AR_UNROLL];
#pragma unroll
                for (int u = 0; u < AR_UNROLL; ++u)
                    if (i + u * stride < count) v[u] = multimem_ld_reduce_f16(base + i + u * stride);
#pragma unroll
                for (int u = 0; u < AR_UNROLL; ++u)
                    if (i + u * stride < count) multimem_st(base + i + u * stride, v[u]);
            }
        }
    }
    ++step;
    sw_rank_barrier(flag_ptrs, channel, rank, world, step, status);  // every rank's slices are stored everywhere
    if (threadIdx.x == 0) *epoch_word = step;
}

}  // namespace wb

extern "C" size_t wmma_ops_switch_allreduce_flag_bytes(void) {
    return static_cast<size_t>(wb::SW_CHANNELS) * wb::SW_CHANNEL_WORDS * sizeof(uint32_t);
}

extern "C" int wmma_ops_switch_allreduce(const void* mc_in, void* mc_out, size_t n_values, int in_is_f32, int rank, int world,
                                         const void* flag_ptrs_dev, int channel, int max_ctas, int* status, void* stream) {
    using namespace wb;
    WB_REQUIRE(mc_in != nullptr && mc_out != nullptr && flag_ptrs_dev != nullptr, WMMA_OPS_ERR_INVALID,
               "switch_allreduce: null pointer");
    WB_REQUIRE(world >= 1 && world <= SW_MAX_WORLD && rank >= 0 && rank < world, WMMA_OPS_ERR_INVALID,
               "switch_allreduce: rank %d / world %d out of range (at most %d ranks)", rank, world, SW_MAX_WORLD);
    WB_REQUIRE(channel >= 0 && channel < SW_CHANNELS, WMMA_OPS_ERR_INVALID, "switch_allreduce: channel %d not in 0..%d", channel,
               SW_CHANNELS - 1);
    WB_REQUIRE(reinterpret_cast<uintptr_t>(mc_in) % 16 == 0 && reinterpret_cast<uintptr_t>(mc_out) % 16 == 0 && n_values % 8 == 0,
               WMMA_OPS_ERR_INVALID, "switch_allreduce: buffers must be 16-byte aligned and a multiple of 8 values long");
    WB_REQUIRE(in_is_f32 || mc_in == mc_out, WMMA_OPS_ERR_INVALID, "switch_allreduce: fp16 partials are summed in place");
    const size_t total = n_values / 8;  // 16-byte units of output
    const size_t base = total / world, extra = total % world;
    const size_t first = static_cast<size_t>(rank) * base + (static_cast<size_t>(rank) < extra ? rank : extra);
    const size_t count = base + (static_cast<size_t>(rank) < extra ? 1 : 0);
    // every rank launches the same number of CTAs (they pair up across ranks), also for an empty slice
    int ctas = max_ctas > 0 ? max_ctas : SW_MAX_CTAS;
    if (ctas > SW_MAX_CTAS) ctas = SW_MAX_CTAS;
    const size_t want = (base + 1 + SW_THREADS - 1) / SW_THREADS;
    if (static_cast<size_t>(ctas) > want) ctas = static_cast<int>(want);
    if (ctas < 1) ctas = 1;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    uint32_t* const* flags = static_cast<uint32_t* const*>(flag_ptrs_dev);
    if (in_is_f32)
        switch_allreduce_kernel<true><<<ctas, SW_THREADS, 0, s>>>(static_cast<const uint4*>(mc_in), static_cast<uint4*>(mc_out), first,
                                                           count, flags, channel, rank, world, status);
    else
        switch_allreduce_kernel<false><<<ctas, SW_THREADS, 0, s>>>(static_cast<const uint4*>(mc_in), static_cast<uint4*>(mc_out), first,
                                                            count, flags, channel, rank, world, status);
    WB_CHECK_CUDA(cudaGetLastError());
    return WMMA_OPS_OK;
}

extern "C" int wmma_ops_switch_allreduce_following(const void* mc_in, void* mc_out, int rows, int cols, int in_is_f32,
                                                   int block_rows, int* block_done, int* seen, int tiles_per_block, int rank,
                                                   int world, const void* flag_ptrs_dev, int channel, int max_ctas, int* status,
                                                   void* stream) {
    using namespace wb;
    WB_REQUIRE(mc_in != nullptr && mc_out != nullptr && flag_ptrs_dev != nullptr && block_done != nullptr && seen != nullptr,
               WMMA_OPS_ERR_INVALID, "switch_allreduce_following: null pointer");
    WB_REQUIRE(world >= 1 && world <= SW_MAX_WORLD && rank >= 0 && rank < world, WMMA_OPS_ERR_INVALID,
               "switch_allreduce_following: rank %d / world %d out of range (at most %d ranks)", rank, world, SW_MAX_WORLD);
    WB_REQUIRE(channel >= 0 && channel < SW_CHANNELS, WMMA_OPS_ERR_INVALID, "switch_allreduce_following: channel %d not in 0..%d",
               channel, SW_CHANNELS - 1);
    WB_REQUIRE(rows >= 1 && cols >= 8 && cols % 8 == 0 && block_rows >= 1 && tiles_per_block >= 1, WMMA_OPS_ERR_INVALID,
               "switch_allreduce_following: rows %d, cols %d (a multiple of 8), block_rows %d, tiles_per_block %d", rows, cols,
               block_rows, tiles_per_block);
    WB_REQUIRE(reinterpret_cast<uintptr_t>(mc_in) % 16 == 0 && reinterpret_cast<uintptr_t>(mc_out) % 16 == 0,
               WMMA_OPS_ERR_INVALID, "switch_allreduce_following: buffers must be 16-byte aligned");
    WB_REQUIRE(in_is_f32 || mc_in == mc_out, WMMA_OPS_ERR_INVALID, "switch_allreduce_following: fp16 partials are summed in place");
    const int n_blocks = (rows + block_rows - 1) / block_rows;
    const size_t row_vecs = static_cast<size_t>(cols) / 8;
    int ctas = max_ctas > 0 ? max_ctas : 32;
    if (ctas > SW_MAX_CTAS) ctas = SW_MAX_CTAS;
    // whole groups of `parts` CTAs per token block: up to 8 CTAs share a block when there are few blocks
    int parts = ctas / n_blocks;
    parts = parts < 1 ? 1 : parts > 8 ? 8 : parts;
    int groups = ctas / parts;
    if (groups > n_blocks) groups = n_blocks;
    ctas = groups * parts;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    uint32_t* const* flags = static_cast<uint32_t* const*>(flag_ptrs_dev);
    if (in_is_f32)
        switch_allreduce_following_kernel<true><<<ctas, SW_THREADS, 0, s>>>(
            static_cast<const uint4*>(mc_in), static_cast<uint4*>(mc_out), n_blocks, parts, block_rows * row_vecs,
            rows * row_vecs, block_done, seen, tiles_per_block, flags, channel, rank, world, status);
    else
        switch_allreduce_following_kernel<false><<<ctas, SW_THREADS, 0, s>>>(
            static_cast<const uint4*>(mc_in), static_cast<uint4*>(mc_out), n_blocks, parts, block_rows * row_vecs,
            rows * row_vecs, block_done, seen, tiles_per_block, flags, channel, rank, world, status);
    WB_CHECK_CUDA(cudaGetLastError());
    return WMMA_OPS_OK;
}
