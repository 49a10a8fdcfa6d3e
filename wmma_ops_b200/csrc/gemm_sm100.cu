// FP16 x FP16 -> FP32 GEMM for sm_100a: persistent, warp-specialised, tcgen05 MMA with
// TMEM accumulators, TMA-fed shared-memory ring, fused alpha/beta epilogue, split-K.
//
// One kernel family takes the place of the reference's GEMM kernels
// (wmma_gemm.hip:45-233 main kernel, :475-667 alpha/beta kernel, :697-877 adaptive kernel,
// wmma_kernel_variants.hpp:28-193 K-unrolled kernel, wmma_kernel_largetile.hpp:169-293,
// wmma_kernels_pingpong.hpp:25-211, wmma_xor_swizzle.hpp:690-844 split-K kernel and
// :334-353 reduce kernel).
//
// Layouts (the reference's): A [M,K] fp16 row-major, B [K,N] fp16 row-major, C [M,N] fp32.
//   A tiles are K-major operands (128 rows x 64 halves = 128-byte rows, SWIZZLE_128B).
//   B tiles are MN-major operands: each TMA box is 64 K-rows x 64 N-halves, so the
//   reference's global->LDS transpose of B (wmma_device_helpers.hpp:90-172) has no
//   counterpart here; the MMA reads B with N contiguous.
//
// Warp roles per CTA (192 threads): warp 0 = TMA producer, warp 1 = TMEM owner + MMA issuer,
// warps 2..5 = epilogue (TMEM -> registers -> alpha*acc + beta*C_in -> global).
// Two TMEM accumulators let the epilogue of one tile overlap the main loop of the next.
#include <mutex>
#include <vector>

#include "host_common.cuh"
#include "ptx.cuh"

namespace wb {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int GEMM_THREADS = 192;
#ifndef WB_RASTER_GROUP_M
#define WB_RASTER_GROUP_M 16
#endif
constexpr int RASTER_GROUP_M = WB_RASTER_GROUP_M;  // m-blocks walked together so a wave reuses A and B in L2

// Epilogue staging. A thread of an epilogue warp holds 32 consecutive columns of ONE output row (its TMEM
// lane); stored directly, each of the warp's 16-byte stores goes to a different line. The warp therefore turns
// its 32 x 32 block through shared memory (rows of 144 bytes: the 16 extra bytes make both the row-wise
// writes and the four-rows-at-a-time reads conflict-free) and writes four full 128-byte row segments per
// instruction. Measured at 8192^3: 1177 -> 1188 TFLOP/s sustained; at 1024^3 the pair tile gains 20 %.
constexpr int EPI_PITCH = 144;
constexpr int EPI_BYTES = 4 * 32 * EPI_PITCH;  // four epilogue warps

// r: this thread's 32 accumulators (row row_w + lane, columns col0 .. col0 + 31). in_row: this thread's row of
// C_in, or null. out: C (or the split-K slice). streaming: final outputs leave with st.cs, partial sums stay.
__device__ __forceinline__ void epilogue_store_block(uint32_t wbase, const uint32_t (&r)[32], float alpha, float beta,
                                                     const float* in_row, bool row_ok, float* out, int row_w, int col0,
                                                     int M, int N, bool streaming, int* status) {
    const int lane = threadIdx.x & 31;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        float4 v;
        v.x = alpha * __uint_as_float(r[4 * j + 0]);
        v.y = alpha * __uint_as_float(r[4 * j + 1]);
        v.z = alpha * __uint_as_float(r[4 * j + 2]);
        v.w = alpha * __uint_as_float(r[4 * j + 3]);
        if (in_row != nullptr && row_ok && col0 + j * 4 < N) {
            const float4 cin = *reinterpret_cast<const float4*>(in_row + col0 + j * 4);
            v.x += beta * cin.x;
            v.y += beta * cin.y;
            v.z += beta * cin.z;
            v.w += beta * cin.w;
        }
        asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(wbase + lane * EPI_PITCH + j * 16), "f"(v.x), "f"(v.y),
                     "f"(v.z), "f"(v.w)
                     : "memory");
    }
    __syncwarp();  // also orders every lane's reads of C_in before the stores below (C_in may be C_out)
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int rr = i * 4 + (lane >> 3);
        const int cc = (lane & 7) * 4;
        float4 v;
        asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
                     : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                     : "r"(wbase + rr * EPI_PITCH + cc * 4)
                     : "memory");
        const int row = row_w + rr;
        const int col = col0 + cc;
        if (row < M && col < N && WB_DEBUG_INDEX(row >= 0 && col >= 0 && col + 4 <= N, status, 100, col)) {
            float4* dst = reinterpret_cast<float4*>(out + static_cast<size_t>(row) * N + col);
            if (streaming) __stcs(dst, v);
            else *dst = v;
        }
    }
    __syncwarp();  // the block is rewritten for the next 32 columns
}

template <int BN>
struct GemmCfg {
    static constexpr int A_BYTES = BM * BK * 2;
    static constexpr int B_BOX_BYTES = BK * 64 * 2;  // one 64(k) x 64(n) box
    static constexpr int B_BYTES = (BN / 64) * B_BOX_BYTES;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int STAGES = (BN == 256) ? 4 : (BN == 128) ? 6 : 8;
    static constexpr int TMEM_COLS = 2 * BN;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/ + EPI_BYTES;
};

struct GemmParams {
    const float* C_in;  // may alias C_out, may be null
    float* C_out;       // [M,N] or, with split_k > 1, the partials [split_k][M][N]
    int M, N, K;
    int m_blocks, n_blocks;
    int split_k;        // >= 1
    int kb_total;       // ceil(K / 64)
    int kb_per_split;   // k-blocks per slice
    float alpha, beta;
    int* status;        // optional device status word
};

__device__ __forceinline__ void report_timeout(int* status, int role, int detail) {
    if (status != nullptr && atomicCAS(status, 0, 1) == 0) {
        status[1] = role;
        status[2] = static_cast<int>(blockIdx.x);
        status[3] = detail;
    }
}

// Work unit -> (m block, n block, k slice). Tiles are walked in groups of RASTER_GROUP_M
// m-blocks, m fastest, which plays the role of the reference's tile rasterisation
// (wmma_xor_swizzle.hpp:171-278, wmma_tile_mapping.hpp:35-434).
__device__ __forceinline__ void decode_unit(const GemmParams& p, int unit, int& mb, int& nb,
                                            int& ks) {
    const int tiles = p.m_blocks * p.n_blocks;
    ks = unit / tiles;
    const int t = unit - ks * tiles;
    const int group_span = RASTER_GROUP_M * p.n_blocks;
    const int g = t / group_span;
    const int first_m = g * RASTER_GROUP_M;
    const int rows = min(RASTER_GROUP_M, p.m_blocks - first_m);
    const int r = t - g * group_span;
    mb = first_m + r % rows;
    nb = r / rows;
}

template <int BN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_f16f32_kernel(const __grid_constant__ CUtensorMap tmap_a,
                   const __grid_constant__ CUtensorMap tmap_b, const GemmParams p) {
    using Cfg = GemmCfg<BN>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t bar_base = smem_base + Cfg::STAGES * Cfg::STAGE_BYTES;
    // barrier slots (8 bytes each): full[STAGES], empty[STAGES], acc_full[2], acc_empty[2], tmem ptr
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (Cfg::STAGES + s); };
    auto acc_full_bar = [&](int b) { return bar_base + 8u * (2 * Cfg::STAGES + b); };
    auto acc_empty_bar = [&](int b) { return bar_base + 8u * (2 * Cfg::STAGES + 2 + b); };
    const uint32_t tmem_slot = bar_base + 8u * (2 * Cfg::STAGES + 4);
    const uint32_t epi_base = bar_base + 256u;  // epilogue staging, after the 256-byte barrier area

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < Cfg::STAGES; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(acc_full_bar(b), 1);
            mbar_init(acc_empty_bar(b), 128);
        }
        fence_barrier_init();
        fence_proxy_async_smem();
        prefetch_tmap(&tmap_a);
        prefetch_tmap(&tmap_b);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    uint32_t tmem_base;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem_base) : "r"(tmem_slot) : "memory");

    const int total_units = p.m_blocks * p.n_blocks * p.split_k;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int unit = blockIdx.x; ok && unit < total_units; unit += gridDim.x) {
                int mb, nb, ks;
                decode_unit(p, unit, mb, nb, ks);
                const int kb0 = ks * p.kb_per_split;
                const int kb1 = min(p.kb_total, kb0 + p.kb_per_split);
                for (int kb = kb0; kb < kb1; ++kb) {
                    if (!mbar_wait(empty_bar(stage), phase ^ 1u)) {
                        report_timeout(p.status, 0, kb);
                        ok = false;
                        break;
                    }
                    const uint32_t a_dst = smem_base + stage * Cfg::STAGE_BYTES;
                    const uint32_t b_dst = a_dst + Cfg::A_BYTES;
                    mbar_arrive_expect_tx(full_bar(stage), Cfg::STAGE_BYTES);
                    tma_load_2d(a_dst, &tmap_a, full_bar(stage), kb * BK, mb * BM);
#pragma unroll
                    for (int j = 0; j < BN / 64; ++j)
                        tma_load_2d(b_dst + j * Cfg::B_BOX_BYTES, &tmap_b, full_bar(stage),
                                    nb * BN + j * 64, kb * BK);
                    if (++stage == Cfg::STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc_f16_f32(BM, BN, /*a_mn=*/false, /*b_mn=*/true);
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            bool ok = true;
            for (int unit = blockIdx.x; ok && unit < total_units; unit += gridDim.x) {
                int mb, nb, ks;
                decode_unit(p, unit, mb, nb, ks);
                const int kb0 = ks * p.kb_per_split;
                const int kb1 = min(p.kb_total, kb0 + p.kb_per_split);
                if (!mbar_wait(acc_empty_bar(acc), acc_phase ^ 1u)) {
                    report_timeout(p.status, 1, -1);
                    break;
                }
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + acc * BN;
                for (int kb = kb0; kb < kb1; ++kb) {
                    if (!mbar_wait(full_bar(stage), phase)) {
                        report_timeout(p.status, 1, kb);
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    const uint32_t a_src = smem_base + stage * Cfg::STAGE_BYTES;
                    const uint32_t b_src = a_src + Cfg::A_BYTES;
#pragma unroll
                    for (int kk = 0; kk < BK / 16; ++kk) {
                        // A: 16 halves = 32 bytes further along the 128-byte swizzled row.
                        const uint64_t a_desc = make_smem_desc_sw128(a_src + kk * 32, 16, 1024);
                        // B: 16 K-rows = two 8-row swizzle atoms = 2048 bytes further.
                        const uint64_t b_desc =
                            make_smem_desc_sw128(b_src + kk * 2048, Cfg::B_BOX_BYTES, 1024);
                        umma_f16(d_tmem, a_desc, b_desc, idesc, (kb > kb0 || kk > 0) ? 1u : 0u);
                    }
                    umma_commit(empty_bar(stage));  // frees the smem stage when the MMAs finish
                    if (++stage == Cfg::STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (!ok) break;
                umma_commit(acc_full_bar(acc));  // accumulator complete -> epilogue
                acc ^= 1;
                if (acc == 0) acc_phase ^= 1u;
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue (warps 2..5)
        const int quad = warp & 3;  // TMEM lane quadrant this warp may read
        const int row_in_tile = quad * 32 + lane;
        int acc = 0;
        uint32_t acc_phase = 0;
        const bool use_cin = (p.beta != 0.0f) && (p.C_in != nullptr) && (p.split_k == 1);
        const float alpha = (p.split_k == 1) ? p.alpha : 1.0f;
        const float beta = p.beta;
        for (int unit = blockIdx.x; unit < total_units; unit += gridDim.x) {
            int mb, nb, ks;
            decode_unit(p, unit, mb, nb, ks);
            if (!mbar_wait(acc_full_bar(acc), acc_phase)) {
                report_timeout(p.status, 2, unit);
                break;
            }
            tc_fence_after_sync();
            const int row = mb * BM + row_in_tile;
            const size_t slice_off = static_cast<size_t>(ks) * p.M * p.N;
            const float* in_row = use_cin ? p.C_in + static_cast<size_t>(row) * p.N : nullptr;
            const uint32_t t_addr = tmem_base + acc * BN + (static_cast<uint32_t>(quad * 32) << 16);
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                uint32_t r[32];
                tmem_ld_32x32b_x32(t_addr + c * 32, r);
                tmem_wait_ld();
                epilogue_store_block(epi_base + quad * (32 * EPI_PITCH), r, alpha, beta, in_row, row < p.M,
                                     p.C_out + slice_off, mb * BM + quad * 32, nb * BN + c * 32, p.M, p.N, p.split_k == 1,
                                     p.status);
            }
            tc_fence_before_sync();
            mbar_arrive(acc_empty_bar(acc));
            acc ^= 1;
            if (acc == 0) acc_phase ^= 1u;
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
    }
}

// ---------------------------------------------------------------------------------------------
// CTA-pair kernel: two CTAs of one cluster share a 256 x 256 output tile. The leader issues
// tcgen05.mma.cta_group::2 (M = 256: 128 rows per CTA); each CTA stages its own 128 rows of A and
// its own 128 of the 256 B columns, so per SM the shared-memory traffic for B is halved
// compared with the 1-CTA 128 x 256 tile. No TMA multicast: every CTA loads what it holds.
// Barriers: the leader's full[] counts the bytes of both CTAs' loads (the peer's TMA reports to
// the leader's barrier); the leader's MMA thread commits to empty[] and acc_full[] of both CTAs
// (one commit per CTA); both CTAs' epilogue threads arrive on the leader's acc_empty[] (256).
constexpr int PAIR_BN = 256;
#ifndef WB_PAIR_KH
#define WB_PAIR_KH 2
#endif
#ifndef WB_PAIR_STAGES
#define WB_PAIR_STAGES (6 / WB_PAIR_KH)
#endif
constexpr int PAIR_KH = WB_PAIR_KH;                  // 64-deep k-blocks per pipeline stage
constexpr int PAIR_STAGES = WB_PAIR_STAGES;
constexpr int PAIR_A_BYTES = BM * BK * 2;            // 16 KB: this CTA's 128 rows of one k-block
constexpr int PAIR_B_BYTES = 2 * BK * 64 * 2;        // 16 KB: this CTA's 128 columns (two boxes) of one k-block
constexpr int PAIR_KB_BYTES = PAIR_A_BYTES + PAIR_B_BYTES;
constexpr int PAIR_STAGE_BYTES = PAIR_KH * PAIR_KB_BYTES;
constexpr int PAIR_SMEM_BYTES = PAIR_STAGES * PAIR_STAGE_BYTES + 1024 + 256 + EPI_BYTES;

__device__ __forceinline__ void decode_pair_unit(const GemmParams& p, int unit, int& mb2, int& nb) {
    // m fastest inside groups of 8 pair-rows (= 16 m-blocks), as in decode_unit
    const int group_rows = RASTER_GROUP_M / 2;
    const int group_span = group_rows * p.n_blocks;
    const int g = unit / group_span;
    const int first = g * group_rows;
    const int rows = min(group_rows, p.m_blocks - first);
    const int r = unit - g * group_span;
    mb2 = first + r % rows;
    nb = r / rows;
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GEMM_THREADS, 1)
gemm_f16f32_pair_kernel(const __grid_constant__ CUtensorMap tmap_a,
                        const __grid_constant__ CUtensorMap tmap_b, const GemmParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t bar_base = smem_base + PAIR_STAGES * PAIR_STAGE_BYTES;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (PAIR_STAGES + s); };
    auto acc_full_bar = [&](int b) { return bar_base + 8u * (2 * PAIR_STAGES + b); };
    auto acc_empty_bar = [&](int b) { return bar_base + 8u * (2 * PAIR_STAGES + 2 + b); };
    const uint32_t tmem_slot = bar_base + 8u * (2 * PAIR_STAGES + 4);
    const uint32_t epi_base = bar_base + 256u;  // after the 256-byte barrier area: 4 warps x 32 rows x 144 bytes

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t cta_rank = cluster_ctarank();  // 0 = leader
    const int cluster_id = blockIdx.x >> 1;
    const int num_clusters = gridDim.x >> 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < PAIR_STAGES; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(acc_full_bar(b), 1);
            mbar_init(acc_empty_bar(b), 256);
        }
        fence_barrier_init();
        fence_proxy_async_smem();
        prefetch_tmap(&tmap_a);
        prefetch_tmap(&tmap_b);
    }
    if (warp == 1) {
        tmem_alloc_pair(tmem_slot, 512);
        tmem_relinquish_pair();
    }
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync();  // both CTAs' barriers exist before anything arrives on them remotely
    tc_fence_after_sync();
    uint32_t tmem_base;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem_base) : "r"(tmem_slot) : "memory");

    const int total_units = p.m_blocks * p.n_blocks;  // m_blocks counts 256-row pair blocks here

    if (warp == 0) {
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int unit = cluster_id; ok && unit < total_units; unit += num_clusters) {
                int mb2, nb;
                decode_pair_unit(p, unit, mb2, nb);
                const int row0 = mb2 * 256 + static_cast<int>(cta_rank) * 128;
                const int col0 = nb * PAIR_BN + static_cast<int>(cta_rank) * 128;
                for (int kb = 0; kb < p.kb_total; kb += PAIR_KH) {
                    if (!mbar_wait(empty_bar(stage), phase ^ 1u)) {
                        report_timeout(p.status, 10, kb);
                        ok = false;
                        break;
                    }
                    if (cta_rank == 0) mbar_arrive_expect_tx(full_bar(stage), 2 * PAIR_STAGE_BYTES);
                    const uint32_t leader_full = mapa(full_bar(stage), 0);
#pragma unroll
                    for (int h = 0; h < PAIR_KH; ++h) {
                        // a k-block past the end of K is filled with zeros by TMA
                        const uint32_t a_dst = smem_base + stage * PAIR_STAGE_BYTES + h * PAIR_KB_BYTES;
                        const uint32_t b_dst = a_dst + PAIR_A_BYTES;
                        tma_load_2d_pair(a_dst, &tmap_a, leader_full, (kb + h) * BK, row0);
                        tma_load_2d_pair(b_dst, &tmap_b, leader_full, col0, (kb + h) * BK);
                        tma_load_2d_pair(b_dst + BK * 64 * 2, &tmap_b, leader_full, col0 + 64, (kb + h) * BK);
                    }
                    if (++stage == PAIR_STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && cta_rank == 0) {
            constexpr uint32_t idesc = make_idesc_f16_f32(256, PAIR_BN, false, true);
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            bool ok = true;
            for (int unit = cluster_id; ok && unit < total_units; unit += num_clusters) {
                if (!mbar_wait(acc_empty_bar(acc), acc_phase ^ 1u)) {
                    report_timeout(p.status, 11, -1);
                    break;
                }
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + acc * PAIR_BN;
                for (int kb = 0; kb < p.kb_total; kb += PAIR_KH) {
                    if (!mbar_wait(full_bar(stage), phase)) {
                        report_timeout(p.status, 11, kb);
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
#pragma unroll
                    for (int h = 0; h < PAIR_KH; ++h) {
                        const uint32_t a_src = smem_base + stage * PAIR_STAGE_BYTES + h * PAIR_KB_BYTES;
                        const uint32_t b_src = a_src + PAIR_A_BYTES;
#pragma unroll
                        for (int kk = 0; kk < BK / 16; ++kk) {
                            const uint64_t a_desc = make_smem_desc_sw128(a_src + kk * 32, 16, 1024);
                            const uint64_t b_desc = make_smem_desc_sw128(b_src + kk * 2048, BK * 64 * 2, 1024);
                            umma_f16_pair(d_tmem, a_desc, b_desc, idesc, (kb > 0 || h > 0 || kk > 0) ? 1u : 0u);
                        }
                    }
                    umma_commit_pair(empty_bar(stage));
                    umma_commit_pair(mapa(empty_bar(stage), 1));
                    if (++stage == PAIR_STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (!ok) break;
                umma_commit_pair(acc_full_bar(acc));
                umma_commit_pair(mapa(acc_full_bar(acc), 1));
                acc ^= 1;
                if (acc == 0) acc_phase ^= 1u;
            }
        }
    } else {
        const int quad = warp & 3;
        const int row_in_tile = quad * 32 + lane;
        int acc = 0;
        uint32_t acc_phase = 0;
        const bool use_cin = (p.beta != 0.0f) && (p.C_in != nullptr);
        const float alpha = p.alpha, beta = p.beta;
        for (int unit = cluster_id; unit < total_units; unit += num_clusters) {
            int mb2, nb;
            decode_pair_unit(p, unit, mb2, nb);
            if (!mbar_wait(acc_full_bar(acc), acc_phase)) {
                report_timeout(p.status, 12, unit);
                break;
            }
            tc_fence_after_sync();
            const int row = mb2 * 256 + static_cast<int>(cta_rank) * 128 + row_in_tile;
            const float* in_row = use_cin ? p.C_in + static_cast<size_t>(row) * p.N : nullptr;
            const uint32_t t_addr = tmem_base + acc * PAIR_BN + (static_cast<uint32_t>(quad * 32) << 16);
#pragma unroll 1
            for (int c = 0; c < PAIR_BN / 32; ++c) {
                uint32_t r[32];
                tmem_ld_32x32b_x32(t_addr + c * 32, r);
                tmem_wait_ld();
                epilogue_store_block(epi_base + quad * (32 * EPI_PITCH), r, alpha, beta, in_row, row < p.M, p.C_out,
                                     mb2 * 256 + static_cast<int>(cta_rank) * 128 + quad * 32, nb * PAIR_BN + c * 32, p.M, p.N,
                                     true, p.status);
            }
            tc_fence_before_sync();
            if (cta_rank == 0) mbar_arrive(acc_empty_bar(acc));
            else mbar_arrive_cluster(mapa(acc_empty_bar(acc), 0));
            acc ^= 1;
            if (acc == 0) acc_phase ^= 1u;
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    cluster_sync();  // the peer's shared memory and barriers stay alive until both are done
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc_pair(tmem_base, 512);
    }
}

// out[i] = alpha * sum_{s ascending} partial[s][i] + beta * c_in[i]; the order of the
// reference's reduce kernel (wmma_xor_swizzle.hpp:334-353). With split == 0 it writes
// beta * c_in (the K == 0 product).
__global__ void __launch_bounds__(256)
splitk_reduce_kernel(float* out, const float* __restrict__ partials, const float* c_in,
                     size_t total4, int split, float alpha, float beta) {
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    const bool use_cin = (beta != 0.0f) && (c_in != nullptr);
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total4;
         i += stride) {
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int s = 0; s < split; ++s) {
            const float4 v = __ldcs(reinterpret_cast<const float4*>(partials) + s * total4 + i);
            acc.x += v.x;
            acc.y += v.y;
            acc.z += v.z;
            acc.w += v.w;
        }
        acc.x *= alpha;
        acc.y *= alpha;
        acc.z *= alpha;
        acc.w *= alpha;
        if (use_cin) {
            const float4 c = reinterpret_cast<const float4*>(c_in)[i];
            acc.x += beta * c.x;
            acc.y += beta * c.y;
            acc.z += beta * c.z;
            acc.w += beta * c.w;
        }
        reinterpret_cast<float4*>(out)[i] = acc;
    }
}

// ---------------------------------------------------------------------------- host side

static int ceil_div(int a, int b) { return (a + b - 1) / b; }

static int tile_bn(int tile_cfg) {
    switch (tile_cfg) {
        case WMMA_OPS_TILE_128x64: return 64;
        case WMMA_OPS_TILE_128x128: return 128;
        case WMMA_OPS_TILE_128x256: return 256;
        case WMMA_OPS_TILE_256x256_PAIR: return 256;
        default: return -1;
    }
}

// Cost model: clocks per 64-deep k-block of one CTA tile, measured on B200 at 8192^3 (the MMA
// alone would need 2*BN clocks; narrower tiles are bound by shared-memory delivery and issue:
// 128x64 reached 33 %, 128x128 58 %, 128x256 78 %, the 256x256 CTA pair 84 % of the MMA rate).
static double kblock_cost(int bn) {
    switch (bn) {
        case 64: return 390.0;
        case 128: return 440.0;
        default: return 656.0;
    }
}
constexpr double PAIR_KBLOCK_COST = 610.0;  // per pair of SMs, 256x256x64

// Measured tile table (wmma_ops_set_tile_table): rows keyed by the shape bucket
// (ceil(M/128), ceil(N/64), ceil(K/64)) and the SM count they were measured on. A product whose
// bucket is in the table gets the measured tile and split; every other product the cost model below.
struct TileTableRow {
    int mb, nb, kb, sms, tile, split;
};
static std::mutex g_tile_table_mu;
static std::vector<TileTableRow> g_tile_table;

static bool tile_table_lookup(int M, int N, int K, int sms, int* tile_cfg, int* split_k) {
    std::lock_guard<std::mutex> lock(g_tile_table_mu);
    if (g_tile_table.empty()) return false;
    const int mb = ceil_div(M, 128), nb = ceil_div(N, 64), kb = ceil_div(K, 64);
    for (const TileTableRow& r : g_tile_table) {
        if (r.mb == mb && r.nb == nb && r.kb == kb && r.sms == sms) {
            *tile_cfg = r.tile;
            *split_k = r.split;
            return true;
        }
    }
    return false;
}

static void select_tile_impl(int M, int N, int K, int sms, int* tile_cfg, int* split_k) {
    if (tile_table_lookup(M, N, K, sms, tile_cfg, split_k)) return;
    const int kb_total = ceil_div(K, BK);
    const int cfgs[3] = {WMMA_OPS_TILE_128x256, WMMA_OPS_TILE_128x128, WMMA_OPS_TILE_128x64};
    double best_time = 0.0;
    int best_cfg = WMMA_OPS_TILE_128x128, best_split = 1;
    for (int i = 0; i < 3; ++i) {
        const int bn = tile_bn(cfgs[i]);
        const int tiles = ceil_div(M, BM) * ceil_div(N, bn);
        int split = 1;
        // Split K when the output tiles cannot occupy half the SMs. Like the reference's
        // plan (wmma_xor_swizzle.hpp:293-332) a slice keeps at least 256 of K and there are
        // at most 32 slices; unlike it the factor is sized to 148 SMs and need not be a
        // power of two.
        if (tiles * 2 <= sms && kb_total >= 8) {
            split = sms / tiles;
            if (split > 32) split = 32;
            if (split > kb_total / 4) split = kb_total / 4;
            if (split < 1) split = 1;
            const int per = ceil_div(kb_total, split);
            split = ceil_div(kb_total, per);
        }
        const int units = tiles * split;
        const int waves = ceil_div(units, sms);
        const int kb_per = ceil_div(kb_total, split);
        // fixed per-unit cost: pipeline fill + epilogue drain, in clocks
        const double unit_cost = kblock_cost(bn) * kb_per + 600.0 + 2.0 * bn;
        double t = waves * unit_cost;
        // the reduce pass: its traffic, and a second launch (about 3 us of clocks) that small products never win back
        if (split > 1) t += 0.02 * split * (static_cast<double>(M) * N / sms) + 6000.0;
        if (i == 0 || t < best_time) {
            best_time = t;
            best_cfg = cfgs[i];
            best_split = split;
        }
    }
    // The CTA-pair tile: a 256 x 256 tile on two SMs has the MMA time of two 128 x 256 tiles but
    // half the B traffic per SM; measured, its k-block runs about 8 % faster than the 1-CTA
    // tile's. It has no split-K path and wants whole pairs of SMs.
    if (best_split == 1 && M > 128 && N > 128) {
        const int pair_tiles = ceil_div(M, 256) * ceil_div(N, 256);
        const int waves = ceil_div(pair_tiles, sms / 2);
        const double t = waves * (PAIR_KBLOCK_COST * kb_total + 600.0 + 512.0);
        if (t < best_time) {
            best_time = t;
            best_cfg = WMMA_OPS_TILE_256x256_PAIR;
        }
    }
    *tile_cfg = best_cfg;
    *split_k = best_split;
}

template <int BN>
static int launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int sms,
                       cudaStream_t stream) {
    using Cfg = GemmCfg<BN>;
    static std::atomic<bool> attr_set[64];  // per device; setting the attribute twice is harmless
    int dev = 0;
    WB_CHECK_CUDA(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64 && !attr_set[dev].load(std::memory_order_acquire)) {
        WB_CHECK_CUDA(cudaFuncSetAttribute(gemm_f16f32_kernel<BN>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           Cfg::SMEM_BYTES));
        attr_set[dev].store(true, std::memory_order_release);
    }
    const int units = p.m_blocks * p.n_blocks * p.split_k;
    const int grid = units < sms ? units : sms;
    gemm_f16f32_kernel<BN><<<grid, GEMM_THREADS, Cfg::SMEM_BYTES, stream>>>(ta, tb, p);
    WB_CHECK_CUDA(cudaGetLastError());
    return WMMA_OPS_OK;
}

static int launch_gemm_pair(const CUtensorMap& ta, const CUtensorMap& tb, GemmParams p, int sms,
                            cudaStream_t stream) {
    static std::atomic<bool> attr_set[64];  // per device; setting the attribute twice is harmless
    int dev = 0;
    WB_CHECK_CUDA(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64 && !attr_set[dev].load(std::memory_order_acquire)) {
        WB_CHECK_CUDA(cudaFuncSetAttribute(gemm_f16f32_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           PAIR_SMEM_BYTES));
        attr_set[dev].store(true, std::memory_order_release);
    }
    p.m_blocks = ceil_div(p.M, 256);
    p.n_blocks = ceil_div(p.N, PAIR_BN);
    const int units = p.m_blocks * p.n_blocks;
    const int clusters = units < sms / 2 ? units : sms / 2;
    gemm_f16f32_pair_kernel<<<2 * clusters, GEMM_THREADS, PAIR_SMEM_BYTES, stream>>>(ta, tb, p);
    WB_CHECK_CUDA(cudaGetLastError());
    return WMMA_OPS_OK;
}

}  // namespace wb

extern "C" int wmma_ops_select_tile(int M, int N, int K, int num_sms, int* tile_cfg, int* split_k) {
    WB_REQUIRE(M >= 1 && N >= 1 && K >= 1, WMMA_OPS_ERR_INVALID,
               "select_tile: M, N, K must be positive (got %d, %d, %d)", M, N, K);
    WB_REQUIRE(tile_cfg != nullptr && split_k != nullptr, WMMA_OPS_ERR_INVALID,
               "select_tile: null output pointer");
    wb::select_tile_impl(M, N, K, num_sms > 0 ? num_sms : 148, tile_cfg, split_k);
    return WMMA_OPS_OK;
}

extern "C" int wmma_ops_set_tile_table(const int* rows, int n_rows) {
    using namespace wb;
    WB_REQUIRE(n_rows >= 0 && (n_rows == 0 || rows != nullptr), WMMA_OPS_ERR_INVALID, "set_tile_table: bad arguments");
    std::vector<TileTableRow> table;
    table.reserve(n_rows);
    for (int i = 0; i < n_rows; ++i) {
        const int* r = rows + 6 * i;
        const int M = r[0], N = r[1], K = r[2], sms = r[3], tile = r[4], split = r[5];
        WB_REQUIRE(M >= 1 && N >= 1 && K >= 1 && sms >= 1, WMMA_OPS_ERR_INVALID,
                   "set_tile_table: row %d has a non-positive shape or SM count", i);
        WB_REQUIRE(tile_bn(tile) > 0, WMMA_OPS_ERR_INVALID, "set_tile_table: row %d names tile %d", i, tile);
        WB_REQUIRE(split >= 1 && split <= ceil_div(K, BK) && (split == 1 || tile != WMMA_OPS_TILE_256x256_PAIR),
                   WMMA_OPS_ERR_INVALID, "set_tile_table: row %d has split_k=%d (1..K/64; the CTA-pair tile has no split)", i,
                   split);
        table.push_back({ceil_div(M, 128), ceil_div(N, 64), ceil_div(K, 64), sms, tile, split});
    }
    std::lock_guard<std::mutex> lock(g_tile_table_mu);
    g_tile_table.swap(table);
    return WMMA_OPS_OK;
}

extern "C" size_t wmma_ops_gemm_workspace_bytes(int M, int N, int K, int split_k) {
    (void)K;
    if (split_k <= 1 || M <= 0 || N <= 0) return 0;
    return static_cast<size_t>(split_k) * static_cast<size_t>(M) * static_cast<size_t>(N) *
           sizeof(float);
}

extern "C" int wmma_ops_gemm_f16f32(const void* A, const void* B, const void* C_in, void* C_out,
                                    int M, int N, int K, float alpha, float beta, int tile_cfg,
                                    int split_k, void* workspace, size_t workspace_bytes,
                                    int* status, void* stream_) {
    using namespace wb;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    WB_REQUIRE(M >= 0 && N >= 0 && K >= 0, WMMA_OPS_ERR_INVALID,
               "gemm: negative dimension (M=%d, N=%d, K=%d)", M, N, K);
    if (M == 0 || N == 0) return WMMA_OPS_OK;
    WB_REQUIRE(C_out != nullptr, WMMA_OPS_ERR_INVALID, "gemm: C_out is null");
    WB_REQUIRE(N % 8 == 0, WMMA_OPS_ERR_INVALID,
               "N must be a multiple of 8 for 16-byte row pitch (got N=%d)", N);
    WB_REQUIRE(K % 8 == 0, WMMA_OPS_ERR_INVALID,
               "K must be a multiple of 8 for 16-byte row pitch (got K=%d)", K);
    WB_REQUIRE((reinterpret_cast<uintptr_t>(C_out) % 16) == 0, WMMA_OPS_ERR_INVALID,
               "C must be 16-byte aligned");
    WB_REQUIRE(C_in == nullptr || (reinterpret_cast<uintptr_t>(C_in) % 16) == 0,
               WMMA_OPS_ERR_INVALID, "C must be 16-byte aligned");

    const size_t total4 = static_cast<size_t>(M) * N / 4;
    const int sms = sm_count();
    auto launch_reduce = [&](const float* partials, int split) -> int {
        size_t blocks = (total4 + 255) / 256;
        const size_t cap = static_cast<size_t>(sms) * 8;
        if (blocks > cap) blocks = cap;
        splitk_reduce_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
            static_cast<float*>(C_out), partials, static_cast<const float*>(C_in), total4, split,
            alpha, beta);
        WB_CHECK_CUDA(cudaGetLastError());
        return WMMA_OPS_OK;
    };
    if (K == 0) return launch_reduce(nullptr, 0);

    WB_REQUIRE(A != nullptr && B != nullptr, WMMA_OPS_ERR_INVALID, "gemm: A or B is null");
    WB_REQUIRE((reinterpret_cast<uintptr_t>(A) % 16) == 0, WMMA_OPS_ERR_INVALID,
               "A must be 16-byte aligned");
    WB_REQUIRE((reinterpret_cast<uintptr_t>(B) % 16) == 0, WMMA_OPS_ERR_INVALID,
               "B must be 16-byte aligned");

    if (tile_cfg == WMMA_OPS_TILE_AUTO) {
        int auto_split = 1;
        select_tile_impl(M, N, K, sms, &tile_cfg, &auto_split);
        if (split_k == 0) split_k = auto_split;
    }
    const int bn = tile_bn(tile_cfg);
    WB_REQUIRE(bn > 0, WMMA_OPS_ERR_INVALID,
               "Invalid tile_config: 0=128x64, 1=128x128, 2=128x256, 3=256x256 (CTA pair)");
    if (split_k < 1) split_k = 1;

    GemmParams p;
    p.M = M;
    p.N = N;
    p.K = K;
    p.m_blocks = ceil_div(M, BM);
    p.n_blocks = ceil_div(N, bn);
    p.kb_total = ceil_div(K, BK);
    if (split_k > p.kb_total) split_k = p.kb_total;
    p.kb_per_split = ceil_div(p.kb_total, split_k);
    split_k = ceil_div(p.kb_total, p.kb_per_split);  // no empty slice
    p.split_k = split_k;
    p.alpha = alpha;
    p.beta = beta;
    p.status = status;
    p.C_in = static_cast<const float*>(C_in);
    if (split_k > 1) {
        const size_t need = wmma_ops_gemm_workspace_bytes(M, N, K, split_k);
        WB_REQUIRE(workspace != nullptr && workspace_bytes >= need, WMMA_OPS_ERR_WORKSPACE,
                   "gemm: split_k=%d needs %zu bytes of workspace (got %zu)", split_k, need,
                   workspace_bytes);
        WB_REQUIRE((reinterpret_cast<uintptr_t>(workspace) % 16) == 0, WMMA_OPS_ERR_INVALID,
                   "workspace must be 16-byte aligned");
        p.C_out = static_cast<float*>(workspace);
    } else {
        p.C_out = static_cast<float*>(C_out);
    }

    CUtensorMap ta, tb;
    int rc = encode_tmap_2d(&ta, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, A, static_cast<uint64_t>(K),
                            static_cast<uint64_t>(M), static_cast<uint64_t>(K) * 2, BK, BM,
                            CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != WMMA_OPS_OK) return rc;
    rc = encode_tmap_2d(&tb, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, B, static_cast<uint64_t>(N),
                        static_cast<uint64_t>(K), static_cast<uint64_t>(N) * 2, 64, BK,
                        CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != WMMA_OPS_OK) return rc;

    if (tile_cfg == WMMA_OPS_TILE_256x256_PAIR && split_k == 1)
        return launch_gemm_pair(ta, tb, p, sms, stream);
    switch (bn) {
        case 64: rc = launch_gemm<64>(ta, tb, p, sms, stream); break;
        case 128: rc = launch_gemm<128>(ta, tb, p, sms, stream); break;
        default: rc = launch_gemm<256>(ta, tb, p, sms, stream); break;
    }
    if (rc != WMMA_OPS_OK) return rc;
    if (split_k > 1) return launch_reduce(static_cast<const float*>(workspace), split_k);
    return WMMA_OPS_OK;
}

// ---------------------------------------------------------------------------------------------
// Split-K GEMM for callers that cannot allocate device memory.
//
// Some hosts of this library may not call cudaMalloc at the point where they need a GEMM: code
// that runs inside another framework's memory pool and must not go around it, plugins that are
// only handed their input and output buffers, and real-time loops where an allocation (which
// may synchronise the device) is not acceptable. The split-K path normally needs a caller-owned
// workspace for its partial products; this entry point keeps that workspace inside the library
// instead, in a fixed array in device memory that every GPU which loads the library holds until
// the process exits.
namespace wb {

constexpr size_t STATIC_SCRATCH_BYTES = 8u << 20;  // 8 MiB = 32 slices of a 256 x 256 fp32 product
static __device__ __align__(256) float g_splitk_scratch[STATIC_SCRATCH_BYTES / sizeof(float)];

// The array's name is only a handle on the host; its device address is looked up once per
// device (with that device current) and cached.
static int static_scratch_ptr(float** out) {
    static float* cached[64] = {};
    static std::mutex mu;
    int dev = 0;
    WB_CHECK_CUDA(cudaGetDevice(&dev));
    WB_REQUIRE(dev >= 0 && dev < 64, WMMA_OPS_ERR_INVALID, "device index %d out of range", dev);
    std::lock_guard<std::mutex> lock(mu);
    if (cached[dev] == nullptr) {
        void* ptr = nullptr;
        WB_CHECK_CUDA(cudaGetSymbolAddress(&ptr, g_splitk_scratch));
        cached[dev] = static_cast<float*>(ptr);
    }
    *out = cached[dev];
    return WMMA_OPS_OK;
}

}  // namespace wb

extern "C" size_t wmma_ops_gemm_static_scratch_bytes(void) { return wb::STATIC_SCRATCH_BYTES; }

extern "C" int wmma_ops_gemm_f16f32_splitk_static(const void* A, const void* B, const void* C_in, void* C_out,
                                                  int M, int N, int K, float alpha, float beta, int tile_cfg,
                                                  int split_k, int* status, void* stream) {
    using namespace wb;
    WB_REQUIRE(M >= 1 && N >= 1 && K >= 1, WMMA_OPS_ERR_INVALID,
               "gemm_splitk_static: M, N, K must be positive (got %d, %d, %d)", M, N, K);
    // Resolve the tile and slice count here, so that the size check below sees the final plan.
    if (tile_cfg == WMMA_OPS_TILE_AUTO) {
        int auto_split = 1;
        select_tile_impl(M, N, K, sm_count(), &tile_cfg, &auto_split);
        if (split_k == 0) split_k = auto_split;
    }
    if (split_k < 1) split_k = 1;
    // the clamp wmma_ops_gemm_f16f32 applies: at most one slice per 64-deep k-block, no empty slice
    const int kb_total = ceil_div(K, BK);
    if (split_k > kb_total) split_k = kb_total;
    split_k = ceil_div(kb_total, ceil_div(kb_total, split_k));
    const size_t need = wmma_ops_gemm_workspace_bytes(M, N, K, split_k);
    WB_REQUIRE(need <= STATIC_SCRATCH_BYTES, WMMA_OPS_ERR_WORKSPACE,
               "gemm_splitk_static: split_k=%d of a %d x %d product needs %zu bytes of partial sums, more than "
               "the built-in scratch of %zu bytes; use wmma_ops_gemm_f16f32 with a workspace of your own",
               split_k, M, N, need, STATIC_SCRATCH_BYTES);
    float* scratch = nullptr;
    int rc = static_scratch_ptr(&scratch);
    if (rc != WMMA_OPS_OK) return rc;
    return wmma_ops_gemm_f16f32(A, B, C_in, C_out, M, N, K, alpha, beta, tile_cfg, split_k, scratch,
                                STATIC_SCRATCH_BYTES, status, stream);
}
