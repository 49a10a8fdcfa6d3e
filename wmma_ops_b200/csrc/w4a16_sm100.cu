// INT4 weight prepack ("W4-B200-v1") and the fused W4A16 GEMM for sm_100a.
//
// The reference snapshot has no INT4 code; the entry points, the packed format and the
// arithmetic  C[M,N] = A[M,K] . ((code - 8) * scale[k / group][n])  are specified here and
// restated on the CPU in oracle/int4.py.
//
// Packed format: uint32 [K/64][N_pad/128][128][8].  Block (kb, nt) is 4 KB and holds, for the
// 128 weight columns n = 128 nt + r, the 64 codes k = 64 kb .. 64 kb + 63 as 8 words per
// column; word j, nibble p holds k = 64 kb + 8 j + {0,2,4,6,1,3,5,7}[p].  Blocks are ordered
// k-block major: the CTAs of a launch walk K in step, so at any moment the whole GPU reads one
// contiguous window of the weights and the requests spread over every memory channel (with
// column-tile-major order the CTAs' streams sat 256 KB apart and camped on a few channels).
//
// Kernel: the weights sit on the 128-row side of the MMA (it computes C^T = W^T . A^T):
//   A operand  = dequantised W^T tile, 128 columns-of-W x 64 k, fp16, K-major, 128-byte swizzle,
//                written to shared memory by eight dequant warps (never to global memory);
//   B operand  = activation tile, BT tokens x 64 k, loaded by TMA straight from A [M,K];
//   accumulator = 128 TMEM lanes (weight columns) x BT columns (tokens), fp32.
// One weight element is dequantised once per 256 tokens, so the same kernel serves decode
// (M = 1..16, HBM-bound) and prefill (M in the thousands, tensor-bound).
// Warps: 2 MMA issuer + TMEM owner; 4..11 workers (each requests, expands and hands over whole
// 4 KB blocks); 12..15 epilogue; 0, 1, 3 idle.  Split-K partials are combined by the last CTA to finish a
// tile (arrival counter, no waiting), summed in ascending slice order.
#include <cstdlib>

#include "host_common.cuh"
#include "ptx.cuh"
#include "w4a16_common.cuh"

#ifndef W4_PREFILL_REGS
#define W4_PREFILL_REGS 104
#endif

namespace wb {

template <int BT, bool WM>
struct W4Cfg {
    static constexpr int X_BYTES = BT * W4_BK * 2;
    static constexpr int S_STAGE = W4_WT_BYTES + X_BYTES;
    // Wt + X ring. One dequant warp owns each stage (DQ = S), and the raw ring is a multiple
    // of S, so every barrier is waited on by the same warp pass after pass: a parity wait can
    // then never be more than one phase away from the barrier's state.
    static constexpr int S = (BT >= 256) ? 4 : (BT >= 64) ? 6 : 8;
    static constexpr int R = (BT >= 256) ? 4 : (BT >= 128) ? 6 : (BT >= 64) ? 12 : (BT >= 32) ? 8 : 16;
    static_assert(S * S_STAGE + R * W4_SLOT_BYTES + 1024 + 512 + 32 * 64 * 4 <= 232448, "shared memory budget");
    static constexpr int DQ = S;
    static_assert(R % S == 0 && DQ <= W4_DQ_WARPS, "ring sizes must nest");
    // Threads that issue MMAs when the workers do not (prefill / mid-size token tiles): with two,
    // alternate k-blocks go to warps 2 and 3, each with its own accumulator, which halves the
    // chain of waits, MMAs and commits a single issuing thread has to walk per k-block. Two
    // accumulators x two sets must fit the 512 TMEM columns, so token tiles up to 128 only.
    static constexpr int NI = (!WM && BT >= 64 && BT <= 128) ? 2 : 1;
    // WM (worker-MMA, decode): every worker accumulates into its own BT columns, two sets
    static constexpr int ACCS = WM ? DQ : NI;
    static constexpr int TMEM_NEED = 2 * ACCS * BT;
    static constexpr int TMEM_COLS = TMEM_NEED <= 32 ? 32 : TMEM_NEED <= 64 ? 64 : TMEM_NEED <= 128 ? 128 : TMEM_NEED <= 256 ? 256 : 512;
    static_assert(TMEM_NEED <= 512, "TMEM budget");
    static constexpr int STAGE_OUT_BYTES = 32 * 64 * 4;  // silu(gate)*up hand-over between epilogue warps
    static constexpr int SMEM_BYTES = S * S_STAGE + R * W4_SLOT_BYTES + 1024 + 512 + STAGE_OUT_BYTES;
    // Registers per thread. The prefill tile is held to 104 (measured: as fast as 128; 96 costs 5 %), which
    // leaves 12 K of the SM's registers, and its shared memory leaves 8 KB: enough for a 192-thread CTA of the
    // all-reduce kernel to run on the same SM while this persistent kernel occupies every SM.
    static constexpr int MAX_REGS = (BT >= 256 && !WM) ? W4_PREFILL_REGS : 128;
};


__device__ __forceinline__ void dq_word_store(uint32_t dst, uint32_t w, __half2 scale2) {
    const uint32_t w8 = w >> 8;
    const uint32_t a = dq_pair(w & 0x000F000Fu, scale2);
    const uint32_t b = dq_pair_hi(w & 0x00F000F0u, scale2);
    const uint32_t c = dq_pair(w8 & 0x000F000Fu, scale2);
    const uint32_t d = dq_pair_hi(w8 & 0x00F000F0u, scale2);
    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(a), "r"(b), "r"(c), "r"(d));
}

template <int BT, bool WM>
__global__ void __maxnreg__((W4Cfg<BT, WM>::MAX_REGS))
w4a16_gemm_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w,
                  const __grid_constant__ CUtensorMap tmap_sc, const W4Params p) {
    using Cfg = W4Cfg<BT, WM>;
    extern __shared__ uint8_t smem_raw_[];
    const uint32_t smem_base = (smem_u32(smem_raw_) + 1023u) & ~1023u;
    const uint32_t raw_base = smem_base + Cfg::S * Cfg::S_STAGE;
    const uint32_t bar_base = raw_base + Cfg::R * W4_SLOT_BYTES;
    auto x_full = [&](int s) { return bar_base + 8u * s; };
    auto wt_full = [&](int s) { return bar_base + 8u * (Cfg::S + s); };
    auto st_empty = [&](int s) { return bar_base + 8u * (2 * Cfg::S + s); };
    auto raw_full = [&](int r) { return bar_base + 8u * (3 * Cfg::S + r); };
    auto acc_full = [&](int b) { return bar_base + 8u * (3 * Cfg::S + 2 * Cfg::R + b); };
    auto acc_empty = [&](int b) { return bar_base + 8u * (3 * Cfg::S + 2 * Cfg::R + 2 + b); };
    const uint32_t tmem_slot = bar_base + 8u * (3 * Cfg::S + 2 * Cfg::R + 4);
    const uint32_t flag_slot = tmem_slot + 8u;
    const uint32_t out_stage = bar_base + 512u;  // 8 KB, used by the fused silu(gate)*up epilogue
    static_assert(8 * (3 * Cfg::S + 2 * Cfg::R + 6) <= 512, "barrier area too small");

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < Cfg::S; ++s) {
            // without worker-issued MMAs one barrier per stage collects both the activation tile's
            // bytes and the worker's "weights expanded" arrival: the MMA issuer then waits once per block
            mbar_init(x_full(s), WM ? 1 : 2);
            mbar_init(wt_full(s), 1);
            mbar_init(st_empty(s), 1);
        }
        for (int r = 0; r < Cfg::R; ++r) {
            mbar_init(raw_full(r), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(acc_full(b), WM ? Cfg::DQ : Cfg::NI);
            mbar_init(acc_empty(b), 128);
        }
        fence_barrier_init();
        fence_proxy_async_smem();
        prefetch_tmap(&tmap_x);
        prefetch_tmap(&tmap_w);
        prefetch_tmap(&tmap_sc);
    }
    if (warp == 2) {
        tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    uint32_t tmem_base;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem_base) : "r"(tmem_slot) : "memory");


    if (warp == 2 || (Cfg::NI == 2 && warp == 3)) {
        // ------------------------------------------------ MMA issuer(s)
        // Issuer q (warp 2 + q) takes the iterations j = q, q + NI, ... of the CTA's k-block
        // sequence (stage j % S) and accumulates into its own accumulator of the current set.
        if (lane == 0 && !WM) {
            constexpr uint32_t idesc = make_idesc_f16_f32(W4_TILE_N, BT, false, false);
            const int q = warp - 2;
            int j = 0;  // iteration index over all units of this CTA
            int acc = 0;
            uint32_t acc_ph = 0;
            bool ok = true;
            W4Unit U;
            for (int ui = 0; ok && w4_unit(p, ui, U); ++ui) {
                const int kb0 = U.kb0, kb1 = U.kb1;
                if (!mbar_wait(acc_empty(acc), acc_ph ^ 1u)) {
                    w4_report(p.status, 2, -1);
                    break;
                }
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + (acc * Cfg::ACCS + q) * BT;
                bool first = true;  // this issuer's first block of the unit overwrites its accumulator
                for (int kb = kb0; kb < kb1; ++kb, ++j) {
                    if (Cfg::NI == 2 && (j & 1) != q) continue;
                    const int s = j % Cfg::S;
                    const uint32_t ph = static_cast<uint32_t>(j / Cfg::S) & 1u;
                    if (!mbar_wait(x_full(s), ph)) {
                        w4_report(p.status, 2, kb);
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    const uint32_t wt_src = smem_base + s * Cfg::S_STAGE;
                    const uint32_t x_src = wt_src + W4_WT_BYTES;
#pragma unroll
                    for (int kk = 0; kk < W4_BK / 16; ++kk) {
                        const uint64_t a_desc = make_smem_desc_sw128(wt_src + kk * 32, 16, 1024);
                        const uint64_t b_desc = make_smem_desc_sw128(x_src + kk * 32, 16, 1024);
                        umma_f16(d_tmem, a_desc, b_desc, idesc, (!first || kk > 0) ? 1u : 0u);
                    }
                    first = false;
                    umma_commit(st_empty(s));
                }
                if (!ok) break;
                umma_commit(acc_full(acc));
                acc ^= 1;
                if (acc == 0) acc_ph ^= 1u;
            }
        }
    } else if (warp >= 4 && warp < 4 + W4_DQ_WARPS) {
        // ------------------------------------------------ dequant warps
        // Warp w (< DQ) expands iterations j = w, w + DQ, w + 2 DQ, ... of this CTA's k-block
        // sequence, a whole 4 KB block each, so DQ blocks are in flight and the fixed costs of
        // an iteration (two waits, a proxy fence, two arrivals) are paid once per block.
        // Worker warps. Warp w (< DQ) owns pipeline stage w and handles iterations j = w, w + DQ,
        // ... of this CTA's k-block sequence end to end: it waits for the packed block it
        // requested earlier, requests the activation tile for its stage, expands the block,
        // hands the stage to the MMA warp and requests the packed block of iteration j + R into
        // the slot it has just emptied. There is no separate producer thread: a single thread
        // issuing every TMA load of the CTA was starved by the workers' shared-memory traffic
        // (about 350 ns per block), while eight warps issuing their own loads are not.
        const int w = warp - 4;
        if (w < Cfg::DQ) {
            W4Cursor cur, pre;
            w4_cursor_start(p, cur);
            w4_cursor_advance(p, cur, w);
            pre = cur;
            auto request_raw = [&](const W4Cursor& c, int jj) {
                const int r = jj % Cfg::R;
                mbar_arrive_expect_tx(raw_full(r), W4_SLOT_BYTES);
                tma_load_2d(raw_base + r * W4_SLOT_BYTES, &tmap_w, raw_full(r), 0, (c.kb * p.n_tiles + c.nt) * 4);
                tma_load_2d(raw_base + r * W4_SLOT_BYTES + W4_RAW_BYTES, &tmap_sc, raw_full(r), c.nt * W4_TILE_N,
                            c.kb / p.group_kb);
            };
            // prologue: this warp's first R / DQ blocks
            for (int i = 0; i < Cfg::R / Cfg::DQ; ++i) {
                if (pre.valid && lane == 0) request_raw(pre, w + i * Cfg::DQ);
                w4_cursor_advance(p, pre, Cfg::DQ);
            }
            for (int j = w; cur.valid; j += Cfg::DQ) {
                const int r = j % Cfg::R;
                const int s = w;  // DQ == S: this warp owns stage w
                const uint32_t ph_r = (j / Cfg::R) & 1;
                const uint32_t ph_s = (j / Cfg::S) & 1;
                if (!mbar_wait(st_empty(s), ph_s ^ 1u)) {
                    w4_report(p.status, 3, -j - 1);
                    break;
                }
                const uint32_t wt = smem_base + s * Cfg::S_STAGE;
                if (lane == 0) {
                    mbar_arrive_expect_tx(x_full(s), Cfg::X_BYTES);
                    tma_load_2d(wt + W4_WT_BYTES, &tmap_x, x_full(s), cur.kb * W4_BK, cur.tt * BT);
                }
                if (!mbar_wait(raw_full(r), ph_r)) {
                    w4_report(p.status, 3, j);
                    break;
                }
                const uint32_t raw = raw_base + r * W4_SLOT_BYTES;
                // Lane reads bytes [16 i, 16 i + 16) of the block for i = 32 q + lane, q = 0..7:
                // row i / 2, 16-byte half i % 2 (conflict-free loads; the swizzled stores are too).
                // All loads are issued before the first store so their latencies overlap.
                uint4 v[8];
                uint32_t sc_bits[8];
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                    const int i = q * 32 + lane;
                    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                                 : "=r"(v[q].x), "=r"(v[q].y), "=r"(v[q].z), "=r"(v[q].w)
                                 : "r"(raw + i * 16));
                    asm volatile("ld.shared.u16 %0, [%1];" : "=r"(sc_bits[q]) : "r"(raw + W4_RAW_BYTES + (i >> 1) * 2));
                }
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                    const int i = q * 32 + lane;
                    const uint32_t row = i >> 1;
                    const uint32_t c_base = (i & 1) * 4;
                    const __half2 scale2 = __half2half2(__ushort_as_half(static_cast<unsigned short>(sc_bits[q])));
                    dq_word_store(wt + sw128_offset(row, c_base + 0), v[q].x, scale2);
                    dq_word_store(wt + sw128_offset(row, c_base + 1), v[q].y, scale2);
                    dq_word_store(wt + sw128_offset(row, c_base + 2), v[q].z, scale2);
                    dq_word_store(wt + sw128_offset(row, c_base + 3), v[q].w, scale2);
                }
                // Every lane's stores consumed its loaded registers, so all loads of the slot have
                // completed before it is refilled below.
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) {
                    if constexpr (WM) {
                        // Decode mode: this warp issues the MMAs of its own block into its own
                        // accumulator (the epilogue adds the DQ accumulators), so no single thread
                        // has to walk every block of the CTA.
                        constexpr uint32_t idesc = make_idesc_f16_f32(W4_TILE_N, BT, false, false);
                        const int u_idx = cur.ui;
                        const int set = u_idx & 1;
                        const bool first = (cur.kb - cur.kb0) < Cfg::DQ;
                        const bool last = (cur.kb + Cfg::DQ) >= cur.kb1;
                        bool good = mbar_wait(x_full(s), ph_s);
                        if (good && first) good = mbar_wait(acc_empty(set), ((u_idx >> 1) & 1) ^ 1u);
                        if (!good) w4_report(p.status, 5, j);
                        tc_fence_after_sync();
                        const uint32_t d_tmem = tmem_base + (set * Cfg::DQ + w) * BT;
#pragma unroll
                        for (int kk = 0; kk < W4_BK / 16; ++kk) {
                            const uint64_t a_desc = make_smem_desc_sw128(wt + kk * 32, 16, 1024);
                            const uint64_t b_desc = make_smem_desc_sw128(wt + W4_WT_BYTES + kk * 32, 16, 1024);
                            umma_f16(d_tmem, a_desc, b_desc, idesc, (first && kk == 0) ? 0u : 1u);
                        }
                        umma_commit(st_empty(s));
                        if (last) umma_commit(acc_full(set));
                    } else {
                        mbar_arrive(x_full(s));
                    }
                    if (pre.valid) request_raw(pre, j + Cfg::R);
                }
                w4_cursor_advance(p, cur, Cfg::DQ);
                w4_cursor_advance(p, pre, Cfg::DQ);
            }
        }
    } else if (warp >= 12) {
        // ------------------------------------------------ epilogue warps
        const int quad = warp & 3;
        const int row = quad * 32 + lane;  // weight column inside the tile
        const int et = threadIdx.x - 384;  // 0..127
        const bool vec16 = (reinterpret_cast<uintptr_t>(p.C16) & 15u) == 0;  // fp16 rows can be written as 16-byte vectors
        int acc = 0;
        uint32_t acc_ph = 0;
        int j0 = 0;  // iteration index of the unit's first k-block (two issuers: which one had it)
        W4Unit U;
        for (int ui = 0; w4_unit(p, ui, U); ++ui) {
            const int nt = U.nt, tt = U.tt, sl = U.sl, nsl = U.nsl;
            // with two MMA issuers, issuer q accumulated the unit's blocks with iteration parity q;
            // a one-block unit leaves the other issuer's accumulator untouched (stale)
            const int unit_blocks = U.kb1 - U.kb0;
            const bool use0 = unit_blocks >= 2 || (j0 & 1) == 0;
            const bool use1 = unit_blocks >= 2 || (j0 & 1) == 1;
            j0 += unit_blocks;
            if (!mbar_wait_relaxed(acc_full(acc), acc_ph, 256)) {
                w4_report(p.status, 4, ui);
                break;
            }
            tc_fence_after_sync();
            const int n = nt * W4_TILE_N + row;
            const int t0 = tt * BT;
            const int tile_id = nt * p.t_tiles + tt;
            const uint32_t t_addr = tmem_base + acc * Cfg::ACCS * BT + (static_cast<uint32_t>(quad * 32) << 16);
            float* part = (nsl > 1)
                              ? p.partials + (static_cast<size_t>(tile_id) * p.max_slices + sl) * (BT * 128)
                              : nullptr;
            constexpr int CH = (BT >= 32) ? 32 : 16;
#pragma unroll 1
            for (int c = 0; c < BT / CH; ++c) {
                uint32_t v[CH];
                if constexpr (CH == 32) tmem_ld_32x32b_x32(t_addr + c * CH, v);
                else tmem_ld_32x32b_x16(t_addr + c * CH, v);
                tmem_wait_ld();
                if constexpr (!WM && Cfg::NI == 2) {
                    uint32_t u1[CH];
                    if constexpr (CH == 32) tmem_ld_32x32b_x32(t_addr + BT + c * CH, u1);
                    else tmem_ld_32x32b_x16(t_addr + BT + c * CH, u1);
                    tmem_wait_ld();
#pragma unroll
                    for (int j = 0; j < CH; ++j) {
                        const float a0 = use0 ? __uint_as_float(v[j]) : 0.f;
                        const float a1 = use1 ? __uint_as_float(u1[j]) : 0.f;
                        v[j] = __float_as_uint(a0 + a1);
                    }
                }
                if constexpr (WM) {
                    // add the other workers' accumulators in worker order; the loads of two
                    // accumulators are in flight together
#pragma unroll 1
                    for (int a = 1; a < Cfg::ACCS; a += 2) {
                        uint32_t u0[CH], u1[CH];
                        if constexpr (CH == 32) {
                            tmem_ld_32x32b_x32(t_addr + a * BT + c * CH, u0);
                            if (a + 1 < Cfg::ACCS) tmem_ld_32x32b_x32(t_addr + (a + 1) * BT + c * CH, u1);
                        } else {
                            tmem_ld_32x32b_x16(t_addr + a * BT + c * CH, u0);
                            if (a + 1 < Cfg::ACCS) tmem_ld_32x32b_x16(t_addr + (a + 1) * BT + c * CH, u1);
                        }
                        tmem_wait_ld();
#pragma unroll
                        for (int j = 0; j < CH; ++j) {
                            float t = __uint_as_float(v[j]) + __uint_as_float(u0[j]);
                            if (a + 1 < Cfg::ACCS) t += __uint_as_float(u1[j]);
                            v[j] = __float_as_uint(t);
                        }
                    }
                }
                if (part != nullptr) {
#pragma unroll
                    for (int j = 0; j < CH; ++j) part[(c * CH + j) * 128 + row] = __uint_as_float(v[j]);
                } else if (p.out_mode == 0) {
                    if (n < p.N) {
#pragma unroll
                        for (int j = 0; j < CH; ++j) {
                            const int t = t0 + c * CH + j;
                            if (t < p.M && WB_DEBUG_INDEX(t >= 0 && n >= 0, p.status, 101, n)) p.C[static_cast<size_t>(t) * p.N + n] = __uint_as_float(v[j]);
                        }
                    }
                } else if (p.out_mode == 1 && vec16) {
                    // fp16 output: a thread holds CH tokens of ONE column, but a row of the output wants 128
                    // columns of one token. Storing element by element (2-byte stores, one branch each) made
                    // the epilogue of a 256-token tile take 10 us, longer than the k-loop of a short-K product.
                    // The chunk is therefore transposed through shared memory ([token][column], 8 KB) and
                    // written as 16-byte vectors: sixteen lanes cover one 256-byte row of the tile.
#pragma unroll
                    for (int j = 0; j < CH; j += 2) {
                        const __half2 h2 = __floats2half2_rn(p.alpha * __uint_as_float(v[j]), p.alpha * __uint_as_float(v[j + 1]));
                        const uint32_t hb = *reinterpret_cast<const uint32_t*>(&h2);
                        asm volatile("st.shared.u16 [%0], %1;" ::"r"(out_stage + (j * 128 + row) * 2),
                                     "h"(static_cast<unsigned short>(hb & 0xffffu))
                                     : "memory");
                        asm volatile("st.shared.u16 [%0], %1;" ::"r"(out_stage + ((j + 1) * 128 + row) * 2),
                                     "h"(static_cast<unsigned short>(hb >> 16))
                                     : "memory");
                    }
                    named_barrier_sync(3, 128);
#pragma unroll
                    for (int ps = 0; ps < CH / 8; ++ps) {
                        const int r = ps * 8 + (et >> 4);  // token row inside the chunk
                        const int cv = (et & 15) * 8;      // first of this thread's eight columns
                        uint4 val;
                        asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                                     : "=r"(val.x), "=r"(val.y), "=r"(val.z), "=r"(val.w)
                                     : "r"(out_stage + (r * 128 + cv) * 2)
                                     : "memory");
                        const int t = t0 + c * CH + r;
                        const int nn = nt * W4_TILE_N + cv;  // N is a multiple of 8: a vector is inside or outside
                        if (t < p.M && nn < p.N && WB_DEBUG_INDEX(t >= 0 && nn >= 0 && nn + 8 <= p.N, p.status, 102, nn))
                            *reinterpret_cast<uint4*>(p.C16 + static_cast<size_t>(t) * p.N + nn) = val;
                    }
                    named_barrier_sync(3, 128);  // the buffer is rewritten by the next chunk
                } else if (p.out_mode == 1) {
                    // output not 16-byte aligned: element by element
                    if (n < p.N) {
#pragma unroll
                        for (int j = 0; j < CH; ++j) {
                            const int t = t0 + c * CH + j;
                            if (t < p.M && WB_DEBUG_INDEX(t >= 0 && n >= 0, p.status, 102, n))
                                p.C16[static_cast<size_t>(t) * p.N + n] = __float2half_rn(p.alpha * __uint_as_float(v[j]));
                        }
                    }
                } else if (vec16) {
                    // Fused gate/up: the tile's rows 0..63 are gate columns and rows 64..127 the up columns of
                    // the same 64 outputs, so thread f of the gate warps and thread f of the up warps hold the
                    // two factors of output f for the chunk's CH tokens. They split the tokens: each sends the
                    // other its values for the half it does not compute (through shared memory), so all four
                    // warps do half of the exponentials each; the products go, as fp16, into a [token][output]
                    // tile in shared memory and leave as 16-byte vectors (eight lanes per 128-byte row).
                    constexpr int H = CH / 2;
                    const bool is_gate = row < 64;
                    const int fl = row & 63;
                    // gate -> up: gate values of tokens [H, CH); up -> gate: up values of tokens [0, H)
                    const uint32_t send = out_stage + (is_gate ? 0 : H * 64 * 4) + fl * 4;
                    const uint32_t recv = out_stage + (is_gate ? H * 64 * 4 : 0) + fl * 4;
#pragma unroll
                    for (int jj = 0; jj < H; ++jj)
                        asm volatile("st.shared.u32 [%0], %1;" ::"r"(send + jj * 64 * 4), "r"(is_gate ? v[H + jj] : v[jj])
                                     : "memory");
                    named_barrier_sync(3, 128);
                    float act[H];
#pragma unroll
                    for (int jj = 0; jj < H; ++jj) {
                        uint32_t other;
                        asm volatile("ld.shared.u32 %0, [%1];" : "=r"(other) : "r"(recv + jj * 64 * 4) : "memory");
                        const float gv = __uint_as_float(is_gate ? v[jj] : other);
                        const float uv = __uint_as_float(is_gate ? other : v[H + jj]);
                        const float gte = p.in_scale * gv;
                        act[jj] = p.alpha * __fdividef(gte, 1.f + __expf(-gte)) * (p.in_scale * uv);
                    }
                    named_barrier_sync(3, 128);  // every value sent has been read: the buffer becomes the output tile
                    const int tb = is_gate ? 0 : H;  // first token (inside the chunk) this thread computed
#pragma unroll
                    for (int jj = 0; jj < H; jj += 2) {
                        const __half2 h2 = __floats2half2_rn(act[jj], act[jj + 1]);
                        const uint32_t hb = *reinterpret_cast<const uint32_t*>(&h2);
                        asm volatile("st.shared.u16 [%0], %1;" ::"r"(out_stage + ((tb + jj) * 64 + fl) * 2),
                                     "h"(static_cast<unsigned short>(hb & 0xffffu))
                                     : "memory");
                        asm volatile("st.shared.u16 [%0], %1;" ::"r"(out_stage + ((tb + jj + 1) * 64 + fl) * 2),
                                     "h"(static_cast<unsigned short>(hb >> 16))
                                     : "memory");
                    }
                    named_barrier_sync(3, 128);
                    const int ldo = p.N / 2;
#pragma unroll
                    for (int ps = 0; ps < (CH * 8 + 127) / 128; ++ps) {
                        const int idx = ps * 128 + et;  // 16-byte vector of the CH x 64 tile
                        const int r = idx >> 3;
                        const int cv = (idx & 7) * 8;
                        if (r < CH) {
                            uint4 val;
                            asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                                         : "=r"(val.x), "=r"(val.y), "=r"(val.z), "=r"(val.w)
                                         : "r"(out_stage + (r * 64 + cv) * 2)
                                         : "memory");
                            const int t = t0 + c * CH + r;
                            const int ff = nt * 64 + cv;  // the output has N / 2 columns, a multiple of 64
                            if (t < p.M && ff < ldo && WB_DEBUG_INDEX(t >= 0 && ff >= 0 && ff + 8 <= ldo, p.status, 103, ff))
                                *reinterpret_cast<uint4*>(p.C16 + static_cast<size_t>(t) * ldo + ff) = val;
                        }
                    }
                    named_barrier_sync(3, 128);  // the tile is rewritten by the next chunk
                } else {
                    // fused gate/up with an output that is not 16-byte aligned: the up warps pass their values
                    // through shared memory, the gate warps compute and store element by element
                    if (row >= 64) {
#pragma unroll
                        for (int j = 0; j < CH; ++j)
                            asm volatile("st.shared.u32 [%0], %1;" ::"r"(out_stage + (j * 64 + row - 64) * 4), "r"(v[j])
                                         : "memory");
                    }
                    named_barrier_sync(3, 128);
                    if (row < 64) {
                        const int f = nt * 64 + row;
                        const int ldo = p.N / 2;
#pragma unroll
                        for (int j = 0; j < CH; ++j) {
                            uint32_t ub;
                            asm volatile("ld.shared.u32 %0, [%1];" : "=r"(ub) : "r"(out_stage + (j * 64 + row) * 4) : "memory");
                            const float gte = p.in_scale * __uint_as_float(v[j]);
                            const float act = p.alpha * (gte / (1.f + __expf(-gte))) * (p.in_scale * __uint_as_float(ub));
                            const int t = t0 + c * CH + j;
                            if (t < p.M && f < ldo) p.C16[static_cast<size_t>(t) * ldo + f] = __float2half_rn(act);
                        }
                    }
                    named_barrier_sync(3, 128);
                }
            }
            tc_fence_before_sync();
            mbar_arrive(acc_empty(acc));
            acc ^= 1;
            if (acc == 0) acc_ph ^= 1u;

            if (p.block_done != nullptr && nsl == 1) {
                // tell whoever follows this kernel that one more column tile of token block tt is in
                // memory: the barrier orders the 128 threads' stores before thread 0's system-scope
                // fence (the readers may sit behind NVLink), which is cumulative over them
                named_barrier_sync(1, 128);
                if (et == 0) {
                    __threadfence_system();
                    atomicAdd(p.block_done + tt, 1);
                }
            }
            if (nsl > 1) {
                // the last slice of this tile to finish sums all partials in slice order
                // One release for the whole CTA: the barrier orders the 128 threads' partial stores
                // before thread 0's gpu-scope fence, which is cumulative over them.
                named_barrier_sync(1, 128);
                if (et == 0) {
                    __threadfence();
                    const int old = atomicAdd(p.counters + tile_id, 1);
                    const uint32_t last = (old == nsl - 1) ? 1u : 0u;
                    if (last) p.counters[tile_id] = 0;  // ready for the next call
                    asm volatile("st.shared.u32 [%0], %1;" ::"r"(flag_slot), "r"(last) : "memory");
                }
                named_barrier_sync(1, 128);
                uint32_t last;
                asm volatile("ld.shared.u32 %0, [%1];" : "=r"(last) : "r"(flag_slot) : "memory");
                if (last) {
                    __threadfence();
                    const float* base = p.partials + static_cast<size_t>(tile_id) * p.max_slices * (BT * 128);
                    const int t_count = min(BT, p.M - t0);
                    if (n < p.N) {
                        // eight tokens at a time so that the loads of a slice are all in flight
                        // together; every element is still summed in ascending slice order
                        for (int tb = 0; tb < t_count; tb += 8) {
                            float sum[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                            for (int s2 = 0; s2 < nsl; ++s2) {
                                float v[8];
#pragma unroll
                                for (int u = 0; u < 8; ++u)
                                    v[u] = (tb + u < t_count)
                                               ? __ldcg(base + (static_cast<size_t>(s2) * BT + tb + u) * 128 + row)
                                               : 0.f;
#pragma unroll
                                for (int u = 0; u < 8; ++u) sum[u] += v[u];
                            }
#pragma unroll
                            for (int u = 0; u < 8; ++u)
                                if (tb + u < t_count) p.C[static_cast<size_t>(t0 + tb + u) * p.N + n] = sum[u];
                        }
                    }
                }
                named_barrier_sync(1, 128);  // flag_slot is reused by the next unit
            }
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == 2) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
    }
}

// ------------------------------------------------------------------ prepack / unpack / dequant
__device__ __constant__ int kNibbleK[8] = {0, 2, 4, 6, 1, 3, 5, 7};

// grid (K/64, N_pad/128), block 128: thread r packs column n = 128*nt + r of k-block kb.
__global__ void __launch_bounds__(128)
int4_prepack_kernel(const uint8_t* __restrict__ codes, uint32_t* __restrict__ q, int K, int N) {
    const int kb = blockIdx.x, nt = blockIdx.y, r = threadIdx.x;
    const int n = nt * 128 + r;
    uint32_t words[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        uint32_t w = 0;
#pragma unroll
        for (int pnib = 0; pnib < 8; ++pnib) {
            const int k = kb * 64 + j * 8 + kNibbleK[pnib];
            const uint32_t c = (n < N) ? (codes[static_cast<size_t>(k) * N + n] & 0xFu) : 0u;
            w |= c << (4 * pnib);
        }
        words[j] = w;
    }
    uint4* dst = reinterpret_cast<uint4*>(q + (static_cast<size_t>(kb) * gridDim.y + nt) * 1024 + r * 8);
    dst[0] = make_uint4(words[0], words[1], words[2], words[3]);
    dst[1] = make_uint4(words[4], words[5], words[6], words[7]);
}

// mode 0: codes uint8 [K,N]; mode 1: fp16 weights [K,N] = (code - 8) * scale[k/group][n]
template <int MODE>
__global__ void __launch_bounds__(128)
int4_unpack_kernel(const uint32_t* __restrict__ q, const __half* __restrict__ scales, void* out, int K,
                   int N, int group) {
    const int kb = blockIdx.x, nt = blockIdx.y, r = threadIdx.x;
    const int n = nt * 128 + r;
    if (n >= N) return;
    const uint4* src = reinterpret_cast<const uint4*>(q + (static_cast<size_t>(kb) * gridDim.y + nt) * 1024 + r * 8);
    const uint4 a = src[0], b = src[1];
    const uint32_t words[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
#pragma unroll
        for (int pnib = 0; pnib < 8; ++pnib) {
            const int k = kb * 64 + j * 8 + kNibbleK[pnib];
            const uint32_t c = (words[j] >> (4 * pnib)) & 0xFu;
            if constexpr (MODE == 0) {
                static_cast<uint8_t*>(out)[static_cast<size_t>(k) * N + n] = static_cast<uint8_t>(c);
            } else {
                const __half s = scales[static_cast<size_t>(k / group) * N + n];
                const __half v = __hmul(__int2half_rn(static_cast<int>(c) - 8), s);
                static_cast<__half*>(out)[static_cast<size_t>(k) * N + n] = v;
            }
        }
    }
}

static int w4_pick_bt(int M) {
    if (M <= 16) return 16;
    if (M <= 32) return 32;
    if (M <= 64) return 64;
    if (M <= 128) return 128;
    return 256;
}

static int w4_select_split(int M, int N, int K, int sms) {
    // Measured on B200 (N = 11008, K = 4096, M = 1..128): cutting K into slices never paid for
    // itself (each slice adds a partial-sum hand-over worth about 25 k-blocks); the balanced plan
    // in w4_make_plan covers the case of too few column tiles. An explicit split_k still works.
    (void)M; (void)N; (void)K; (void)sms;
    return 1;
}

// Products with few activation rows and no explicit K split go to the streaming decode kernel.
static bool w4_use_stream(int M, int N, int K, int split_k) {
    const long long blocks = static_cast<long long>((N + W4_TILE_N - 1) / W4_TILE_N) * (K / W4_BK);
    return M >= 1 && M <= W4_STREAM_MAX_M && split_k == 0 && blocks < (1ll << 30);
}


// How a product is cut into work units.
struct W4Plan {
    int bt, n_tiles, t_tiles, kb_total;
    int split;       // K-slices per tile in the classic plan
    int balanced;    // 1: equal runs of 8-block chunks per CTA (see w4_unit)
    int max_slices;  // slices a tile can have
    int grid;
    bool partials() const { return balanced || split > 1; }
    size_t workspace_bytes() const {
        if (!partials()) return 0;
        const int tiles = n_tiles * t_tiles;
        return w4_counter_bytes(tiles) + static_cast<size_t>(tiles) * max_slices * bt * 128 * sizeof(float);
    }
};

static W4Plan w4_make_plan(int M, int N, int K, int split_k, int sms) {
    W4Plan pl;
    pl.bt = w4_pick_bt(M);
    pl.n_tiles = (N + 127) / 128;
    pl.t_tiles = (M + pl.bt - 1) / pl.bt;
    pl.kb_total = K / 64;
    pl.balanced = 0;
    // Balanced plan only when the column tiles alone would leave most SMs idle: measured on B200
    // (K = 4096) its partial-sum hand-over costs about as much as 25 k-blocks, so with 86 tiles on
    // 148 SMs the plain plan (one whole tile per CTA) is as fast and needs no workspace.
    if (split_k == 0 && pl.bt <= 32 && pl.t_tiles == 1 && pl.kb_total % W4_CHUNK == 0 && pl.kb_total >= 2 * W4_CHUNK &&
        2 * pl.n_tiles <= sms) {
        // deal chunks of 8 k-blocks to the SMs in equal runs
        const int cpt = pl.kb_total / W4_CHUNK;
        const long long total_chunks = static_cast<long long>(cpt) * pl.n_tiles;
        pl.grid = total_chunks < sms ? static_cast<int>(total_chunks) : sms;
        const int per = static_cast<int>(total_chunks / pl.grid);  // >= 1
        pl.balanced = 1;
        pl.split = 1;
        pl.max_slices = (cpt + per - 1) / per + 1;
        return pl;
    }
    int split = split_k == 0 ? w4_select_split(M, N, K, sms) : split_k;
    if (split < 1) split = 1;
    if (split > pl.kb_total) split = pl.kb_total;
    pl.split = split;
    pl.max_slices = split;
    const long long units = static_cast<long long>(pl.n_tiles) * pl.t_tiles * split;
    pl.grid = units < sms ? static_cast<int>(units) : sms;
    return pl;
}

template <int BT, bool WM>
static int launch_w4(const CUtensorMap& tx, const CUtensorMap& tw, const CUtensorMap& tsc, const W4Params& p,
                     int grid, cudaStream_t stream) {
    using Cfg = W4Cfg<BT, WM>;
    static std::atomic<bool> attr_set[64];  // per device; setting the attribute twice is harmless
    int dev = 0;
    WB_CHECK_CUDA(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64 && !attr_set[dev].load(std::memory_order_acquire)) {
        WB_CHECK_CUDA(cudaFuncSetAttribute(w4a16_gemm_kernel<BT, WM>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES));
        attr_set[dev].store(true, std::memory_order_release);
    }
    w4a16_gemm_kernel<BT, WM><<<grid, W4_THREADS, Cfg::SMEM_BYTES, stream>>>(tx, tw, tsc, p);
    WB_CHECK_CUDA(cudaGetLastError());
    return WMMA_OPS_OK;
}

static int check_w4_shape(int K, int N) {
    WB_REQUIRE(K >= 64 && K % 64 == 0, WMMA_OPS_ERR_INVALID, "K must be a positive multiple of 64 (got K=%d)", K);
    WB_REQUIRE(N >= 8 && N % 8 == 0, WMMA_OPS_ERR_INVALID, "N must be a positive multiple of 8 (got N=%d)", N);
    return WMMA_OPS_OK;
}

}  // namespace wb

extern "C" int wmma_ops_int4_prepack(const void* codes_u8, void* qweight, int K, int N, void* stream) {
    using namespace wb;
    int rc = check_w4_shape(K, N);
    if (rc != WMMA_OPS_OK) return rc;
    WB_REQUIRE(codes_u8 != nullptr && qweight != nullptr, WMMA_OPS_ERR_INVALID, "int4_prepack: null pointer");
    WB_REQUIRE(reinterpret_cast<uintptr_t>(qweight) % 16 == 0, WMMA_OPS_ERR_INVALID, "qweight must be 16-byte aligned");
    dim3 grid(K / 64, (N + 127) / 128);
    int4_prepack_kernel<<<grid, 128, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint8_t*>(codes_u8), static_cast<uint32_t*>(qweight), K, N);
    WB_CHECK_CUDA(cudaGetLastError());
    return WMMA_OPS_OK;
}

extern "C" int wmma_ops_int4_unpack(const void* qweight, void* codes_u8, int K, int N, void* stream) {
    using namespace wb;
    int rc = check_w4_shape(K, N);
    if (rc != WMMA_OPS_OK) return rc;
    WB_REQUIRE(codes_u8 != nullptr && qweight != nullptr, WMMA_OPS_ERR_INVALID, "int4_unpack: null pointer");
    dim3 grid(K / 64, (N + 127) / 128);
    int4_unpack_kernel<0><<<grid, 128, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint32_t*>(qweight), nullptr, codes_u8, K, N, 1);
    WB_CHECK_CUDA(cudaGetLastError());
    return WMMA_OPS_OK;
}

extern "C" int wmma_ops_int4_dequant(const void* qweight, const void* scales, void* W_f16, int K, int N,
                                     int group_size, void* stream) {
    using namespace wb;
    int rc = check_w4_shape(K, N);
    if (rc != WMMA_OPS_OK) return rc;
    WB_REQUIRE(qweight != nullptr && scales != nullptr && W_f16 != nullptr, WMMA_OPS_ERR_INVALID,
               "int4_dequant: null pointer");
    WB_REQUIRE(group_size > 0 && K % group_size == 0, WMMA_OPS_ERR_INVALID,
               "group_size must divide K (got group_size=%d, K=%d)", group_size, K);
    dim3 grid(K / 64, (N + 127) / 128);
    int4_unpack_kernel<1><<<grid, 128, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint32_t*>(qweight), static_cast<const __half*>(scales), W_f16, K, N, group_size);
    WB_CHECK_CUDA(cudaGetLastError());
    return WMMA_OPS_OK;
}

extern "C" int wmma_ops_w4a16_select_split(int M, int N, int K, int num_sms) {
    if (M < 1 || N < 8 || K < 64) return 1;
    return wb::w4_select_split(M, N, K, num_sms > 0 ? num_sms : 148);
}

extern "C" size_t wmma_ops_w4a16_workspace_bytes(int M, int N, int K, int split_k) {
    if (M < 1 || N < 8 || K < 64 || K % 64 != 0) return 0;
    if (wb::w4_use_stream(M, N, K, split_k)) return 0;  // the decode kernel keeps its sums on chip
    return wb::w4_make_plan(M, N, K, split_k, wb::sm_count()).workspace_bytes();
}

extern "C" int wmma_ops_w4a16_gemm(const void* A, const void* qweight, const void* scales, void* C, int M,
                                   int N, int K, int group_size, int split_k, void* workspace,
                                   size_t workspace_bytes, int* status, void* stream_) {
    return wmma_ops_w4a16_gemm_ex(A, qweight, scales, C, M, N, K, group_size, split_k, WMMA_OPS_W4_OUT_F32, 1.0f, 1.0f,
                                  workspace, workspace_bytes, status, stream_);
}

extern "C" int wmma_ops_w4a16_token_block(int M) { return wb::w4_pick_bt(M < 1 ? 1 : M); }

extern "C" int wmma_ops_w4a16_gemm_blocks(const void* A, const void* qweight, const void* scales, void* C, int M,
                                          int N, int K, int group_size, int split_k, int out_mode, float alpha,
                                          float in_scale, void* workspace, size_t workspace_bytes, int* block_done,
                                          int* status, void* stream_);

extern "C" int wmma_ops_w4a16_gemm_ex(const void* A, const void* qweight, const void* scales, void* C, int M,
                                      int N, int K, int group_size, int split_k, int out_mode, float alpha, float in_scale,
                                      void* workspace, size_t workspace_bytes, int* status, void* stream_) {
    return wmma_ops_w4a16_gemm_blocks(A, qweight, scales, C, M, N, K, group_size, split_k, out_mode, alpha, in_scale,
                                      workspace, workspace_bytes, nullptr, status, stream_);
}

extern "C" int wmma_ops_w4a16_gemm_blocks(const void* A, const void* qweight, const void* scales, void* C, int M,
                                          int N, int K, int group_size, int split_k, int out_mode, float alpha,
                                          float in_scale, void* workspace, size_t workspace_bytes, int* block_done,
                                          int* status, void* stream_) {
    using namespace wb;
    WB_REQUIRE(block_done == nullptr || (M > W4_STREAM_MAX_M && split_k <= 1), WMMA_OPS_ERR_INVALID,
               "w4a16: block completion counters are for products with more than %d rows and no K split", W4_STREAM_MAX_M);
    WB_REQUIRE(out_mode >= WMMA_OPS_W4_OUT_F32 && out_mode <= WMMA_OPS_W4_OUT_F16_SILU_MUL, WMMA_OPS_ERR_INVALID,
               "w4a16: unknown out_mode %d", out_mode);
    WB_REQUIRE(out_mode != WMMA_OPS_W4_OUT_F16_SILU_MUL || N % 128 == 0, WMMA_OPS_ERR_INVALID,
               "w4a16: the fused gate/up epilogue needs N to be a multiple of 128 (got N=%d)", N);
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    WB_REQUIRE(M >= 0, WMMA_OPS_ERR_INVALID, "w4a16: negative M");
    int rc = check_w4_shape(K, N);
    if (rc != WMMA_OPS_OK) return rc;
    if (M == 0) return WMMA_OPS_OK;
    WB_REQUIRE(group_size >= 64 && group_size % 64 == 0 && K % group_size == 0, WMMA_OPS_ERR_INVALID,
               "group_size must be a multiple of 64 that divides K (got group_size=%d, K=%d)", group_size, K);
    WB_REQUIRE(A != nullptr && qweight != nullptr && scales != nullptr && C != nullptr, WMMA_OPS_ERR_INVALID,
               "w4a16: null pointer");
    WB_REQUIRE(reinterpret_cast<uintptr_t>(A) % 16 == 0, WMMA_OPS_ERR_INVALID, "A must be 16-byte aligned");
    WB_REQUIRE(reinterpret_cast<uintptr_t>(qweight) % 16 == 0, WMMA_OPS_ERR_INVALID,
               "qweight must be 16-byte aligned");
    WB_REQUIRE(reinterpret_cast<uintptr_t>(scales) % 16 == 0, WMMA_OPS_ERR_INVALID,
               "scales must be 16-byte aligned");

    const int sms = sm_count();
    // fp16 and fused outputs of the tcgen05 kernel come straight from the accumulators
    if (split_k == 0 && out_mode != WMMA_OPS_W4_OUT_F32 && !w4_use_stream(M, N, K, split_k)) split_k = 1;
    const W4Plan plan = w4_make_plan(M, N, K, split_k, sms);
    const int bt = plan.bt;
    W4Params p;
    p.X = static_cast<const __half*>(A);
    p.qweight = static_cast<const uint32_t*>(qweight);
    p.scales = static_cast<const __half*>(scales);
    p.C = static_cast<float*>(C);
    p.C16 = static_cast<__half*>(C);
    p.out_mode = out_mode;
    p.alpha = alpha;
    p.in_scale = in_scale;
    p.M = M;
    p.N = N;
    p.K = K;
    p.n_tiles = plan.n_tiles;
    p.t_tiles = plan.t_tiles;
    p.kb_total = plan.kb_total;
    p.group_kb = group_size / 64;
    p.group_shift = -1;
    for (int sh = 0; sh < 24; ++sh)
        if ((1 << sh) == p.group_kb) p.group_shift = sh;
    p.status = status;
    p.block_done = block_done;
    // Order of the units. Token block by token block (all column tiles of a block, then the next block) when
    // a consumer follows the kernel block by block, and also whenever the packed weights are the smaller
    // operand (K N / 2 bytes against 2 M K): the CTAs of a wave then share one or a few activation tiles and
    // re-read the weights, which stay in the L2, instead of sharing a few weight tiles and re-reading all
    // activations from memory every wave (measured at 8192 x 4096 x 4096: L2 hit rate 74 -> 91 %, DRAM
    // throughput 22 -> 6 % of peak, 240 -> 234 us).
#ifdef W4_ORDER_OLD
    p.tt_major = block_done != nullptr ? 1 : 0;
#else
    p.tt_major = (block_done != nullptr || static_cast<long long>(N) <= 4ll * M) ? 1 : 0;
#endif
    p.split = plan.split;
    p.balanced = plan.balanced;
    p.max_slices = plan.max_slices;
    p.partials = nullptr;
    p.counters = nullptr;
    if (w4_use_stream(M, N, K, split_k)) {
        // decode: one pass over the packed weights, every CTA owning a range of columns
        const W4DecodePlan dp = w4_decode_plan(M, N, K, group_size, out_mode, sms);
        p.n_tiles = dp.n_tiles;
        p.t_tiles = 1;
        p.kb_total = dp.kb_total;
        p.split = 1;
        p.balanced = 0;
        p.max_slices = 1;
        return w4_decode_launch(p, dp, stream);
    }
    WB_REQUIRE(block_done == nullptr || !plan.partials(), WMMA_OPS_ERR_INVALID,
               "w4a16: block completion counters need a plan without partial sums (pass split_k = 1)");
    WB_REQUIRE(out_mode == WMMA_OPS_W4_OUT_F32 || !plan.partials(), WMMA_OPS_ERR_INVALID,
               "w4a16: fp16 / fused outputs need a plan without partial sums (pass split_k = 1)");
    if (plan.partials()) {
        const size_t need = plan.workspace_bytes();
        WB_REQUIRE(workspace != nullptr && workspace_bytes >= need, WMMA_OPS_ERR_WORKSPACE,
                   "w4a16: this product is cut into partial sums and needs %zu bytes of zero-initialised workspace "
                   "(got %zu); see wmma_ops_w4a16_workspace_bytes",
                   need, workspace_bytes);
        WB_REQUIRE(reinterpret_cast<uintptr_t>(workspace) % 16 == 0, WMMA_OPS_ERR_INVALID,
                   "workspace must be 16-byte aligned");
        p.counters = static_cast<int*>(workspace);
        p.partials = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) +
                                              w4_counter_bytes(p.n_tiles * p.t_tiles));
    }
    CUtensorMap tx;
    rc = encode_tmap_2d(&tx, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, A, static_cast<uint64_t>(K),
                        static_cast<uint64_t>(M), static_cast<uint64_t>(K) * 2, W4_BK, bt,
                        CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != WMMA_OPS_OK) return rc;
    // qweight seen as int32 [4 * blocks][256]: one 4 KB block = a box of 4 rows x 1 KB
    CUtensorMap tw, tsc;
    rc = encode_tmap_2d(&tw, CU_TENSOR_MAP_DATA_TYPE_INT32, qweight, 256,
                        static_cast<uint64_t>(p.n_tiles) * p.kb_total * 4, 1024, 256, 4, CU_TENSOR_MAP_SWIZZLE_NONE);
    if (rc != WMMA_OPS_OK) return rc;
    rc = encode_tmap_2d(&tsc, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, scales, static_cast<uint64_t>(N),
                        static_cast<uint64_t>(K / group_size), static_cast<uint64_t>(N) * 2, W4_TILE_N, 1,
                        CU_TENSOR_MAP_SWIZZLE_NONE);
    if (rc != WMMA_OPS_OK) return rc;
    // decode mode (workers issue their own MMAs) needs every unit to give each of the eight
    // workers at least one block; the balanced plan's units are whole 8-block chunks
    const bool wm = bt <= 32 && (plan.balanced || (p.kb_total / p.split) >= 8);
    const int grid = plan.grid;
    switch (bt) {
        case 16: return wm ? launch_w4<16, true>(tx, tw, tsc, p, grid, stream) : launch_w4<16, false>(tx, tw, tsc, p, grid, stream);
        case 32: return wm ? launch_w4<32, true>(tx, tw, tsc, p, grid, stream) : launch_w4<32, false>(tx, tw, tsc, p, grid, stream);
        case 64: return launch_w4<64, false>(tx, tw, tsc, p, grid, stream);
        case 128: return launch_w4<128, false>(tx, tw, tsc, p, grid, stream);
        default: return launch_w4<256, false>(tx, tw, tsc, p, grid, stream);
    }
}
