// INT4 weight prepack ("W4-B200-v1") and the fused W4A16 GEMM for sm_100a.
//
// The reference snapshot has no INT4 code; the entry points, the packed format and the
// arithmetic  C[M,N] = A[M,K] . ((code - 8) * scale[k / group][n])  are specified here and
// restated on the CPU in oracle/int4.py.
//
// Packed format: uint32 [N_pad/128][K/64][128][8].  Block (nt, kb) is 4 KB and holds, for the
// 128 weight columns n = 128 nt + r, the 64 codes k = 64 kb .. 64 kb + 63 as 8 words per
// column; word j, nibble p holds k = 64 kb + 8 j + {0,2,4,6,1,3,5,7}[p].  A CTA streams the
// blocks of one column tile as contiguous 4 KB bulk copies, so HBM sees long sequential reads.
//
// Kernel: the weights sit on the 128-row side of the MMA (it computes C^T = W^T . A^T):
//   A operand  = dequantised W^T tile, 128 columns-of-W x 64 k, fp16, K-major, 128-byte swizzle,
//                written to shared memory by eight dequant warps (never to global memory);
//   B operand  = activation tile, BT tokens x 64 k, loaded by TMA straight from A [M,K];
//   accumulator = 128 TMEM lanes (weight columns) x BT columns (tokens), fp32.
// One weight element is dequantised once per 256 tokens, so the same kernel serves decode
// (M = 1..16, HBM-bound) and prefill (M in the thousands, tensor-bound).
// Warps: 0 raw-weight producer, 1 activation producer, 2 MMA issuer + TMEM owner, 3 idle,
// 4..11 dequant (each expands every eighth 4 KB block), 12..15 epilogue.  Split-K partials are combined by the last CTA to finish a
// tile (arrival counter, no waiting), summed in ascending slice order.
#include "host_common.cuh"
#include "ptx.cuh"

namespace wb {

constexpr int W4_TILE_N = 128;     // weight columns per CTA tile (MMA M)
constexpr int W4_BK = 64;          // k per pipeline step
constexpr int W4_RAW_BYTES = 4096; // one packed block
constexpr int W4_WT_BYTES = W4_TILE_N * W4_BK * 2;
constexpr int W4_THREADS = 512;
constexpr int W4_DQ_WARPS = 8;     // each dequant warp expands a whole 4 KB block; 8 blocks in flight

template <int BT>
struct W4Cfg {
    static constexpr int X_BYTES = BT * W4_BK * 2;
    static constexpr int S_STAGE = W4_WT_BYTES + X_BYTES;
    // Wt + X ring. One dequant warp owns each stage (DQ = S), and the raw ring is a multiple
    // of S, so every barrier is waited on by the same warp pass after pass: a parity wait can
    // then never be more than one phase away from the barrier's state.
    static constexpr int S = (BT >= 256) ? 4 : (BT >= 128) ? 6 : 8;
    static constexpr int R = (BT >= 256) ? 8 : (BT >= 128) ? 6 : (BT >= 32) ? 8 : 16;
    static constexpr int DQ = S;
    static_assert(R % S == 0 && DQ <= W4_DQ_WARPS, "ring sizes must nest");
    static constexpr int TMEM_COLS = (2 * BT < 32) ? 32 : 2 * BT;
    static constexpr int SMEM_BYTES = S * S_STAGE + R * W4_RAW_BYTES + 1024 + 512;
};

struct W4Params {
    const uint32_t* qweight;
    const __half* scales;
    float* C;
    float* partials;   // [tiles][split][BT][128]
    int* counters;     // [tiles]
    int M, N, K;
    int n_tiles, t_tiles, split;
    int kb_total;
    int group_kb;      // k-blocks per scale group (group_size / 64)
    int* status;
};

__device__ __forceinline__ void w4_report(int* status, int role, int detail) {
    if (status != nullptr && atomicCAS(status, 0, 2) == 0) {
        status[1] = role;
        status[2] = static_cast<int>(blockIdx.x);
        status[3] = detail;
    }
}

__device__ __forceinline__ void w4_decode(const W4Params& p, int unit, int& nt, int& tt, int& sl,
                                          int& kb0, int& kb1) {
    sl = unit % p.split;
    const int t = unit / p.split;
    tt = t % p.t_tiles;
    nt = t / p.t_tiles;
    kb0 = static_cast<int>(static_cast<long long>(sl) * p.kb_total / p.split);
    kb1 = static_cast<int>(static_cast<long long>(sl + 1) * p.kb_total / p.split);
}

// Position of a dequant warp in the CTA's sequence of k-block iterations.
struct W4Cursor {
    int unit, nt, kb, kb1;
    bool valid;
};

__device__ __forceinline__ void w4_cursor_start(const W4Params& p, int total_units, W4Cursor& c) {
    c.unit = blockIdx.x;
    c.valid = c.unit < total_units;
    if (c.valid) {
        int tt, sl, kb0;
        w4_decode(p, c.unit, c.nt, tt, sl, kb0, c.kb1);
        c.kb = kb0;
    }
}

// Moves the cursor `steps` iterations forward, crossing into later work units as needed.
__device__ __forceinline__ void w4_cursor_advance(const W4Params& p, int total_units, W4Cursor& c,
                                                  int steps) {
    if (!c.valid) return;
    c.kb += steps;
    while (c.kb >= c.kb1) {
        const int over = c.kb - c.kb1;
        c.unit += gridDim.x;
        if (c.unit >= total_units) {
            c.valid = false;
            return;
        }
        int tt, sl, kb0;
        w4_decode(p, c.unit, c.nt, tt, sl, kb0, c.kb1);
        c.kb = kb0 + over;
    }
}

// (code - 8) * scale for the two codes that sit 16 bits apart in t (already masked):
// 0x6400 | code is the fp16 number 1024 + code, so subtracting 1032 gives code - 8 exactly;
// the product is one fp16 multiply (round to nearest even).
__device__ __forceinline__ uint32_t dq_pair(uint32_t t, __half2 scale2) {
    const uint32_t h = t | 0x64006400u;
    const __half2 v = __hsub2(*reinterpret_cast<const __half2*>(&h), __half2half2(__ushort_as_half(0x6408)));
    const __half2 r = __hmul2(v, scale2);
    return *reinterpret_cast<const uint32_t*>(&r);
}

__device__ __forceinline__ void dq_word_store(uint32_t dst, uint32_t w, __half2 scale2) {
    const uint32_t a = dq_pair(w & 0x000F000Fu, scale2);
    const uint32_t b = dq_pair((w >> 4) & 0x000F000Fu, scale2);
    const uint32_t c = dq_pair((w >> 8) & 0x000F000Fu, scale2);
    const uint32_t d = dq_pair((w >> 12) & 0x000F000Fu, scale2);
    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(a), "r"(b), "r"(c), "r"(d)
                 : "memory");
}

// The eight scales one lane needs for a block: rows 16 q + lane / 2, q = 0..7.
__device__ __forceinline__ void w4_load_scales(const W4Params& p, const W4Cursor& c, int lane,
                                               __half (&sc)[8]) {
    const int grp = c.kb / p.group_kb;
    const __half* base = p.scales + static_cast<size_t>(grp) * p.N;
#pragma unroll
    for (int q = 0; q < 8; ++q) {
        const int n = c.nt * W4_TILE_N + 16 * q + (lane >> 1);
        sc[q] = (n < p.N) ? __ldg(base + n) : __ushort_as_half(0);
    }
}

template <int BT>
__global__ void __launch_bounds__(W4_THREADS, 1)
w4a16_gemm_kernel(const __grid_constant__ CUtensorMap tmap_x, const W4Params p) {
    using Cfg = W4Cfg<BT>;
    extern __shared__ uint8_t smem_raw_[];
    const uint32_t smem_base = (smem_u32(smem_raw_) + 1023u) & ~1023u;
    const uint32_t raw_base = smem_base + Cfg::S * Cfg::S_STAGE;
    const uint32_t bar_base = raw_base + Cfg::R * W4_RAW_BYTES;
    auto x_full = [&](int s) { return bar_base + 8u * s; };
    auto wt_full = [&](int s) { return bar_base + 8u * (Cfg::S + s); };
    auto st_empty = [&](int s) { return bar_base + 8u * (2 * Cfg::S + s); };
    auto raw_full = [&](int r) { return bar_base + 8u * (3 * Cfg::S + r); };
    auto raw_empty = [&](int r) { return bar_base + 8u * (3 * Cfg::S + Cfg::R + r); };
    auto acc_full = [&](int b) { return bar_base + 8u * (3 * Cfg::S + 2 * Cfg::R + b); };
    auto acc_empty = [&](int b) { return bar_base + 8u * (3 * Cfg::S + 2 * Cfg::R + 2 + b); };
    const uint32_t tmem_slot = bar_base + 8u * (3 * Cfg::S + 2 * Cfg::R + 4);
    const uint32_t flag_slot = tmem_slot + 8u;
    static_assert(8 * (3 * Cfg::S + 2 * Cfg::R + 6) <= 512, "barrier area too small");

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < Cfg::S; ++s) {
            mbar_init(x_full(s), 1);
            mbar_init(wt_full(s), 1);
            mbar_init(st_empty(s), 1);
        }
        for (int r = 0; r < Cfg::R; ++r) {
            mbar_init(raw_full(r), 1);
            mbar_init(raw_empty(r), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(acc_full(b), 1);
            mbar_init(acc_empty(b), 128);
        }
        fence_barrier_init();
        fence_proxy_async_smem();
        prefetch_tmap(&tmap_x);
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

    const int total_units = p.n_tiles * p.t_tiles * p.split;

    if (warp == 0) {
        // ------------------------------------------------ raw packed-weight producer
        if (lane == 0) {
            int r = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int unit = blockIdx.x; ok && unit < total_units; unit += gridDim.x) {
                int nt, tt, sl, kb0, kb1;
                w4_decode(p, unit, nt, tt, sl, kb0, kb1);
                const uint32_t* src =
                    p.qweight + (static_cast<size_t>(nt) * p.kb_total + kb0) * (W4_RAW_BYTES / 4);
                for (int kb = kb0; kb < kb1; ++kb, src += W4_RAW_BYTES / 4) {
                    if (!mbar_wait(raw_empty(r), ph ^ 1u)) {
                        w4_report(p.status, 0, kb);
                        ok = false;
                        break;
                    }
                    mbar_arrive_expect_tx(raw_full(r), W4_RAW_BYTES);
                    bulk_load_1d(raw_base + r * W4_RAW_BYTES, src, W4_RAW_BYTES, raw_full(r));
                    if (++r == Cfg::R) {
                        r = 0;
                        ph ^= 1u;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------ activation producer
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int unit = blockIdx.x; ok && unit < total_units; unit += gridDim.x) {
                int nt, tt, sl, kb0, kb1;
                w4_decode(p, unit, nt, tt, sl, kb0, kb1);
                for (int kb = kb0; kb < kb1; ++kb) {
                    if (!mbar_wait(st_empty(s), ph ^ 1u)) {
                        w4_report(p.status, 1, kb);
                        ok = false;
                        break;
                    }
                    mbar_arrive_expect_tx(x_full(s), Cfg::X_BYTES);
                    tma_load_2d(smem_base + s * Cfg::S_STAGE + W4_WT_BYTES, &tmap_x, x_full(s),
                                kb * W4_BK, tt * BT);
                    if (++s == Cfg::S) {
                        s = 0;
                        ph ^= 1u;
                    }
                }
            }
        }
    } else if (warp == 2) {
        // ------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc_f16_f32(W4_TILE_N, BT, false, false);
            int s = 0;
            uint32_t ph = 0;
            int acc = 0;
            uint32_t acc_ph = 0;
            bool ok = true;
            for (int unit = blockIdx.x; ok && unit < total_units; unit += gridDim.x) {
                int nt, tt, sl, kb0, kb1;
                w4_decode(p, unit, nt, tt, sl, kb0, kb1);
                if (!mbar_wait(acc_empty(acc), acc_ph ^ 1u)) {
                    w4_report(p.status, 2, -1);
                    break;
                }
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + acc * BT;
                for (int kb = kb0; kb < kb1; ++kb) {
                    if (!mbar_wait(x_full(s), ph) || !mbar_wait(wt_full(s), ph)) {
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
                        umma_f16(d_tmem, a_desc, b_desc, idesc, (kb > kb0 || kk > 0) ? 1u : 0u);
                    }
                    umma_commit(st_empty(s));
                    if (++s == Cfg::S) {
                        s = 0;
                        ph ^= 1u;
                    }
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
        const int w = warp - 4;
        W4Cursor cur;
        w4_cursor_start(p, total_units, cur);
        w4_cursor_advance(p, total_units, cur, w);
        if (w >= Cfg::DQ) cur.valid = false;
        __half sc_cur[8], sc_next[8];
        if (cur.valid) w4_load_scales(p, cur, lane, sc_cur);
        for (int j = w; cur.valid; j += Cfg::DQ) {
            // the scales of this warp's next block are requested now and used an iteration later
            W4Cursor nxt = cur;
            w4_cursor_advance(p, total_units, nxt, Cfg::DQ);
            if (nxt.valid) w4_load_scales(p, nxt, lane, sc_next);

            const int r = j % Cfg::R;
            const int s = j % Cfg::S;
            const uint32_t ph_r = (j / Cfg::R) & 1;
            const uint32_t ph_s = (j / Cfg::S) & 1;
            if (!mbar_wait(raw_full(r), ph_r)) {
                w4_report(p.status, 3, j);
                break;
            }
            if (!mbar_wait(st_empty(s), ph_s ^ 1u)) {
                w4_report(p.status, 3, -j - 1);
                break;
            }
            const uint32_t raw = raw_base + r * W4_RAW_BYTES;
            const uint32_t wt = smem_base + s * Cfg::S_STAGE;
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                // lane reads bytes [16 i, 16 i + 16) of the block, i = 32 q + lane: row i / 2,
                // 16-byte half i % 2 (conflict-free loads; the swizzled stores are too)
                const int i = q * 32 + lane;
                const uint32_t row = i >> 1;
                const uint32_t c_base = (i & 1) * 4;
                uint4 v;
                asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                             : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                             : "r"(raw + i * 16)
                             : "memory");
                const __half2 scale2 = __half2half2(sc_cur[q]);
                dq_word_store(wt + sw128_offset(row, c_base + 0), v.x, scale2);
                dq_word_store(wt + sw128_offset(row, c_base + 1), v.y, scale2);
                dq_word_store(wt + sw128_offset(row, c_base + 2), v.z, scale2);
                dq_word_store(wt + sw128_offset(row, c_base + 3), v.w, scale2);
            }
            // Every lane's stores consumed its loaded registers, so all loads of the packed
            // block have completed; only now may the producer refill the slot.
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(raw_empty(r));
                mbar_arrive(wt_full(s));
            }
            cur = nxt;
#pragma unroll
            for (int q = 0; q < 8; ++q) sc_cur[q] = sc_next[q];
        }
    } else if (warp >= 12) {
        // ------------------------------------------------ epilogue warps
        const int quad = warp & 3;
        const int row = quad * 32 + lane;  // weight column inside the tile
        const int et = threadIdx.x - 384;  // 0..127
        int acc = 0;
        uint32_t acc_ph = 0;
        for (int unit = blockIdx.x; unit < total_units; unit += gridDim.x) {
            int nt, tt, sl, kb0, kb1;
            w4_decode(p, unit, nt, tt, sl, kb0, kb1);
            if (!mbar_wait(acc_full(acc), acc_ph)) {
                w4_report(p.status, 4, unit);
                break;
            }
            tc_fence_after_sync();
            const int n = nt * W4_TILE_N + row;
            const int t0 = tt * BT;
            const int tile_id = nt * p.t_tiles + tt;
            const uint32_t t_addr = tmem_base + acc * BT + (static_cast<uint32_t>(quad * 32) << 16);
            float* part = (p.split > 1)
                              ? p.partials + (static_cast<size_t>(tile_id) * p.split + sl) * (BT * 128)
                              : nullptr;
            constexpr int CH = (BT >= 32) ? 32 : 16;
#pragma unroll 1
            for (int c = 0; c < BT / CH; ++c) {
                uint32_t v[CH];
                if constexpr (CH == 32) tmem_ld_32x32b_x32(t_addr + c * CH, v);
                else tmem_ld_32x32b_x16(t_addr + c * CH, v);
                tmem_wait_ld();
                if (part != nullptr) {
#pragma unroll
                    for (int j = 0; j < CH; ++j) part[(c * CH + j) * 128 + row] = __uint_as_float(v[j]);
                } else if (n < p.N) {
#pragma unroll
                    for (int j = 0; j < CH; ++j) {
                        const int t = t0 + c * CH + j;
                        if (t < p.M) p.C[static_cast<size_t>(t) * p.N + n] = __uint_as_float(v[j]);
                    }
                }
            }
            tc_fence_before_sync();
            mbar_arrive(acc_empty(acc));
            acc ^= 1;
            if (acc == 0) acc_ph ^= 1u;

            if (p.split > 1) {
                // the last slice of this tile to finish sums all partials in slice order
                __threadfence();
                named_barrier_sync(1, 128);
                if (et == 0) {
                    const int old = atomicAdd(p.counters + tile_id, 1);
                    const uint32_t last = (old == p.split - 1) ? 1u : 0u;
                    if (last) p.counters[tile_id] = 0;  // ready for the next call
                    asm volatile("st.shared.u32 [%0], %1;" ::"r"(flag_slot), "r"(last) : "memory");
                }
                named_barrier_sync(1, 128);
                uint32_t last;
                asm volatile("ld.shared.u32 %0, [%1];" : "=r"(last) : "r"(flag_slot) : "memory");
                if (last) {
                    __threadfence();
                    const float* base = p.partials + static_cast<size_t>(tile_id) * p.split * (BT * 128);
                    const int t_count = min(BT, p.M - t0);
                    if (n < p.N) {
                        for (int t = 0; t < t_count; ++t) {
                            float sum = 0.f;
                            for (int s2 = 0; s2 < p.split; ++s2)
                                sum += __ldcg(base + (static_cast<size_t>(s2) * BT + t) * 128 + row);
                            p.C[static_cast<size_t>(t0 + t) * p.N + n] = sum;
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
    uint4* dst = reinterpret_cast<uint4*>(q + (static_cast<size_t>(nt) * (K / 64) + kb) * 1024 + r * 8);
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
    const uint4* src = reinterpret_cast<const uint4*>(q + (static_cast<size_t>(nt) * (K / 64) + kb) * 1024 + r * 8);
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
    const int bt = w4_pick_bt(M);
    const int tiles = ((N + 127) / 128) * ((M + bt - 1) / bt);
    const int kb_total = K / 64;
    // Measured on B200 (N=11008, K=4096): the partial-sum traffic and the serial reduce of the
    // last CTA cost more than the idle SMs save once a tile holds more than a few tokens.
    if (tiles >= sms || kb_total < 16 || M > 4) return 1;
    int best = 1;
    double best_cost = 0.0;
    const int max_split = kb_total / 8 < 16 ? kb_total / 8 : 16;
    for (int s = 1; s <= max_split; ++s) {
        const int units = tiles * s;
        const int waves = (units + sms - 1) / sms;
        const int per = (kb_total + s - 1) / s;
        // a unit costs its k-blocks plus a fixed fill/drain of about six k-blocks,
        // and each extra slice adds partial traffic proportional to the token tile
        const double cost = waves * (per + 6.0 + (s > 1 ? 0.02 * bt : 0.0));
        if (s == 1 || cost < best_cost) {
            best_cost = cost;
            best = s;
        }
    }
    return best;
}

static size_t w4_counter_bytes(int tiles) { return (static_cast<size_t>(tiles) * 4 + 255) / 256 * 256; }

template <int BT>
static int launch_w4(const CUtensorMap& tx, const W4Params& p, int sms, cudaStream_t stream) {
    using Cfg = W4Cfg<BT>;
    static bool attr_set[64] = {};
    int dev = 0;
    WB_CHECK_CUDA(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        WB_CHECK_CUDA(cudaFuncSetAttribute(w4a16_gemm_kernel<BT>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES));
        attr_set[dev] = true;
    }
    const int units = p.n_tiles * p.t_tiles * p.split;
    const int grid = units < sms ? units : sms;
    w4a16_gemm_kernel<BT><<<grid, W4_THREADS, Cfg::SMEM_BYTES, stream>>>(tx, p);
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
    (void)K;
    if (split_k <= 1 || M < 1 || N < 1) return 0;
    const int bt = wb::w4_pick_bt(M);
    const int tiles = ((N + 127) / 128) * ((M + bt - 1) / bt);
    return wb::w4_counter_bytes(tiles) + static_cast<size_t>(tiles) * split_k * bt * 128 * sizeof(float);
}

extern "C" int wmma_ops_w4a16_gemm(const void* A, const void* qweight, const void* scales, void* C, int M,
                                   int N, int K, int group_size, int split_k, void* workspace,
                                   size_t workspace_bytes, int* status, void* stream_) {
    using namespace wb;
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
    const int bt = w4_pick_bt(M);
    W4Params p;
    p.qweight = static_cast<const uint32_t*>(qweight);
    p.scales = static_cast<const __half*>(scales);
    p.C = static_cast<float*>(C);
    p.M = M;
    p.N = N;
    p.K = K;
    p.n_tiles = (N + 127) / 128;
    p.t_tiles = (M + bt - 1) / bt;
    p.kb_total = K / 64;
    p.group_kb = group_size / 64;
    p.status = status;
    if (split_k == 0) split_k = w4_select_split(M, N, K, sms);
    if (split_k < 1) split_k = 1;
    if (split_k > p.kb_total) split_k = p.kb_total;
    p.split = split_k;
    p.partials = nullptr;
    p.counters = nullptr;
    if (split_k > 1) {
        const size_t need = wmma_ops_w4a16_workspace_bytes(M, N, K, split_k);
        WB_REQUIRE(workspace != nullptr && workspace_bytes >= need, WMMA_OPS_ERR_WORKSPACE,
                   "w4a16: split_k=%d needs %zu bytes of zero-initialised workspace (got %zu)", split_k, need,
                   workspace_bytes);
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
    switch (bt) {
        case 16: return launch_w4<16>(tx, p, sms, stream);
        case 32: return launch_w4<32>(tx, p, sms, stream);
        case 64: return launch_w4<64>(tx, p, sms, stream);
        case 128: return launch_w4<128>(tx, p, sms, stream);
        default: return launch_w4<256>(tx, p, sms, stream);
    }
}
