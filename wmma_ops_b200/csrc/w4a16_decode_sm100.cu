// W4A16 decode kernel: C[M,N] = X[M,K] @ dequant(qweight, scales) for M <= 16 activation rows.
//
// The reference tree has no INT4 code; this kernel belongs to the W4A16 entry point this library
// defines (include/wmma_ops_b200.h, wmma_ops_w4a16_gemm). With a handful of activation rows the
// product is one pass over the packed weights, so the kernel is organised around the byte stream:
//
//   * Column ownership. In the packed layout all columns of one 64-deep k-block are contiguous
//     (32 bytes per column), so a CTA that owns the columns [n0, n1) reads, for every k-block, one
//     contiguous segment of (n1 - n0) * 32 bytes. Columns are dealt to the CTAs in groups of 16
//     (one m16n8k16 row tile), as evenly as the group count allows; a CTA walks the whole K range
//     of its columns, so no partial sums cross CTA boundaries, there is no workspace, no ticket and
//     no tail. When there are too few column groups for that (narrow outputs), a cluster of 2 or 4
//     CTAs shares a column range, each CTA takes one part of K, and the parts are added through
//     distributed shared memory in rank order.
//   * All loads in flight at once. The 16 warps of a CTA take the k-blocks round-robin. Each warp
//     owns a private ring of shared-memory slots, one segment per slot, filled by one bulk copy
//     (cp.async.bulk) that its lane 0 issues; for K = 4096 the four segments of a warp fit the ring,
//     so every byte the CTA will read is requested in the first microsecond.
//   * Expansion next to the MMA. A warp expands a segment in registers straight into
//     mma.sync.m16n8k16 A fragments (the weights are the 16-row operand, the tokens the 8-column
//     one): a code or'ed into the mantissa of a fp16 constant and one fp16 subtraction give the
//     exact integer code - 8. The fp32 sum of each 64-deep block is then multiplied by the group's
//     fp16 scale. The MMAs of a k-step are issued for several column groups back to back
//     (independent accumulators), so that no warp waits on a chain of dependent MMAs. The legacy
//     tensor pipe (mma.sync) is what bounds the kernel: one m16n8k16 takes 16-24 cycles of an SM
//     sub-partition, so a variant that left half of the zero points to an extra constant-operand
//     MMA chain (fewer ALU instructions, 5e-7 relative error) was slower, not faster.
//   * The 16 warps' tiles are added in warp order in shared memory (deterministic), and the output
//     stage (fp32, fp16 with alpha, or silu(gate) * up) writes the result.
//
// Every mbarrier wait is bounded; a wait that gives up records {code 4, warp, block, detail} in the
// status word and the CTA finishes its control flow (including every cluster barrier) without
// touching the data again.
#include <cuda_runtime.h>

#include "host_common.cuh"
#include "w4a16_common.cuh"

namespace wb {

constexpr int SC_WARPS = 16;
constexpr int SC_THREADS = SC_WARPS * 32;
constexpr int SC_GROUP_COLS = 16;                        // columns per group (one MMA row tile)
constexpr int SC_GROUP_BYTES = SC_GROUP_COLS * 32;       // one group of one k-block
constexpr int SC_SMEM_LIMIT = 227 * 1024;

__device__ __forceinline__ void mma_m16n8k16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                             uint32_t b0, uint32_t b1, const float (&c)[4]) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(c[0]), "f"(c[1]), "f"(c[2]), "f"(c[3]));
}

__device__ __forceinline__ uint32_t h2_bits(__half2 v) { return *reinterpret_cast<const uint32_t*>(&v); }
__device__ __forceinline__ __half2 bits_h2(uint32_t v) { return *reinterpret_cast<const __half2*>(&v); }

// Two of the four fp16 pairs (k, k+1) of one packed word, as the exact integers code - 8: `w` is the
// word (pairs 0 and 1) or the word shifted right by 8 (pairs 2 and 3). Nibble p of a word holds k
// offset {0,2,4,6,1,3,5,7}[p], so the two codes of a pair sit 16 bits apart. A code in bits 0..3 of a
// half-word or'ed with 0x6400 is the fp16 number 1024 + code, a code in bits 4..7 or'ed with 0x5400
// is 64 + code; one fp16 subtraction each (1032, 72) leaves code - 8.
__device__ __forceinline__ void sc_expand_pairs(uint32_t w, uint32_t& lo, uint32_t& hi) {
    const uint32_t t0 = (w & 0x000F000Fu) | 0x64006400u;
    const uint32_t t1 = (w & 0x00F000F0u) | 0x54005400u;
    lo = h2_bits(__hsub2(bits_h2(t0), bits_h2(0x64086408u)));
    hi = h2_bits(__hsub2(bits_h2(t1), bits_h2(0x54805480u)));
}

#ifdef SC_TIMELINE
__device__ long long sc_timeline[148 * 16 * 8];
#define SC_MARK(i) do { if (lane == 0) sc_timeline[(blockIdx.x * 16 + warp) * 8 + (i)] = clock64(); } while (0)
#else
#define SC_MARK(i) do { } while (0)
#endif

__device__ __forceinline__ void sc_report(int* status, int warp, int detail) {
    if (status != nullptr && atomicCAS(status, 0, 4) == 0) {
        status[1] = warp;
        status[2] = static_cast<int>(blockIdx.x);
        status[3] = detail;
    }
}

// How the launch is cut up; computed on the host (w4_decode_plan) and passed by value.
struct ScPlan {
    int uq, ur;        // cluster c owns the units [c*uq + min(c, ur), ...): uq = units / clusters, ur = units % clusters
    int kq, kr;        // CTA rank r of a cluster owns the k-blocks [r*kq + min(r, kr), ...)
    int gpu;           // groups per unit: 1, or 2 in the fused gate/up mode
    int ksplit;        // CTAs per cluster
    int upc;           // units per chunk (a chunk is what one pass over K accumulates in registers)
    int depth;         // ring slots per warp
    int slot_bytes;    // bytes of one slot
    int pitch;         // floats per token row of the reduction tiles
    int red_off;       // byte offsets into dynamic shared memory
    int out_off;
    int bar_off;
    int smem_bytes;
    int overlap;       // 1: launched as a programmatic dependent launch
};

// Column (first of 16) of group j of a chunk that starts at unit v0.
template <bool GU>
__device__ __forceinline__ int sc_group_col(int v0, int j) {
    if (!GU) return (v0 + j) * SC_GROUP_COLS;
    // fused gate/up: unit v is the 16 gate columns 128*(v/4) + 16*(v%4) and the up columns 64 further on
    const int v = v0 + (j >> 1);
    return (v >> 2) * 128 + (v & 3) * 16 + (j & 1) * 64;
}

struct ScXFrag {
    uint4 a[2];  // X[token][64 kb + 16 t .. + 15]: eight (k, k+1) words, two per MMA
};

template <int ROWS>
__device__ __forceinline__ void sc_load_x(const W4Params& p, const __half* xrow, int kb, int g, ScXFrag (&x)[ROWS]) {
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
    for (int o = 0; o < ROWS; ++o) {
        x[o].a[0] = x[o].a[1] = zero;
        if (g + 8 * o < p.M) {
            const uint4* src = reinterpret_cast<const uint4*>(xrow + static_cast<size_t>(8 * o) * p.K + kb * W4_BK);
            x[o].a[0] = __ldg(src);
            x[o].a[1] = __ldg(src + 1);
        }
    }
}

// The fp16 scales of k-block kb for this lane's columns g and g + 8 of every group of the chunk that
// starts at unit v0 (low / high half of one register per group; zero past the chunk or past N).
template <int NCG, bool GU>
__device__ __forceinline__ void sc_load_scales(const W4Params& p, int v0, int ncg, int kb, int g, uint32_t (&sc)[NCG]) {
    const int grp = p.group_shift >= 0 ? (kb >> p.group_shift) : (kb / p.group_kb);
    const unsigned short* srow = reinterpret_cast<const unsigned short*>(p.scales) + static_cast<size_t>(grp) * p.N;
#pragma unroll
    for (int j = 0; j < NCG; ++j) {
        const int c = sc_group_col<GU>(v0, j) + g;
        const uint32_t lo = (j < ncg && c < p.N) ? __ldg(srow + c) : 0u;
        const uint32_t hi = (j < ncg && c + 8 < p.N) ? __ldg(srow + c + 8) : 0u;
        sc[j] = lo | (hi << 16);
    }
}

__device__ __forceinline__ void sc_store_out(const W4Params& p, int tok, int col, float v) {
    if (col >= p.N || !WB_DEBUG_INDEX(tok >= 0 && tok < p.M && col >= 0, p.status, 105, col)) return;
    if (p.out_mode == WMMA_OPS_W4_OUT_F32) p.C[static_cast<size_t>(tok) * p.N + col] = v;
    else p.C16[static_cast<size_t>(tok) * p.N + col] = __float2half_rn(p.alpha * v);
}

// ROWS: 8-token groups in use (1: M <= 8, 2: M <= 16). NCG: column groups a chunk may hold, worked
// on JB at a time. GU: fused gate/up output (a unit is a gate group and the up group 64 columns
// further on).
template <int ROWS, int NCG, int JB, bool GU>
__global__ void __launch_bounds__(SC_THREADS, 1) w4a16_decode_kernel(const W4Params p, const ScPlan pl) {
    static_assert(NCG % JB == 0, "column groups are worked on in whole blocks");
    // With two token groups the registers do not hold a second set of activation fragments: the
    // activations of a k-block are then loaded at the top of its own iteration (ahead of the wait for
    // the weights) instead of one iteration earlier.
    constexpr bool XPRE = ROWS == 1;
    extern __shared__ __align__(128) uint8_t sc_smem[];
    const uint32_t smem_base = smem_u32(sc_smem);
    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    const int g = lane >> 2;
    const int t = lane & 3;
    // let the next kernel of the stream start its prologue as SMs free up (it waits for this one to
    // complete before it reads anything this one writes)
    asm volatile("griddepcontrol.launch_dependents;");
    SC_MARK(0);
#ifdef SC_TIMELINE
    if (lane == 0) sc_timeline[(blockIdx.x * 16 + warp) * 8 + 7] = static_cast<long long>(globaltimer_ns());
#endif

    const int rank = pl.ksplit > 1 ? static_cast<int>(cluster_ctarank()) : 0;
    const int cluster = pl.ksplit > 1 ? static_cast<int>(blockIdx.x) / pl.ksplit : static_cast<int>(blockIdx.x);
    const int u0 = cluster * pl.uq + (cluster < pl.ur ? cluster : pl.ur);
    const int u1 = u0 + pl.uq + (cluster < pl.ur ? 1 : 0);
    const int k0 = rank * pl.kq + (rank < pl.kr ? rank : pl.kr);
    const int k1 = k0 + pl.kq + (rank < pl.kr ? 1 : 0);
    const int nkb = k1 - k0 > warp ? (k1 - k0 - warp + SC_WARPS - 1) / SC_WARPS : 0;  // this warp's k-blocks per chunk
    const size_t row_words = static_cast<size_t>(p.n_tiles) * (W4_RAW_BYTES / 4);     // words per k-block row

    float* red = reinterpret_cast<float*>(sc_smem + pl.red_off);      // [warp][token][pitch]
    float* cta_out = reinterpret_cast<float*>(sc_smem + pl.out_off);  // [token][pitch]
    const uint32_t ring = smem_base + static_cast<uint32_t>(warp * pl.depth * pl.slot_bytes);
    const uint8_t* ring_ptr = sc_smem + warp * pl.depth * pl.slot_bytes;
    const uint32_t bars = smem_base + static_cast<uint32_t>(pl.bar_off) + static_cast<uint32_t>(warp * pl.depth) * 8u;

    if (lane == 0) {
        for (int s = 0; s < pl.depth; ++s) mbar_init(bars + 8u * s, 1);
        fence_barrier_init();
        fence_proxy_async_smem();
    }
    __syncwarp();
    SC_MARK(1);

    // The next item to request: chunk rq_v0 (its first unit), k-block index rq_i of this warp.
    int rq_v0 = u0, rq_i = 0, rq_slot = 0;
    // Requests the next item into slot rq_slot and moves on. Lane 0 only; false when nothing is left.
    auto request = [&]() -> bool {
        if (nkb == 0 || rq_v0 >= u1) return false;
        const int kb = k0 + warp + SC_WARPS * rq_i;
        const int nun = (u1 - rq_v0 < pl.upc ? u1 - rq_v0 : pl.upc);
        const int ncg = nun * pl.gpu;
        const uint32_t bar = bars + 8u * rq_slot;
        const uint32_t dst = ring + static_cast<uint32_t>(rq_slot * pl.slot_bytes);
        const uint32_t* row = p.qweight + static_cast<size_t>(kb) * row_words;
        mbar_arrive_expect_tx(bar, static_cast<uint32_t>(ncg * SC_GROUP_BYTES));
        if (!GU) {
            bulk_load_1d(dst, row + static_cast<size_t>(rq_v0) * (SC_GROUP_BYTES / 4), static_cast<uint32_t>(ncg * SC_GROUP_BYTES), bar);
        } else {
            for (int j = 0; j < ncg; ++j)
                bulk_load_1d(dst + static_cast<uint32_t>(j * SC_GROUP_BYTES), row + static_cast<size_t>(sc_group_col<GU>(rq_v0, j)) * 8,
                             SC_GROUP_BYTES, bar);
        }
        if (++rq_i == nkb) {
            rq_i = 0;
            rq_v0 += pl.upc;
        }
        if (++rq_slot == pl.depth) rq_slot = 0;
        return true;
    };
    // The first k-block's activations and scales are requested before the weight segments: once
    // ~150 KB of bulk copies per SM are queued in the memory system, a small load issued behind them
    // waits until they have drained (measured: 3.3 us instead of 0.6 us to the first usable block).
    // With overlapped decode launches (programmatic dependent launch; the caller promises that the
    // packed weights are not produced by the kernels just before this one) it is the other way
    // round: the CTA may be here while the previous kernel is still finishing, so it requests its
    // weights first and touches activations, scales and output only after griddepcontrol.wait.
    const __half* xrow = p.X + static_cast<size_t>(g) * p.K + 16 * t;
    ScXFrag x_first[ROWS];
    uint32_t sc_first[NCG];
    const int ncg_first = (u1 - u0 < pl.upc ? u1 - u0 : pl.upc) * pl.gpu;
    if (!pl.overlap) {
        asm volatile("griddepcontrol.wait;" ::: "memory");
        if (nkb > 0) {
            if (XPRE) sc_load_x<ROWS>(p, xrow, k0 + warp, g, x_first);
            sc_load_scales<NCG, GU>(p, u0, ncg_first, k0 + warp, g, sc_first);
        }
    }
    if (lane == 0) {
        for (int s = 0; s < pl.depth; ++s)
            if (!request()) break;
    }
    SC_MARK(2);
    if (pl.overlap) {
        asm volatile("griddepcontrol.wait;" ::: "memory");
        if (nkb > 0) {
            if (XPRE) sc_load_x<ROWS>(p, xrow, k0 + warp, g, x_first);
            sc_load_scales<NCG, GU>(p, u0, ncg_first, k0 + warp, g, sc_first);
        }
    }

    bool ok = true;
    int slot = 0;
    uint32_t phase = 0;

    for (int v0 = u0; v0 < u1; v0 += pl.upc) {
        const int nun = (u1 - v0 < pl.upc ? u1 - v0 : pl.upc);
        const int ncg = nun * pl.gpu;
        const int col0 = sc_group_col<GU>(v0, 0);  // without GU the chunk's columns are contiguous from here

        float acc[NCG][ROWS][4];
#pragma unroll
        for (int j = 0; j < NCG; ++j)
#pragma unroll
            for (int o = 0; o < ROWS; ++o) acc[j][o][0] = acc[j][o][1] = acc[j][o][2] = acc[j][o][3] = 0.f;

        // activations and scales of the chunk's first k-block; the scales of columns g and g + 8 of
        // group j share one register (low / high half)
        ScXFrag x_next[ROWS];
        uint32_t sc_next[NCG];
        auto load_scales = [&](int kb) { sc_load_scales<NCG, GU>(p, v0, ncg, kb, g, sc_next); };
        if (nkb > 0) {
            if (v0 == u0) {
                if (XPRE) {
#pragma unroll
                    for (int o = 0; o < ROWS; ++o) x_next[o] = x_first[o];
                }
#pragma unroll
                for (int j = 0; j < NCG; ++j) sc_next[j] = sc_first[j];
            } else {
                if (XPRE) sc_load_x<ROWS>(p, xrow, k0 + warp, g, x_next);
                load_scales(k0 + warp);
            }
        }

#pragma unroll 1
        for (int i = 0; i < nkb; ++i) {
            ScXFrag x[ROWS];
            uint32_t sc[NCG];
            if (XPRE) {
#pragma unroll
                for (int o = 0; o < ROWS; ++o) x[o] = x_next[o];
            } else {
                sc_load_x<ROWS>(p, xrow, k0 + warp + SC_WARPS * i, g, x);
            }
#pragma unroll
            for (int j = 0; j < NCG; ++j) sc[j] = sc_next[j];
            if (i + 1 < nkb) {
                const int kbn = k0 + warp + SC_WARPS * (i + 1);
                if (XPRE) sc_load_x<ROWS>(p, xrow, kbn, g, x_next);
                load_scales(kbn);
            }
#ifdef SC_TIMELINE
            const long long tw0 = clock64();
#endif
            if (ok && !mbar_wait(bars + 8u * slot, phase)) {
                sc_report(p.status, warp, i);
                ok = false;
            }
            ok = __all_sync(0xffffffffu, ok);
            if (i == 0 && v0 == u0) SC_MARK(3);
#ifdef SC_TIMELINE
            if (lane == 0 && i > 0) sc_timeline[(blockIdx.x * 16 + warp) * 8 + 6] += clock64() - tw0;
            if (lane == 0 && i == 0) sc_timeline[(blockIdx.x * 16 + warp) * 8 + 6] = 0;
#endif
#ifdef SC_NOCOMPUTE
            if (false) {
#else
            if (ok) {
#endif
                const float zero4[4] = {0.f, 0.f, 0.f, 0.f};
                const uint2* sl = reinterpret_cast<const uint2*>(ring_ptr + slot * pl.slot_bytes);
#pragma unroll
                for (int jb = 0; jb < NCG; jb += JB) {
                    if (jb < ncg) {
                        // Weights are the MMA's A operand (rows = columns g and g + 8 of a group), the
                        // activations its B operand (columns = tokens): the expanded pairs land in the
                        // A registers as computed and the B registers are the words of X as loaded.
                        // All JB groups of the block are worked on whether or not the chunk has them (no
                        // branch between the MMAs; a group past the chunk's last reads stale shared
                        // memory and its sums are never stored).
                        uint2 wa[JB], wb[JB];
#pragma unroll
                        for (int jj = 0; jj < JB; ++jj) {
                            wa[jj] = sl[(16 * (jb + jj) + g) * 4 + t];      // words 2t, 2t+1: k 16t .. 16t+15
                            wb[jj] = sl[(16 * (jb + jj) + 8 + g) * 4 + t];
                        }
                        float d[JB][ROWS][4];
#pragma unroll
                        for (int ks = 0; ks < 4; ++ks) {
#pragma unroll
                            for (int jj = 0; jj < JB; ++jj) {
                                const uint32_t ua = (ks & 2) ? wa[jj].y : wa[jj].x;
                                const uint32_t ub = (ks & 2) ? wb[jj].y : wb[jj].x;
                                uint32_t a0, a1, a2, a3;
                                sc_expand_pairs((ks & 1) ? (ua >> 8) : ua, a0, a2);
                                sc_expand_pairs((ks & 1) ? (ub >> 8) : ub, a1, a3);
#pragma unroll
                                for (int o = 0; o < ROWS; ++o) {
                                    const uint4 xv = x[o].a[ks >> 1];
                                    const uint32_t b0 = (ks & 1) ? xv.z : xv.x;
                                    const uint32_t b1 = (ks & 1) ? xv.w : xv.y;
                                    if (ks == 0) mma_m16n8k16(d[jj][o], a0, a1, a2, a3, b0, b1, zero4);
                                    else mma_m16n8k16(d[jj][o], a0, a1, a2, a3, b0, b1, d[jj][o]);
                                }
                            }
                        }
#pragma unroll
                        for (int jj = 0; jj < JB; ++jj) {
                            const __half2 sc2 = bits_h2(sc[jb + jj]);
                            const float f0 = __low2float(sc2), f1 = __high2float(sc2);
#pragma unroll
                            for (int o = 0; o < ROWS; ++o) {
                                acc[jb + jj][o][0] = fmaf(d[jj][o][0], f0, acc[jb + jj][o][0]);
                                acc[jb + jj][o][1] = fmaf(d[jj][o][1], f0, acc[jb + jj][o][1]);
                                acc[jb + jj][o][2] = fmaf(d[jj][o][2], f1, acc[jb + jj][o][2]);
                                acc[jb + jj][o][3] = fmaf(d[jj][o][3], f1, acc[jb + jj][o][3]);
                            }
                        }
                    }
                }
            }
            // every lane's reads of the slot have returned: their values were used by the MMAs above
            __syncwarp();
            if (lane == 0 && ok) request();
            if (++slot == pl.depth) {
                slot = 0;
                phase ^= 1u;
            }
        }
        if (v0 == u0) SC_MARK(4);

        // ---- this warp's tile of the chunk: [token][column], tokens below M only
        float* mine = red + static_cast<size_t>(warp) * p.M * pl.pitch;
#pragma unroll
        for (int j = 0; j < NCG; ++j) {
            if (j < ncg) {
#pragma unroll
                for (int o = 0; o < ROWS; ++o) {
                    const int tok = 8 * o + 2 * t;
                    float* dst = mine + tok * pl.pitch + 16 * j + g;
                    if (tok < p.M) {
                        dst[0] = acc[j][o][0];
                        dst[8] = acc[j][o][2];
                    }
                    if (tok + 1 < p.M) {
                        dst[pl.pitch] = acc[j][o][1];
                        dst[pl.pitch + 8] = acc[j][o][3];
                    }
                }
            }
        }
        __syncthreads();

        // ---- add the 16 warps' tiles in warp order
        const int ncols = ncg * SC_GROUP_COLS;
        const bool direct = pl.ksplit == 1 && !GU;  // sums go straight to the output stage
        for (int e = tid; e < p.M * ncols; e += SC_THREADS) {
            const int tok = e / ncols;
            const int c = e - tok * ncols;
            const float* src = red + tok * pl.pitch + c;
            float v = 0.f;
#pragma unroll
            for (int w = 0; w < SC_WARPS; ++w) v += src[static_cast<size_t>(w) * p.M * pl.pitch];
            if (direct) sc_store_out(p, tok, col0 + c, v);
            else cta_out[tok * pl.pitch + c] = v;
        }
        if (!direct) {
            if (pl.ksplit > 1) cluster_sync();
            else __syncthreads();
            if (rank == 0) {
                // the cluster's parts in rank order; rank 0 is this CTA
                uint32_t peer[4];
                const uint32_t out_addr = smem_base + static_cast<uint32_t>(pl.out_off);
                for (int r = 1; r < pl.ksplit; ++r) peer[r] = mapa(out_addr, static_cast<uint32_t>(r));
                auto total = [&](int tok, int c) {
                    float v = cta_out[tok * pl.pitch + c];
                    for (int r = 1; r < pl.ksplit; ++r) {
                        float q;
                        asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(q) : "r"(peer[r] + static_cast<uint32_t>(tok * pl.pitch + c) * 4u) : "memory");
                        v += q;
                    }
                    return v;
                };
                if (!GU) {
                    for (int e = tid; e < p.M * ncols; e += SC_THREADS) {
                        const int tok = e / ncols;
                        const int c = e - tok * ncols;
                        sc_store_out(p, tok, col0 + c, total(tok, c));
                    }
                } else {
                    // fused gate/up: groups 2u and 2u+1 of the chunk are the gate and up columns of the
                    // same 16 outputs
                    const int nout = nun * SC_GROUP_COLS;
                    const int ldo = p.N / 2;
                    for (int e = tid; e < p.M * nout; e += SC_THREADS) {
                        const int tok = e / nout;
                        const int r = e - tok * nout;
                        const int u = r >> 4, c = r & 15;
                        const float gate = total(tok, 32 * u + c);
                        const float up = total(tok, 32 * u + 16 + c);
                        const int v = v0 + u;
                        const int fcol = (v >> 2) * 64 + (v & 3) * 16 + c;
                        const float act = p.alpha * (gate / (1.f + __expf(-gate))) * up;
                        if (fcol < ldo && WB_DEBUG_INDEX(tok < p.M, p.status, 106, fcol))
                            p.C16[static_cast<size_t>(tok) * ldo + fcol] = __float2half_rn(act);
                    }
                }
            }
        }
        if (v0 == u0) SC_MARK(5);
        // the tiles and the CTA's sums may be overwritten by the next chunk (and read by rank 0 until here)
        if (pl.ksplit > 1) cluster_sync();
        else if (v0 + pl.upc < u1) __syncthreads();
    }
}

// ---------------------------------------------------------------------------------------------- host
// Kernel variants: up to 8 tokens with chunks of up to 5 or 8 column groups, up to 16 tokens with 6.
static int sc_ncg(int M, int longest_groups) {
    if (M > 8) return 6;
    return longest_groups <= 5 ? 5 : 8;
}

W4DecodePlan w4_decode_plan(int M, int N, int K, int out_mode, int sms) {
    W4DecodePlan d;
    d.kb_total = K / W4_BK;
    d.n_tiles = (N + W4_TILE_N - 1) / W4_TILE_N;
    d.gpu = out_mode == WMMA_OPS_W4_OUT_F16_SILU_MUL ? 2 : 1;
    d.units = d.gpu == 2 ? N / 32 : (N + SC_GROUP_COLS - 1) / SC_GROUP_COLS;
    // K split across a cluster only when it evens out the column shares by more than a tenth and
    // every CTA still has a k-block for each warp
    d.ksplit = 1;
    double best = 0.0;
    for (int s = 1; s <= 4; s *= 2) {
        if (s > 1 && d.kb_total / s < SC_WARPS) break;
        const int clusters = sms / s < d.units ? sms / s : d.units;
        if (clusters < 1) break;
        const int longest = (d.units + clusters - 1) / clusters;
        const double eff = static_cast<double>(d.units) / (static_cast<double>(longest) * clusters) *
                           (static_cast<double>(clusters) * s / sms);
        if (eff > best * 1.1) {
            best = eff;
            d.ksplit = s;
        }
    }
    d.clusters = sms / d.ksplit < d.units ? sms / d.ksplit : d.units;
    const int longest = (d.units + d.clusters - 1) / d.clusters;
    d.ncg = sc_ncg(M, longest * d.gpu);
    const int cap = d.ncg / d.gpu;  // units a chunk can hold
    const int chunks = (longest + cap - 1) / cap;
    d.upc = (longest + chunks - 1) / chunks;  // even chunks
    const int cols = d.upc * d.gpu * SC_GROUP_COLS;
    d.slot_bytes = d.upc * d.gpu * SC_GROUP_BYTES;
    d.pitch = cols + 4;  // 4 or 20 modulo 32: a quad's rows 2t land in different banks
    const int red_bytes = SC_WARPS * M * d.pitch * 4;
    const int out_bytes = M * d.pitch * 4;
    // one group block past the last slot may be read (and ignored) by the kernel: keep it inside the allocation
    const int fixed = red_bytes + out_bytes + SC_WARPS * 16 * 8 + 1024 + 8 * SC_GROUP_BYTES;
    int depth = (SC_SMEM_LIMIT - fixed) / (SC_WARPS * d.slot_bytes);
    const int kb_cta = (d.kb_total + d.ksplit - 1) / d.ksplit;
    const int items = ((kb_cta + SC_WARPS - 1) / SC_WARPS) * chunks;  // per warp
    if (depth > items) depth = items;
    if (depth > 16) depth = 16;
    if (depth < 1) depth = 1;
    d.depth = depth;
    const int ring_bytes = SC_WARPS * depth * d.slot_bytes;
    d.red_off = (ring_bytes + 127) / 128 * 128;
    d.out_off = d.red_off + (red_bytes + 127) / 128 * 128;
    d.bar_off = d.out_off + (out_bytes + 127) / 128 * 128;
    d.smem_bytes = d.bar_off + SC_WARPS * depth * 8;
    if (d.smem_bytes < ring_bytes + 8 * SC_GROUP_BYTES) d.smem_bytes = ring_bytes + 8 * SC_GROUP_BYTES;
    d.grid = d.clusters * d.ksplit;
    return d;
}

// 1: decode launches are programmatic dependent launches (set by wmma_ops_set_w4a16_overlap)
static std::atomic<int> g_w4_overlap{0};

template <int ROWS, int NCG, int JB, bool GU>
static int sc_launch(const W4Params& p, const ScPlan& pl, int grid, cudaStream_t stream) {
    static std::atomic<bool> attr_set[64];  // per device; setting the attribute twice is harmless
    int dev = 0;
    WB_CHECK_CUDA(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64 && !attr_set[dev].load(std::memory_order_acquire)) {
        WB_CHECK_CUDA(cudaFuncSetAttribute(w4a16_decode_kernel<ROWS, NCG, JB, GU>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           SC_SMEM_LIMIT));
        attr_set[dev].store(true, std::memory_order_release);
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(SC_THREADS);
    cfg.dynamicSmemBytes = pl.smem_bytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int n = 0;
    if (pl.ksplit > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = pl.ksplit;
        attr[n].val.clusterDim.y = 1;
        attr[n].val.clusterDim.z = 1;
        ++n;
    }
    if (pl.overlap) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    WB_CHECK_CUDA(cudaLaunchKernelEx(&cfg, w4a16_decode_kernel<ROWS, NCG, JB, GU>, p, pl));
    return WMMA_OPS_OK;
}

int w4_decode_launch(const W4Params& p, const W4DecodePlan& d, cudaStream_t stream) {
    WB_REQUIRE(d.smem_bytes <= SC_SMEM_LIMIT, WMMA_OPS_ERR_INVALID, "w4a16 decode: plan needs %d bytes of shared memory",
               d.smem_bytes);
    ScPlan pl;
    pl.uq = d.units / d.clusters;
    pl.ur = d.units % d.clusters;
    pl.kq = d.kb_total / d.ksplit;
    pl.kr = d.kb_total % d.ksplit;
    pl.gpu = d.gpu;
    pl.ksplit = d.ksplit;
    pl.upc = d.upc;
    pl.depth = d.depth;
    pl.slot_bytes = d.slot_bytes;
    pl.pitch = d.pitch;
    pl.red_off = d.red_off;
    pl.out_off = d.out_off;
    pl.bar_off = d.bar_off;
    pl.smem_bytes = d.smem_bytes;
    pl.overlap = g_w4_overlap.load(std::memory_order_relaxed);
    const bool gu = d.gpu == 2;
    if (d.ncg == 6) return gu ? sc_launch<2, 6, 2, true>(p, pl, d.grid, stream) : sc_launch<2, 6, 2, false>(p, pl, d.grid, stream);
    if (d.ncg == 5) return gu ? sc_launch<1, 5, 5, true>(p, pl, d.grid, stream) : sc_launch<1, 5, 5, false>(p, pl, d.grid, stream);
    return gu ? sc_launch<1, 8, 4, true>(p, pl, d.grid, stream) : sc_launch<1, 8, 4, false>(p, pl, d.grid, stream);
}

}  // namespace wb

extern "C" int wmma_ops_set_w4a16_overlap(int enable) {
    wb::g_w4_overlap.store(enable ? 1 : 0, std::memory_order_relaxed);
    return WMMA_OPS_OK;
}

#ifdef SC_TIMELINE
extern "C" int wmma_ops_debug_timeline(long long* host_out) {
    return cudaMemcpyFromSymbol(host_out, wb::sc_timeline, sizeof(long long) * 148 * 16 * 8) == cudaSuccess ? 0 : 2;
}
#endif

extern "C" int wmma_ops_w4a16_decode_plan(int M, int N, int K, int out_mode, int num_sms, int* plan) {
    using namespace wb;
    WB_REQUIRE(plan != nullptr, WMMA_OPS_ERR_INVALID, "w4a16_decode_plan: null output pointer");
    WB_REQUIRE(M >= 1 && M <= W4_STREAM_MAX_M && N >= 8 && N % 8 == 0 && K >= 64 && K % 64 == 0, WMMA_OPS_ERR_INVALID,
               "w4a16_decode_plan: needs 1 <= M <= %d, N %% 8 == 0, K %% 64 == 0 (got %d, %d, %d)", W4_STREAM_MAX_M, M, N, K);
    WB_REQUIRE(out_mode != WMMA_OPS_W4_OUT_F16_SILU_MUL || N % 128 == 0, WMMA_OPS_ERR_INVALID,
               "w4a16_decode_plan: the fused gate/up output needs N %% 128 == 0 (got N=%d)", N);
    const W4DecodePlan d = w4_decode_plan(M, N, K, out_mode, num_sms > 0 ? num_sms : 148);
    const int v[11] = {d.grid, d.clusters, d.ksplit, d.units, d.gpu, d.upc, d.depth, d.slot_bytes, d.pitch, d.smem_bytes, d.ncg};
    for (int i = 0; i < 11; ++i) plan[i] = v[i];
    return WMMA_OPS_OK;
}
