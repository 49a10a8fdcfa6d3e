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
//   * Weights in flight from the first microsecond. The 16 warps of a CTA take the k-blocks
//     round-robin. Each warp owns a private ring of shared-memory slots, one weight segment per slot,
//     filled by one bulk copy (cp.async.bulk) that its lane 0 issues; for K = 4096 the four segments
//     of a warp fit the ring, so every weight byte the CTA will read is requested at once.
//   * Activations and scales staged once. The activations (one bulk copy per row) and the fp16
//     scales (plain 8-byte loads issued before any bulk copy) of a K segment are staged in shared
//     memory ahead of the weight requests; the segment is all of K when that fits beside the ring.
//   * Expansion next to the MMA. A warp expands a segment in registers straight into
//     mma.sync.m16n8k16 A fragments (the weights are the 16-row operand, the tokens the 8-column
//     one): a code or'ed into the mantissa of a fp16 constant and one fp16 subtraction give the
//     exact integer code - 8. The fp32 sum of each 64-deep block is then multiplied by the group's
//     fp16 scale. The MMAs of a k-step are issued for several column groups back to back
//     (independent accumulators), so that no warp waits on a chain of dependent MMAs. The legacy
//     tensor pipe (mma.sync) is what bounds the k-loop: measured with per-warp cycle counters it
//     costs about 23 cycles of an SM sub-partition per m16n8k16, with 8 or with 16 activation rows
//     and whatever the integer work beside it (a variant that left half of the zero points to an
//     extra constant-operand MMA chain, 5e-7 relative error, was slower, not faster).
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
    int slot_bytes;    // bytes of one slot (the packed weights of a chunk's columns for one k-block)
    int seg_kb;        // k-blocks per segment: the activations and scales of one segment are staged at a time
    int xs_off;        // staged activations [M][x_pitch bytes]
    int x_pitch;       // seg_kb * 128 + 16 bytes (the 16 spread the rows of a quad over the banks)
    int ss_off;        // staged fp16 scales [groups of the segment][ss_pitch bytes]
    int ss_pitch;
    int pitch;         // floats per token row of the reduction tiles
    int red_off;       // byte offsets into dynamic shared memory
    int out_off;
    int bar_off;
    int smem_bytes;
    int alias_red;     // 1: the reduction tiles lie over the ring (every cluster has one chunk)
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
    const uint32_t stage_bar = smem_base + static_cast<uint32_t>(pl.bar_off) + static_cast<uint32_t>(SC_WARPS * pl.depth) * 8u;

    if (lane == 0) {
        for (int s = 0; s < pl.depth; ++s) mbar_init(bars + 8u * s, 1);
        if (warp == 0) mbar_init(stage_bar, 1);
        fence_barrier_init();
        fence_proxy_async_smem();
    }
    __syncthreads();

    // The next weight segment to request: chunk rq_v0 (its first unit), k-block index rq_i of this warp.
    int rq_v0 = u0, rq_i = 0, rq_slot = 0;
    auto request = [&]() {  // lane 0; does nothing when no item is left
        if (nkb == 0 || rq_v0 >= u1) return;
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
    };

    // Activations and scales are staged in shared memory one K segment at a time, ahead of the weight
    // requests. Activations: one bulk copy per row (the segment's part of it), issued by warp 0.
    // Scales: plain 8-byte loads by all threads, issued before any bulk copy of the CTA and stored to
    // shared memory once the weight requests are out. What was tried before: plain loads inside the
    // k-loop (issued behind ~150 KB of queued bulk copies per SM, a small load took 3.5 us to come
    // back), one bulk copy per activation row per k-block, and one bulk copy per scale group (the SM
    // accepts bulk copies at about one per 20 cycles per issuing lane, so 30 small copies from one
    // warp cost more than all the weight requests).
    uint32_t stage_phase = 0;
    bool ok = true;  // false once a bounded wait gave up
    constexpr int SC_STAGE_LOADS = 4;  // 8-byte scale loads per thread and round
    // Stages the scales of chunk (v0, nun) and k-blocks [ks0, ks1), and with with_x the activations.
    // All threads. `before_x` and `after_x` run after the scale loads are issued, around the
    // activation copies, and before the loaded values are needed.
    auto stage = [&](int v0, int nun, int ks0, int ks1, bool with_x, auto&& before_x, auto&& after_x) {
        const int ncg = nun * pl.gpu;
        const int c0 = sc_group_col<GU>(v0, 0);
        int span = sc_group_col<GU>(v0, ncg - 1) + SC_GROUP_COLS - c0;  // columns from the chunk's first to its last
        if (c0 + span > p.N) span = p.N - c0;
        const int g0 = p.group_shift >= 0 ? (ks0 >> p.group_shift) : (ks0 / p.group_kb);
        const int g1 = p.group_shift >= 0 ? ((ks1 - 1) >> p.group_shift) : ((ks1 - 1) / p.group_kb);
        const int ng = g1 - g0 + 1;
        const int per_row = span >> 2;          // 8-byte words per scale row (span is a multiple of 8... of 4 scales)
        const int words = ng * per_row;
        bool first = true;
        for (int base = 0; base < words; base += SC_THREADS * SC_STAGE_LOADS) {
            uint32_t lo[SC_STAGE_LOADS], hi[SC_STAGE_LOADS];
            int dst[SC_STAGE_LOADS];
#pragma unroll
            for (int q = 0; q < SC_STAGE_LOADS; ++q) {
                const int e = base + q * SC_THREADS + tid;
                dst[q] = -1;
                if (e < words) {
                    const int gi = e / per_row;
                    const int c4 = e - gi * per_row;
                    const __half* src = p.scales + static_cast<size_t>(g0 + gi) * p.N + c0 + 4 * c4;
                    asm volatile("ld.global.nc.v2.u32 {%0, %1}, [%2];" : "=r"(lo[q]), "=r"(hi[q]) : "l"(src));
                    dst[q] = pl.ss_off + gi * pl.ss_pitch + c4 * 8;
                }
            }
            if (first) {
                before_x();
                if (with_x && warp == 0) {
                    const uint32_t xbytes = static_cast<uint32_t>((ks1 - ks0) * 128);
                    if (lane == 0) mbar_arrive_expect_tx(stage_bar, static_cast<uint32_t>(p.M) * xbytes);
                    __syncwarp();
                    if (lane < p.M)
                        bulk_load_1d(smem_base + static_cast<uint32_t>(pl.xs_off + lane * pl.x_pitch),
                                     p.X + static_cast<size_t>(lane) * p.K + ks0 * W4_BK, xbytes, stage_bar);
                }
                after_x();
                first = false;
            }
#pragma unroll
            for (int q = 0; q < SC_STAGE_LOADS; ++q)
                if (dst[q] >= 0) *reinterpret_cast<uint2*>(sc_smem + dst[q]) = make_uint2(lo[q], hi[q]);
        }
        __syncthreads();  // the scales are in place for every warp
        if (with_x) {
            if (ok && !mbar_wait(stage_bar, stage_phase)) {
                sc_report(p.status, warp, 30000);
                ok = false;
            }
            stage_phase ^= 1u;
        }
    };
    const int seg_first_end = k0 + pl.seg_kb < k1 ? k0 + pl.seg_kb : k1;
    const bool one_segment = seg_first_end == k1;
    const int nun_first = (u1 - u0 < pl.upc ? u1 - u0 : pl.upc);
    auto first_requests = [&]() {
        if (lane == 0)
            for (int s = 0; s < pl.depth; ++s) request();
    };
    // With overlapped decode launches (programmatic dependent launch; the caller promises that the
    // packed weights and their scales are not produced by the kernels just before this one) the CTA
    // may be here while the previous kernel of the stream is still finishing: it loads its scales and
    // requests its weights first, and touches activations and output only after griddepcontrol.wait.
    // In an ordinary launch the wait returns at once, and the activation copies go out ahead of the
    // weights.
    auto nothing = [] {};
    if (pl.overlap) {
        stage(u0, nun_first, k0, seg_first_end, true,
              [&] {
                  first_requests();
                  asm volatile("griddepcontrol.wait;" ::: "memory");
              },
              nothing);
    } else {
        asm volatile("griddepcontrol.wait;" ::: "memory");
        stage(u0, nun_first, k0, seg_first_end, true, nothing, first_requests);
    }

    // this lane's activation words within a staged row: token g (and g + 8), k 16t .. 16t+15 of a
    // k-block; tokens past M read the last row (their MMA columns are never stored)
    int x_lane_off[ROWS];
#pragma unroll
    for (int o = 0; o < ROWS; ++o) {
        const int row = g + 8 * o < p.M ? g + 8 * o : p.M - 1;
        x_lane_off[o] = pl.xs_off + row * pl.x_pitch + t * 32;
    }
    int slot = 0;
    uint32_t phase = 0;

    for (int v0 = u0; v0 < u1; v0 += pl.upc) {
        const int nun = (u1 - v0 < pl.upc ? u1 - v0 : pl.upc);
        const int ncg = nun * pl.gpu;
        const int col0 = sc_group_col<GU>(v0, 0);  // without GU the chunk's columns are contiguous from here
        int sc_lane_off[NCG];                      // this lane's scale of group j within a staged scale row
#pragma unroll
        for (int j = 0; j < NCG; ++j) sc_lane_off[j] = (sc_group_col<GU>(v0, j) - col0 + g) * 2;

        float acc[NCG][ROWS][4];
#pragma unroll
        for (int j = 0; j < NCG; ++j)
#pragma unroll
            for (int o = 0; o < ROWS; ++o) acc[j][o][0] = acc[j][o][1] = acc[j][o][2] = acc[j][o][3] = 0.f;

        int i = 0;  // index of this warp's next k-block within the chunk
        for (int ks0 = k0; ks0 < k1; ks0 += pl.seg_kb) {
            const int ks1 = ks0 + pl.seg_kb < k1 ? ks0 + pl.seg_kb : k1;
            if (!(v0 == u0 && ks0 == k0)) {
                // a new segment or chunk: every warp is done with what is staged, then it is replaced
                // (the activations only if they change)
                __syncthreads();
                stage(v0, nun, ks0, ks1, !one_segment, nothing, nothing);
            }
            const int g_first = p.group_shift >= 0 ? (ks0 >> p.group_shift) : (ks0 / p.group_kb);

#pragma unroll 1
            for (; k0 + warp + SC_WARPS * i < ks1; ++i) {
                const int kb = k0 + warp + SC_WARPS * i;
                if (ok && !mbar_wait(bars + 8u * slot, phase)) {
                    sc_report(p.status, warp, i);
                    ok = false;
                }
                ok = __all_sync(0xffffffffu, ok);
                if (ok) {
                    const uint2* sl = reinterpret_cast<const uint2*>(ring_ptr + slot * pl.slot_bytes);
                    const int grel = (p.group_shift >= 0 ? (kb >> p.group_shift) : (kb / p.group_kb)) - g_first;
                    const uint8_t* ssc = sc_smem + pl.ss_off + grel * pl.ss_pitch;
                    uint4 xa[ROWS][2];
#pragma unroll
                    for (int o = 0; o < ROWS; ++o) {
                        const uint4* xs = reinterpret_cast<const uint4*>(sc_smem + x_lane_off[o] + (kb - ks0) * 128);
                        xa[o][0] = xs[0];
                        xa[o][1] = xs[1];
                    }
                    const float zero4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                    for (int jb = 0; jb < NCG; jb += JB) {
                        if (jb < ncg) {
                            // Weights are the MMA's A operand (rows = columns g and g + 8 of a group),
                            // the activations its B operand (columns = tokens): the expanded pairs land
                            // in the A registers as computed and the B registers are the words of X as
                            // loaded. All JB groups of the block are worked on whether or not the chunk
                            // has them (no branch between the MMAs; a group past the chunk's last reads
                            // stale shared memory and its sums are never stored).
                            uint2 wa[JB], wb[JB];
#pragma unroll
                            for (int jj = 0; jj < JB; ++jj) {
                                wa[jj] = sl[(16 * (jb + jj) + g) * 4 + t];      // words 2t, 2t+1: k 16t .. 16t+15
                                wb[jj] = sl[(16 * (jb + jj) + 8 + g) * 4 + t];
                            }
                            float d[JB][ROWS][4];
                            // The expansion of k-step ks + 1 is written between the MMAs of k-step ks.
                            uint32_t ea[2][JB][4];
                            auto expand = [&](int jj, int ks, uint32_t (&e)[4]) {
                                const uint32_t ua = (ks & 2) ? wa[jj].y : wa[jj].x;
                                const uint32_t ub = (ks & 2) ? wb[jj].y : wb[jj].x;
                                sc_expand_pairs((ks & 1) ? (ua >> 8) : ua, e[0], e[2]);
                                sc_expand_pairs((ks & 1) ? (ub >> 8) : ub, e[1], e[3]);
                            };
#pragma unroll
                            for (int jj = 0; jj < JB; ++jj) expand(jj, 0, ea[0][jj]);
#pragma unroll
                            for (int ks = 0; ks < 4; ++ks) {
#pragma unroll
                                for (int jj = 0; jj < JB; ++jj) {
#pragma unroll
                                    for (int o = 0; o < ROWS; ++o) {
                                        const uint4 xv = xa[o][ks >> 1];
                                        const uint32_t b0 = (ks & 1) ? xv.z : xv.x;
                                        const uint32_t b1 = (ks & 1) ? xv.w : xv.y;
                                        const uint32_t(&e)[4] = ea[ks & 1][jj];
                                        if (ks == 0) mma_m16n8k16(d[jj][o], e[0], e[1], e[2], e[3], b0, b1, zero4);
                                        else mma_m16n8k16(d[jj][o], e[0], e[1], e[2], e[3], b0, b1, d[jj][o]);
                                    }
                                    if (ks < 3) expand(jj, ks + 1, ea[(ks + 1) & 1][jj]);
                                }
                            }
#pragma unroll
                            for (int jj = 0; jj < JB; ++jj) {
                                // the scales of columns g and g + 8 of the group (stale past N: those
                                // columns are never stored)
                                const float f0 = __half2float(*reinterpret_cast<const __half*>(ssc + sc_lane_off[jb + jj]));
                                const float f1 = __half2float(*reinterpret_cast<const __half*>(ssc + sc_lane_off[jb + jj] + 16));
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
                if (ok && lane == 0) request();
                if (++slot == pl.depth) {
                    slot = 0;
                    phase ^= 1u;
                }
            }
        }

        // ---- this warp's tile of the chunk: [token][column], tokens below M only
        if (pl.alias_red) __syncthreads();  // the tiles lie over the ring: every warp has read its last slot
        float* mine = red + static_cast<size_t>(warp) * p.M * pl.pitch;
#pragma unroll
        for (int j = 0; j < NCG; ++j) {
            if (j < ncg) {
                const int cj = sc_group_col<GU>(v0, j) - col0;  // the group's place in the chunk's span of columns
#pragma unroll
                for (int o = 0; o < ROWS; ++o) {
                    const int tok = 8 * o + 2 * t;
                    float* dst = mine + tok * pl.pitch + (GU ? 16 * j : cj) + g;
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
                        const float gate = p.in_scale * total(tok, 32 * u + c);
                        const float up = p.in_scale * total(tok, 32 * u + 16 + c);
                        const int v = v0 + u;
                        const int fcol = (v >> 2) * 64 + (v & 3) * 16 + c;
                        const float act = p.alpha * (gate / (1.f + __expf(-gate))) * up;
                        if (fcol < ldo && WB_DEBUG_INDEX(tok < p.M, p.status, 106, fcol))
                            p.C16[static_cast<size_t>(tok) * ldo + fcol] = __float2half_rn(act);
                    }
                }
            }
        }
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

W4DecodePlan w4_decode_plan(int M, int N, int K, int group_size, int out_mode, int sms) {
    W4DecodePlan d;
    const int group_kb = group_size / W4_BK;
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
    // the chunk's span of columns, first to last: its own columns, or with the fused gate/up output
    // the tiles its units touch
    const int span = d.gpu == 1 ? cols : ((d.upc + 2) / 4 + 1) * W4_TILE_N;
    d.ss_pitch = (span * 2 + 15) / 16 * 16;
    const int red_bytes = SC_WARPS * M * d.pitch * 4;
    const int out_bytes = (M * d.pitch * 4 + 127) / 128 * 128;
    const int bar_bytes = (SC_WARPS * 16 + 1) * 8 + 120;
    // one group block past the last slot may be read (and ignored) by the kernel: keep it inside the allocation
    const int slack = 8 * SC_GROUP_BYTES;
    const int kb_cta = (d.kb_total + d.ksplit - 1) / d.ksplit;
    const int items = ((kb_cta + SC_WARPS - 1) / SC_WARPS) * chunks;  // per warp
    // Segments are whole rounds of the 16 warps and whole scale groups. The longest segment that
    // leaves the ring two slots per warp (or all items, if fewer) is taken; with one chunk per
    // cluster nothing is requested into the ring once its last slot has been read, so the reduction
    // tiles may lie over it, which is taken when it buys a deeper ring.
    int unit_kb = SC_WARPS;
    while (unit_kb % group_kb != 0) unit_kb += SC_WARPS;
    const int want = items < 2 ? items : 2;
    int seg = (kb_cta + unit_kb - 1) / unit_kb * unit_kb;
    int depth = 0;
    for (;;) {
        const int x_bytes = (M * (seg * 128 + 16) + 127) / 128 * 128;
        const int ss_bytes = (((seg + group_kb - 1) / group_kb + 1) * d.ss_pitch + 127) / 128 * 128;
        auto depth_for = [&](bool alias) {
            const int fixed = x_bytes + ss_bytes + out_bytes + bar_bytes + slack + 256 + (alias ? 0 : red_bytes);
            const int room = SC_SMEM_LIMIT - fixed;
            int dd = room > 0 ? room / (SC_WARPS * d.slot_bytes) : 0;
            if (alias && SC_WARPS * dd * d.slot_bytes + slack < red_bytes) dd = 0;  // the tiles must fit under the ring
            return dd < items ? dd : items;
        };
        depth = depth_for(false);
        d.alias_red = 0;
        if (chunks == 1 && depth < items) {
            const int da = depth_for(true);
            if (da > depth) {
                depth = da;
                d.alias_red = 1;
            }
        }
        if (depth >= want || seg <= unit_kb) break;
        seg = (seg / 2 + unit_kb - 1) / unit_kb * unit_kb;  // halve, in whole units
    }
    if (depth > 16) depth = 16;
    if (depth < 1) depth = 1;
    d.depth = depth;
    d.seg_kb = seg;
    d.x_pitch = seg * 128 + 16;
    const int x_bytes = (M * d.x_pitch + 127) / 128 * 128;
    const int ss_bytes = (((seg + group_kb - 1) / group_kb + 1) * d.ss_pitch + 127) / 128 * 128;
    const int ring_bytes = SC_WARPS * depth * d.slot_bytes;
    const int ring_span = (ring_bytes + slack + 127) / 128 * 128;
    if (d.alias_red) {
        d.red_off = 0;
        d.xs_off = ring_span > red_bytes ? ring_span : (red_bytes + 127) / 128 * 128;
    } else {
        d.red_off = ring_span;
        d.xs_off = d.red_off + (red_bytes + 127) / 128 * 128;
    }
    d.ss_off = d.xs_off + x_bytes;
    d.out_off = d.ss_off + ss_bytes;
    d.bar_off = d.out_off + out_bytes;
    d.smem_bytes = d.bar_off + bar_bytes;
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
    pl.seg_kb = d.seg_kb;
    pl.xs_off = d.xs_off;
    pl.x_pitch = d.x_pitch;
    pl.ss_off = d.ss_off;
    pl.ss_pitch = d.ss_pitch;
    pl.alias_red = d.alias_red;
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


extern "C" int wmma_ops_w4a16_decode_plan(int M, int N, int K, int group_size, int out_mode, int num_sms, int* plan) {
    using namespace wb;
    WB_REQUIRE(plan != nullptr, WMMA_OPS_ERR_INVALID, "w4a16_decode_plan: null output pointer");
    WB_REQUIRE(M >= 1 && M <= W4_STREAM_MAX_M && N >= 8 && N % 8 == 0 && K >= 64 && K % 64 == 0, WMMA_OPS_ERR_INVALID,
               "w4a16_decode_plan: needs 1 <= M <= %d, N %% 8 == 0, K %% 64 == 0 (got %d, %d, %d)", W4_STREAM_MAX_M, M, N, K);
    WB_REQUIRE(out_mode != WMMA_OPS_W4_OUT_F16_SILU_MUL || N % 128 == 0, WMMA_OPS_ERR_INVALID,
               "w4a16_decode_plan: the fused gate/up output needs N %% 128 == 0 (got N=%d)", N);
    WB_REQUIRE(group_size >= 64 && group_size % 64 == 0 && K % group_size == 0, WMMA_OPS_ERR_INVALID,
               "w4a16_decode_plan: group_size must be a multiple of 64 that divides K (got %d)", group_size);
    const W4DecodePlan d = w4_decode_plan(M, N, K, group_size, out_mode, num_sms > 0 ? num_sms : 148);
    const int v[14] = {d.grid, d.clusters, d.ksplit, d.units, d.gpu, d.upc, d.depth, d.slot_bytes, d.pitch, d.smem_bytes, d.ncg,
                       d.alias_red, d.seg_kb, d.x_pitch};
    for (int i = 0; i < 14; ++i) plan[i] = v[i];
    return WMMA_OPS_OK;
}
