// Streaming W4A16 kernel for decode: C[M,N] = X[M,K] @ dequant(qweight, scales) with M <= 16.
//
// Takes the place of the reference's fused dequant GEMV/GEMM path for small batches
// (quant_kernels.hpp: the INT4 weights are expanded next to the MMA, never written back to memory).
// With one or a few activation rows the product is a single pass over the packed weights, so the
// kernel is built around the byte stream, not around the tensor core:
//
//   * all 4 KB weight blocks of all column tiles, in tile-major order, are dealt to the CTAs in
//     equal contiguous runs (one CTA per SM), so every SM streams the same number of bytes;
//   * the 16 warps of a CTA are 8 k-lanes x 2 column halves: warp (lane kl, half h) takes the
//     64-column half h (2 KB, contiguous) of every 8th block of the run. Each warp owns a private
//     ring of SD_DEPTH shared-memory slots; its lane 0 refills a slot with one bulk copy as soon as
//     the warp has finished the half block that was in it, so 64 copies per SM are in flight and
//     no thread issues more than one copy per item;
//   * a warp expands its half block straight into mma.sync A fragments in registers (the weights
//     are the 16-row operand, the tokens the 8-column one; the k order inside a fragment is chosen
//     so that one 64-bit shared load per thread feeds four MMAs and no operand is moved),
//     multiplies by the integer-valued fp16 weights code - 8 (exact) with fp32 accumulation and
//     applies the group's fp16 scale to the fp32 sum of the block;
//   * the k-lanes' tiles of a column tile are added in lane order in shared memory, one tile late
//     (double-buffered, so no CTA-wide barrier per tile); if the tile is shared with other CTAs
//     the sum goes to the workspace, and when the CTA has streamed all its blocks it takes a
//     ticket per shared tile: the last CTA to arrive adds the parts in CTA order (deterministic)
//     and writes the output.
//
// Every mbarrier wait is bounded; a wait that gives up records {code 4, warp, block, detail} in the
// status word and the CTA finishes its control flow without touching the data again.
#include <cuda_runtime.h>

#include "host_common.cuh"
#include "w4a16_common.cuh"

namespace wb {

constexpr int SD_KLANES = 8;
constexpr int SD_WARPS = 2 * SD_KLANES;
constexpr int SD_THREADS = SD_WARPS * 32;
constexpr int SD_ITEM_BYTES = W4_RAW_BYTES / 2;  // 64 columns x 64 k
constexpr int SD_RED_PITCH = 64 + 4;         // floats; rows 2t of a quad of lanes land 8 banks apart

// Shared-memory budget. HI (9..16 activation rows) keeps 16-row warp tiles and a shallower ring.
template <bool HI>
struct SdCfg {
    static constexpr int DEPTH = HI ? 2 : 4;                  // ring slots per warp
    static constexpr int ROWS8 = HI ? 2 : 1;                  // 8-row groups of the MMA tile in use
    static constexpr int RING_BYTES = SD_WARPS * DEPTH * SD_ITEM_BYTES;
    static constexpr int TILE_FLOATS = ROWS8 * 8 * SD_RED_PITCH;  // one warp's tile of one unit
    static constexpr int RED_BYTES = 2 * SD_WARPS * TILE_FLOATS * 4;  // two units' tiles
    static constexpr int BAR_BYTES = (SD_WARPS * DEPTH + 4) * 8 + 64;
    static constexpr int SMEM_BYTES = 1024 + RING_BYTES + RED_BYTES + BAR_BYTES;
    static_assert(SMEM_BYTES <= 232448, "streaming decode kernel: shared memory over the per-CTA limit");
};

// The blocks of all column tiles, in tile-major order, are cut into gridDim.x runs: with
// q = blocks / CTAs and r = blocks % CTAs, the first r CTAs take q + 1 blocks and the rest q.
struct SdRun {
    int q, r;    // as above
    int b0, b1;  // this CTA's run
    int t0;      // first column tile the run touches
};

__device__ __forceinline__ int sd_run_start(const SdRun& run, int cta) {
    return cta * run.q + (cta < run.r ? cta : run.r);
}

// CTA whose run holds block x.
__device__ __forceinline__ int sd_owner(const SdRun& run, int x) {
    const int big = run.r * (run.q + 1);  // blocks held by the CTAs with q + 1 blocks
    return x < big ? x / (run.q + 1) : run.r + (x - big) / run.q;
}

__device__ __forceinline__ SdRun sd_make_run(const W4Params& p) {
    SdRun run;
    const int total = p.kb_total * p.n_tiles;  // the launcher checks that this fits
    run.q = total / static_cast<int>(gridDim.x);
    run.r = total % static_cast<int>(gridDim.x);
    run.b0 = sd_run_start(run, static_cast<int>(blockIdx.x));
    run.b1 = sd_run_start(run, static_cast<int>(blockIdx.x) + 1);
    run.t0 = run.b0 / p.kb_total;
    return run;
}

// Part of column tile nt that this CTA's run covers: k-blocks [kb0, kb1), which are blocks
// off, off + 1, ... of the run.
struct SdUnit {
    int nt, kb0, kb1, off;
};

__device__ __forceinline__ bool sd_unit(const W4Params& p, const SdRun& run, int ui, SdUnit& u) {
    const int tile = run.t0 + ui;
    const int lo = tile * p.kb_total;
    const int s = run.b0 > lo ? run.b0 : lo;
    const int e = run.b1 < lo + p.kb_total ? run.b1 : lo + p.kb_total;
    if (s >= e) return false;
    u.nt = tile;
    u.kb0 = s - lo;
    u.kb1 = e - lo;
    u.off = s - run.b0;
    return true;
}

// For a unit that does not cover its whole tile: it is part `sl` of the tile's `nsl` parts.
__device__ __forceinline__ void sd_slices(const W4Params& p, const SdRun& run, const SdUnit& u, int& sl, int& nsl) {
    const int lo = u.nt * p.kb_total;
    const int c_first = sd_owner(run, lo);
    const int c_last = sd_owner(run, lo + p.kb_total - 1);
    sl = static_cast<int>(blockIdx.x) - c_first;
    nsl = c_last - c_first + 1;
}

// A block of the run. The blocks of a run go to the eight k-lanes round-robin (lane kl takes blocks
// kl, kl + 8, ... of the run, across tile boundaries), so the lanes' loads differ by one block at most.
struct SdPos {
    int nt, kb;
};

__device__ __forceinline__ void sd_normalize(SdPos& c, int kbt) {
    while (c.kb >= kbt) {
        c.kb -= kbt;
        ++c.nt;
    }
}

__device__ __forceinline__ void mma_m16n8k16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                             uint32_t b0, uint32_t b1, const float (&c)[4]) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(c[0]), "f"(c[1]), "f"(c[2]), "f"(c[3]));
}

__device__ __forceinline__ uint32_t h2_bits(__half2 v) { return *reinterpret_cast<const uint32_t*>(&v); }
__device__ __forceinline__ __half2 bits_h2(uint32_t v) { return *reinterpret_cast<const __half2*>(&v); }

// The eight codes of one packed word (k offsets 0..7 of one column) as four fp16 pairs (k, k+1)
// of code - 8. Nibble p holds k offset {0,2,4,6,1,3,5,7}[p], so the two codes of pair q sit 16 bits
// apart at bit 4q. 0x6400 | code is 1024 + code; a code left in bits 4..7 makes 1024 + 16 * code,
// and fma(x, 1/16, -72) brings it to code - 8. Both forms are exact.
__device__ __forceinline__ void sd_expand_word(uint32_t w, uint32_t (&b)[4]) {
    const uint32_t w8 = w >> 8;
    const uint32_t t0 = (w & 0x000F000Fu) | 0x64006400u;
    const uint32_t t1 = (w & 0x00F000F0u) | 0x64006400u;
    const uint32_t t2 = (w8 & 0x000F000Fu) | 0x64006400u;
    const uint32_t t3 = (w8 & 0x00F000F0u) | 0x64006400u;
    const __half2 c1032 = bits_h2(0x64086408u);
    const __half2 sixteenth = bits_h2(0x2C002C00u);
    const __half2 m72 = bits_h2(0xD480D480u);
    b[0] = h2_bits(__hsub2(bits_h2(t0), c1032));
    b[1] = h2_bits(__hfma2(bits_h2(t1), sixteenth, m72));
    b[2] = h2_bits(__hsub2(bits_h2(t2), c1032));
    b[3] = h2_bits(__hfma2(bits_h2(t3), sixteenth, m72));
}

__device__ __forceinline__ void sd_report(int* status, int warp, int detail) {
    if (status != nullptr && atomicCAS(status, 0, 4) == 0) {
        status[1] = warp;
        status[2] = static_cast<int>(blockIdx.x);
        status[3] = detail;
    }
}

// Activation fragments of one 64-deep block for this lane: X rows (tokens) g and g + 8,
// k = 16 t .. 16 t + 15. Each 32-bit word is a (k, k+1) pair: two consecutive words are the B
// operand of one MMA.
struct SdXFrag {
    uint4 lo[2];  // token g:     [0] k 16t..16t+7, [1] k 16t+8..16t+15
    uint4 hi[2];  // token g + 8
};

// xrow: this lane's row g of X, advanced to column 16 t; rows at or past M read as zero.
template <bool HI>
__device__ __forceinline__ void sd_load_x(const W4Params& p, const __half* xrow, int kb, int g, SdXFrag& x) {
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    x.lo[0] = x.lo[1] = x.hi[0] = x.hi[1] = zero;
    const uint4* src = reinterpret_cast<const uint4*>(xrow + kb * W4_BK);
    if (g < p.M) {
        x.lo[0] = __ldg(src);
        x.lo[1] = __ldg(src + 1);
    }
    if (HI && g + 8 < p.M) {
        src += p.K;  // 8 rows of K halves = K uint4
        x.hi[0] = __ldg(src);
        x.hi[1] = __ldg(src + 1);
    }
}

// The scales of columns c and c + 32 of the warp's 64-column half for k-block kb, each as the
// low half of a word. c = nt * 128 + half * 64 + lane.
__device__ __forceinline__ void sd_load_scales(const W4Params& p, int c, int kb, uint32_t& s0, uint32_t& s1) {
    const int grp = p.group_shift >= 0 ? (kb >> p.group_shift) : (kb / p.group_kb);
    const unsigned short* src = reinterpret_cast<const unsigned short*>(p.scales) + static_cast<size_t>(grp) * p.N + c;
    s0 = c < p.N ? __ldg(src) : 0u;
    s1 = c + 32 < p.N ? __ldg(src + 32) : 0u;
}

__device__ __forceinline__ void sd_epilogue(const W4Params& p, int nt, int row, int c, float v0, float v1) {
    // v0: column c of the tile, v1: column c + 64
    if (row >= p.M) return;
    const int n0 = nt * W4_TILE_N + c;
    const int n1 = n0 + 64;
    if (p.out_mode == WMMA_OPS_W4_OUT_F32) {
        if (n0 < p.N) p.C[static_cast<size_t>(row) * p.N + n0] = v0;
        if (n1 < p.N) p.C[static_cast<size_t>(row) * p.N + n1] = v1;
    } else if (p.out_mode == WMMA_OPS_W4_OUT_F16) {
        if (n0 < p.N) p.C16[static_cast<size_t>(row) * p.N + n0] = __float2half_rn(p.alpha * v0);
        if (n1 < p.N) p.C16[static_cast<size_t>(row) * p.N + n1] = __float2half_rn(p.alpha * v1);
    } else {
        // columns 0..63 of a tile are gate columns, 64..127 the up columns of the same outputs
        const int f = nt * 64 + c;
        const int ldo = p.N / 2;
        const float act = p.alpha * (v0 / (1.f + __expf(-v0))) * v1;
        if (f < ldo) p.C16[static_cast<size_t>(row) * ldo + f] = __float2half_rn(act);
    }
}

// HI: the product has more than 8 activation rows (rows 8..15 of the MMA tile are in use).
template <bool HI>
__global__ void __launch_bounds__(SD_THREADS, 1) w4a16_stream_kernel(const W4Params p) {
    using Cfg = SdCfg<HI>;
    constexpr int DEPTH = Cfg::DEPTH;
    constexpr int ROWS = Cfg::ROWS8;
    extern __shared__ uint8_t sd_smem_raw[];
    const uint32_t raw_addr = smem_u32(sd_smem_raw);
    const uint32_t base = (raw_addr + 1023u) & ~1023u;
    uint8_t* base_ptr = sd_smem_raw + (base - raw_addr);
    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    const int g = lane >> 2;
    const int t = lane & 3;
    const int half = warp & 1;  // column half of the tile
    const int kl = warp >> 1;   // k-lane
    // let the next kernel of the stream start its own prologue as soon as SMs free up (it waits
    // for this one to complete before it reads anything this one writes)
    asm volatile("griddepcontrol.launch_dependents;");

    const int ring_off = warp * (DEPTH * SD_ITEM_BYTES);
    // red[b][warp]: the warps' tiles of the units with parity b, [token row][column] with pitch SD_RED_PITCH
    float* red = reinterpret_cast<float*>(base_ptr + Cfg::RING_BYTES);
    const uint32_t bars = base + Cfg::RING_BYTES + Cfg::RED_BYTES;
    auto full = [&](int s) { return bars + static_cast<uint32_t>(warp * DEPTH + s) * 8u; };
    auto unit_done = [&](int b) { return bars + static_cast<uint32_t>(SD_WARPS * DEPTH + b) * 8u; };
    auto reduced = [&](int b) { return bars + static_cast<uint32_t>(SD_WARPS * DEPTH + 2 + b) * 8u; };
    const uint32_t flag_slot = bars + static_cast<uint32_t>(SD_WARPS * DEPTH + 4) * 8u;

    const SdRun run = sd_make_run(p);
    const int kbt = p.kb_total;
    const int nb = run.b1 - run.b0;
    const int n_items = nb > kl ? (nb - kl + SD_KLANES - 1) / SD_KLANES : 0;  // this lane's blocks
    SdPos cur;  // the block being consumed
    cur.nt = run.t0;
    cur.kb = run.b0 - run.t0 * kbt + kl;
    sd_normalize(cur, kbt);
    if (lane == 0) {
        for (int s = 0; s < DEPTH; ++s) mbar_init(full(s), 1);
        if (warp == 0) {
            for (int b = 0; b < 2; ++b) {
                mbar_init(unit_done(b), SD_WARPS);
                mbar_init(reduced(b), SD_WARPS);
            }
        }
        fence_barrier_init();
        fence_proxy_async_smem();
    }
    __syncthreads();

    auto request = [&](const SdPos& c, int s) {
        // this warp's column half of k-block c.kb of column tile c.nt into slot s of its ring
        const uint32_t* src = p.qweight + (static_cast<size_t>(c.kb) * p.n_tiles + c.nt) * (W4_RAW_BYTES / 4) +
                              half * (SD_ITEM_BYTES / 4);
        mbar_arrive_expect_tx(full(s), SD_ITEM_BYTES);
        bulk_load_1d(base + ring_off + s * SD_ITEM_BYTES, src, SD_ITEM_BYTES, full(s));
    };

    SdPos pf = cur;  // the block DEPTH items ahead
    int issued = 0;
    for (int s = 0; s < DEPTH; ++s) {
        if (issued < n_items) {
            if (lane == 0) request(pf, s);
            ++issued;
            pf.kb += SD_KLANES;
            sd_normalize(pf, kbt);
        }
    }
    // Everything above touches only the packed weights. When the caller has switched on
    // overlapped decode launches (programmatic dependent launch; it then promises that the packed
    // weights are not produced by the kernels just before this one), the CTA got here while the
    // previous kernel was still finishing and its own weight blocks are already on their way. The
    // activations, the scales, the workspace and the output are only touched once that kernel is
    // complete. In an ordinary launch the wait returns at once.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const __half* xrow = p.X + static_cast<size_t>(g) * p.K + 16 * t;
    SdXFrag x_next;
    uint32_t sc0_next = 0u, sc1_next = 0u;
    if (n_items > 0) {
        sd_load_x<HI>(p, xrow, cur.kb, g, x_next);
        sd_load_scales(p, cur.nt * W4_TILE_N + half * 64 + lane, cur.kb, sc0_next, sc1_next);
    }

    int pend_nt[2] = {0, 0}, pend_nsl[2] = {1, 1};  // shared tiles whose hand-over is still due
    int n_pending = 0;
    int it = 0;      // items this warp has consumed
    bool ok = true;  // false once a wait gave up
    const float zero4[4] = {0.f, 0.f, 0.f, 0.f};
    const int c_out = tid & 63;  // output column (and column + 64) this thread sums
    const int r_out = tid >> 6;  // output rows r_out, r_out + 8

    // Adds the warps' tiles of unit v (parity v & 1) in lane order and writes the tile's output, or
    // parks it in the workspace when other CTAs hold parts of the tile. Runs one unit late: by the
    // time a warp gets here every warp has long flushed unit v, so nobody waits for the lane that
    // happened to have one block more in that unit.
    auto reduce_unit = [&](int v) {
        SdUnit u;
        sd_unit(p, run, v, u);
        const int b = v & 1;
        if (ok && !mbar_wait(unit_done(b), static_cast<uint32_t>(v >> 1) & 1u)) {
            sd_report(p.status, warp, 10000 + v);
            ok = false;
        }
        const float* tiles = red + b * (SD_WARPS * Cfg::TILE_FLOATS);
        float vsum[ROWS][2];
#pragma unroll
        for (int i = 0; i < ROWS; ++i) {
            const float* src = tiles + (r_out + 8 * i) * SD_RED_PITCH + c_out;
            float a0 = 0.f, a1 = 0.f;
#pragma unroll
            for (int w = 0; w < SD_KLANES; ++w) {
                a0 += src[(2 * w) * Cfg::TILE_FLOATS];
                a1 += src[(2 * w + 1) * Cfg::TILE_FLOATS];
            }
            vsum[i][0] = a0;
            vsum[i][1] = a1;
        }
        // this warp is done with the tiles of parity b
        __syncwarp();
        if (lane == 0) mbar_arrive(reduced(b));
        if (u.kb0 == 0 && u.kb1 == p.kb_total) {
#pragma unroll
            for (int i = 0; i < ROWS; ++i) sd_epilogue(p, u.nt, r_out + 8 * i, c_out, vsum[i][0], vsum[i][1]);
        } else {
            // a tile shared with other CTAs: park the part in the workspace; the hand-over (fence,
            // ticket, sum by the last CTA) waits until this CTA has streamed all its blocks, so the
            // round trip to the L2 is paid once per CTA and not inside the stream
            int sl, nsl;
            sd_slices(p, run, u, sl, nsl);
            float* part = p.partials + (static_cast<size_t>(u.nt) * p.max_slices + sl) * (16 * W4_TILE_N);
#pragma unroll
            for (int i = 0; i < ROWS; ++i) {
                const int row = r_out + 8 * i;
                if (row < p.M) {
                    part[row * W4_TILE_N + c_out] = vsum[i][0];
                    part[row * W4_TILE_N + c_out + 64] = vsum[i][1];
                }
            }
            if (n_pending < 2) {
                pend_nt[n_pending] = u.nt;
                pend_nsl[n_pending] = nsl;
            }
            ++n_pending;
        }
    };

    int n_units = 0;
    for (int ui = 0;; ++ui) {
        SdUnit u;
        if (!sd_unit(p, run, ui, u)) break;
        n_units = ui + 1;
        // acc[o][jj]: tokens 8o .. 8o+7 (this lane: 2t, 2t+1) x columns 16jj+g ([0],[1]) and 16jj+8+g ([2],[3])
        float acc[ROWS][4][4];
#pragma unroll
        for (int o = 0; o < ROWS; ++o)
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) acc[o][jj][0] = acc[o][jj][1] = acc[o][jj][2] = acc[o][jj][3] = 0.f;

#pragma unroll 1
        while (it < n_items && cur.nt == u.nt) {
            const SdXFrag x = x_next;
            const uint32_t sc0 = sc0_next, sc1 = sc1_next;
            // fetch the next item's activations and scales now: they come from the L2 or HBM
            SdPos nxt = cur;
            nxt.kb += SD_KLANES;
            sd_normalize(nxt, kbt);
            if (it + 1 < n_items) {
                sd_load_x<HI>(p, xrow, nxt.kb, g, x_next);
                sd_load_scales(p, nxt.nt * W4_TILE_N + half * 64 + lane, nxt.kb, sc0_next, sc1_next);
            }
            const int s = it % DEPTH;
            const uint32_t ph = static_cast<uint32_t>(it / DEPTH) & 1u;
            if (ok && !mbar_wait(full(s), ph)) {
                sd_report(p.status, warp, it);
                ok = false;
            }
            ok = __all_sync(0xffffffffu, ok);
            if (ok) {
                const uint2* slot = reinterpret_cast<const uint2*>(base_ptr + ring_off + s * SD_ITEM_BYTES);
#pragma unroll
                for (int jj = 0; jj < 4; ++jj) {
                    // The weights are the MMA's A operand (rows = columns 16jj+g and 16jj+8+g of the
                    // half), the activations its B operand (columns = tokens): the expanded pairs
                    // land in the A registers as they are computed and the B registers are the
                    // words of X as loaded, so no operand is moved.
                    const uint2 wa = slot[(16 * jj + g) * 4 + t];      // words 2t, 2t+1: k 16t .. 16t+15
                    const uint2 wb = slot[(16 * jj + 8 + g) * 4 + t];
                    uint32_t a0[4], a1[4], b0[4], b1[4];
                    sd_expand_word(wa.x, a0);
                    sd_expand_word(wa.y, a1);
                    sd_expand_word(wb.x, b0);
                    sd_expand_word(wb.y, b1);
                    const float f0 = __half2float(__ushort_as_half(static_cast<unsigned short>(
                        __shfl_sync(0xffffffffu, (jj & 2) ? sc1 : sc0, 16 * (jj & 1) + g))));
                    const float f1 = __half2float(__ushort_as_half(static_cast<unsigned short>(
                        __shfl_sync(0xffffffffu, (jj & 2) ? sc1 : sc0, 16 * (jj & 1) + 8 + g))));
#pragma unroll
                    for (int o = 0; o < ROWS; ++o) {
                        const uint4 x0 = o ? x.hi[0] : x.lo[0];
                        const uint4 x1 = o ? x.hi[1] : x.lo[1];
                        float d[4];
                        mma_m16n8k16(d, a0[0], b0[0], a0[1], b0[1], x0.x, x0.y, zero4);
                        mma_m16n8k16(d, a0[2], b0[2], a0[3], b0[3], x0.z, x0.w, d);
                        mma_m16n8k16(d, a1[0], b1[0], a1[1], b1[1], x1.x, x1.y, d);
                        mma_m16n8k16(d, a1[2], b1[2], a1[3], b1[3], x1.z, x1.w, d);
                        acc[o][jj][0] = fmaf(d[0], f0, acc[o][jj][0]);
                        acc[o][jj][1] = fmaf(d[1], f0, acc[o][jj][1]);
                        acc[o][jj][2] = fmaf(d[2], f1, acc[o][jj][2]);
                        acc[o][jj][3] = fmaf(d[3], f1, acc[o][jj][3]);
                    }
                }
            }
            // every lane's reads of the slot have returned: their values were used by the MMAs above
            __syncwarp();
            if (issued < n_items) {
                if (ok && lane == 0) request(pf, s);
                ++issued;
                pf.kb += SD_KLANES;
                sd_normalize(pf, kbt);
            }
            ++it;
            cur = nxt;
        }

        // ---- flush this warp's tile of unit ui; the tiles of unit ui - 2 must have been added up
        const int b = ui & 1;
        if (ui >= 2 && ok && !mbar_wait(reduced(b), static_cast<uint32_t>((ui >> 1) - 1) & 1u)) {
            sd_report(p.status, warp, 20000 + ui);
            ok = false;
        }
        float* mine = red + (b * SD_WARPS + warp) * Cfg::TILE_FLOATS;
#pragma unroll
        for (int o = 0; o < ROWS; ++o)
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) {
                float* dst = mine + (8 * o + 2 * t) * SD_RED_PITCH + 16 * jj + g;
                dst[0] = acc[o][jj][0];
                dst[SD_RED_PITCH] = acc[o][jj][1];
                dst[8] = acc[o][jj][2];
                dst[SD_RED_PITCH + 8] = acc[o][jj][3];
            }
        __syncwarp();
        if (lane == 0) mbar_arrive(unit_done(b));
        if (ui >= 1) reduce_unit(ui - 1);
    }
    if (n_units >= 1) reduce_unit(n_units - 1);

    // ---- hand-over of the shared tiles (only the first and the last tile of a run can be shared)
    if (n_pending > 2) {
        if (tid == 0) sd_report(p.status, -1, n_pending);
        n_pending = 2;
    }
    __syncthreads();  // all threads' partial sums are stored
    if (n_pending == 0) return;
    // one release for the CTA: the barrier above ordered all threads' stores before thread 0's
    // gpu-scope fence, which is cumulative over them
    if (tid == 0) {
        __threadfence();
        // both tickets are in flight together
        const int old0 = atomicAdd(p.counters + pend_nt[0], 1);
        const int old1 = n_pending > 1 ? atomicAdd(p.counters + pend_nt[1], 1) : -1;
        for (int k = 0; k < n_pending; ++k) {
            const uint32_t last = ((k == 0 ? old0 : old1) == pend_nsl[k] - 1) ? 1u : 0u;
            if (last) p.counters[pend_nt[k]] = 0;  // ready for the next call
            asm volatile("st.shared.u32 [%0], %1;" ::"r"(flag_slot + 4 * k), "r"(last) : "memory");
        }
    }
    __syncthreads();
    for (int k = 0; k < n_pending; ++k) {
        uint32_t last;
        asm volatile("ld.shared.u32 %0, [%1];" : "=r"(last) : "r"(flag_slot + 4 * k) : "memory");
        if (!last) continue;
        __threadfence();
        // the last CTA to arrive adds the parts in CTA order
        const float* all = p.partials + static_cast<size_t>(pend_nt[k]) * p.max_slices * (16 * W4_TILE_N);
        float sum[ROWS][2];
#pragma unroll
        for (int i = 0; i < ROWS; ++i) sum[i][0] = sum[i][1] = 0.f;
        // four parts at a time, so that their loads (L2 round trips) are in flight together; the
        // additions stay in CTA order
        for (int s0 = 0; s0 < pend_nsl[k]; s0 += 4) {
            float q[4][ROWS][2];
#pragma unroll
            for (int d2 = 0; d2 < 4; ++d2)
#pragma unroll
                for (int i = 0; i < ROWS; ++i) {
                    const int row = r_out + 8 * i;
                    const bool on = s0 + d2 < pend_nsl[k] && row < p.M;
                    const float* src = all + static_cast<size_t>(s0 + d2) * (16 * W4_TILE_N) + row * W4_TILE_N + c_out;
                    q[d2][i][0] = on ? __ldcg(src) : 0.f;
                    q[d2][i][1] = on ? __ldcg(src + 64) : 0.f;
                }
#pragma unroll
            for (int d2 = 0; d2 < 4; ++d2)
#pragma unroll
                for (int i = 0; i < ROWS; ++i) {
                    sum[i][0] += q[d2][i][0];
                    sum[i][1] += q[d2][i][1];
                }
        }
#pragma unroll
        for (int i = 0; i < ROWS; ++i) sd_epilogue(p, pend_nt[k], r_out + 8 * i, c_out, sum[i][0], sum[i][1]);
    }
}

W4StreamPlan w4_stream_plan(int N, int K, int sms) {
    W4StreamPlan pl;
    pl.n_tiles = (N + W4_TILE_N - 1) / W4_TILE_N;
    pl.kb_total = K / W4_BK;
    const long long blocks = static_cast<long long>(pl.n_tiles) * pl.kb_total;
    pl.grid = blocks < sms ? static_cast<int>(blocks) : sms;
    const int per = static_cast<int>(blocks / pl.grid);  // shortest run, >= 1
    pl.max_slices = (pl.kb_total + per - 1) / per + 1;
    return pl;
}

// 1: decode launches are programmatic dependent launches (set by wmma_ops_set_w4a16_overlap)
static int g_w4_overlap = 0;

template <bool HI>
static int sd_launch(const W4Params& p, int grid, cudaStream_t stream) {
    static bool attr_set[64] = {};
    int dev = 0;
    WB_CHECK_CUDA(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        WB_CHECK_CUDA(cudaFuncSetAttribute(w4a16_stream_kernel<HI>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           SdCfg<HI>::SMEM_BYTES));
        attr_set[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(SD_THREADS);
    cfg.dynamicSmemBytes = SdCfg<HI>::SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_w4_overlap ? 1 : 0;
    WB_CHECK_CUDA(cudaLaunchKernelEx(&cfg, w4a16_stream_kernel<HI>, p));
    return WMMA_OPS_OK;
}

int w4_stream_launch(const W4Params& p, int grid, cudaStream_t stream) {
    return p.M > 8 ? sd_launch<true>(p, grid, stream) : sd_launch<false>(p, grid, stream);
}

}  // namespace wb

extern "C" int wmma_ops_set_w4a16_overlap(int enable) {
    wb::g_w4_overlap = enable ? 1 : 0;
    return WMMA_OPS_OK;
}
