// Definitions of the W4A16 kernel (w4a16_sm100.cu): launch parameters, the walk over work units
// and the exact dequant step.
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>
#include <cstdint>

#include "ptx.cuh"

namespace wb {

constexpr int W4_TILE_N = 128;     // weight columns per CTA tile (MMA M)
constexpr int W4_BK = 64;          // k per pipeline step
constexpr int W4_RAW_BYTES = 4096; // one packed block
constexpr int W4_SLOT_BYTES = W4_RAW_BYTES + W4_TILE_N * 2;  // + the block's 128 fp16 scales
constexpr int W4_WT_BYTES = W4_TILE_N * W4_BK * 2;
constexpr int W4_THREADS = 512;
constexpr int W4_DQ_WARPS = 8;     // each dequant warp expands a whole 4 KB block; 8 blocks in flight

struct W4Params {
    const __half* X;   // activations [M, K] (read directly by the decode kernel)
    const uint32_t* qweight;
    const __half* scales;
    float* C;          // fp32 output (out_mode 0)
    __half* C16;       // fp16 output (out_mode 1: [M,N]; out_mode 2: [M,N/2])
    int out_mode;      // 0: C = acc; 1: C16 = half(alpha*acc); 2: C16 = half(alpha*silu(gate)*up)
    float alpha;
    float in_scale;    // out_mode 2 only: gate and up are multiplied by this before silu(gate) * up (a scale of the input, folded in)
    float* partials;   // [tiles][split][BT][128]
    int* counters;     // [tiles]
    int M, N, K;
    int n_tiles, t_tiles, split;
    int balanced;      // 1: k-blocks are dealt to the CTAs in equal runs of 8-block chunks (decode)
    int max_slices;    // slices a tile can have (= split in the classic plan): stride of partials
    int kb_total;
    int group_kb;      // k-blocks per scale group (group_size / 64)
    int group_shift;   // log2(group_kb) when it is a power of two, else -1
    int* status;
    int* block_done;   // optional: block_done[tt] is incremented when a column tile of token block tt has been written
    int tt_major;      // 1: units walk all column tiles of a token block before the next block (set with block_done)
};

__device__ __forceinline__ void w4_report(int* status, int role, int detail) {
    if (status != nullptr && atomicCAS(status, 0, 2) == 0) {
        status[1] = role;
        status[2] = static_cast<int>(blockIdx.x);
        status[3] = detail;
    }
}

// One work unit of a CTA: the k-blocks [kb0, kb1) of the tile (nt, tt); it is slice `sl` of `nsl`
// slices of that tile.
struct W4Unit {
    int nt, tt, sl, nsl, kb0, kb1;
};

constexpr int W4_CHUNK = 8;  // k-blocks per chunk in the balanced plan

// CTA that owns chunk x when total chunks TC are dealt to G CTAs in runs [c*TC/G, (c+1)*TC/G).
__device__ __forceinline__ int w4_chunk_owner(long long x, long long TC, long long G) {
    long long c = x * G / TC;
    while ((c + 1) * TC / G <= x) ++c;
    while (c * TC / G > x) --c;
    return static_cast<int>(c);
}

// The ui-th work unit of this CTA (ui = 0, 1, ...). Returns false past the last one.
// Classic plan: units (tile, K-slice) are dealt round-robin, unit = blockIdx.x + ui * gridDim.x.
// Balanced plan (decode, one token tile): all k-blocks of all column tiles, in tile-major order and
// cut into chunks of 8, are dealt to the CTAs in equal contiguous runs, so every SM streams the
// same number of bytes; a run covers parts of one to three tiles and each part is a unit.
__device__ __forceinline__ bool w4_unit(const W4Params& p, int ui, W4Unit& u) {
    if (!p.balanced) {
        const int unit = static_cast<int>(blockIdx.x) + ui * static_cast<int>(gridDim.x);
        if (unit >= p.n_tiles * p.t_tiles * p.split) return false;
        u.sl = unit % p.split;
        u.nsl = p.split;
        const int t = unit / p.split;
        if (p.tt_major) {
            // token block by token block: a block's output is complete after its n_tiles tiles, early in
            // the launch, so that a consumer (the sum over the ranks) can follow the kernel block by block
            u.nt = t % p.n_tiles;
            u.tt = t / p.n_tiles;
        } else {
            u.tt = t % p.t_tiles;
            u.nt = t / p.t_tiles;
        }
        u.kb0 = static_cast<int>(static_cast<long long>(u.sl) * p.kb_total / p.split);
        u.kb1 = static_cast<int>(static_cast<long long>(u.sl + 1) * p.kb_total / p.split);
        return true;
    }
    const long long cpt = p.kb_total / W4_CHUNK;  // chunks per tile
    const long long TC = cpt * p.n_tiles;
    const long long G = gridDim.x;
    const long long c0 = static_cast<long long>(blockIdx.x) * TC / G;
    const long long c1 = static_cast<long long>(blockIdx.x + 1) * TC / G;
    const long long tile = c0 / cpt + ui;
    const long long start = c0 > tile * cpt ? c0 : tile * cpt;
    const long long end = c1 < (tile + 1) * cpt ? c1 : (tile + 1) * cpt;
    if (start >= end) return false;
    u.nt = static_cast<int>(tile);
    u.tt = 0;
    u.kb0 = static_cast<int>(start - tile * cpt) * W4_CHUNK;
    u.kb1 = static_cast<int>(end - tile * cpt) * W4_CHUNK;
    const int c_first = w4_chunk_owner(tile * cpt, TC, G);
    const int c_last = w4_chunk_owner((tile + 1) * cpt - 1, TC, G);
    u.sl = static_cast<int>(blockIdx.x) - c_first;
    u.nsl = c_last - c_first + 1;
    return true;
}

// Position of a worker warp in the CTA's sequence of k-block iterations.
struct W4Cursor {
    int ui, nt, tt, kb, kb0, kb1;
    bool valid;
};

__device__ __forceinline__ void w4_cursor_start(const W4Params& p, W4Cursor& c) {
    W4Unit u;
    c.ui = 0;
    c.valid = w4_unit(p, 0, u);
    c.nt = u.nt; c.tt = u.tt; c.kb = c.kb0 = u.kb0; c.kb1 = u.kb1;
}

// Moves the cursor `steps` iterations forward, crossing into later work units as needed.
__device__ __forceinline__ void w4_cursor_advance(const W4Params& p, W4Cursor& c, int steps) {
    if (!c.valid) return;
    c.kb += steps;
    while (c.kb >= c.kb1) {
        const int over = c.kb - c.kb1;
        W4Unit u;
        if (!w4_unit(p, ++c.ui, u)) {
            c.valid = false;
            return;
        }
        c.nt = u.nt; c.tt = u.tt; c.kb0 = u.kb0; c.kb1 = u.kb1;
        c.kb = c.kb0 + over;
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

// The same for two codes that sit in bits 4..7 and 20..23 of t (masked with 0x00F000F0, not shifted):
// 0x5400 | (code << 4) is the fp16 number 64 + code (the mantissa step at 64 is 1/16), so subtracting 72
// gives code - 8 exactly. Saves the shift that would bring the nibble down to bit 0.
__device__ __forceinline__ uint32_t dq_pair_hi(uint32_t t, __half2 scale2) {
    const uint32_t h = t | 0x54005400u;
    const __half2 v = __hsub2(*reinterpret_cast<const __half2*>(&h), __half2half2(__ushort_as_half(0x5480)));
    const __half2 r = __hmul2(v, scale2);
    return *reinterpret_cast<const uint32_t*>(&r);
}

// ---------------------------------------------------------------- decode kernel
// (w4a16_decode_sm100.cu) for products with at most W4_STREAM_MAX_M activation rows.
constexpr int W4_STREAM_MAX_M = 16;

// Bytes at the start of a workspace that hold the per-tile arrival counters of the tcgen05 kernel's
// partial-sum plans. The area has a fixed size for every product with up to 16384 tiles, so that a
// caller who reuses one zero-initialised buffer for products of different shapes never gets one
// call's partial sums into the counters of the next (the kernels leave the counters at zero).
inline size_t w4_counter_bytes(int tiles) {
    const size_t need = (static_cast<size_t>(tiles) * 4 + 255) / 256 * 256;
    return need < 65536 ? 65536 : need;
}

// How the decode kernel cuts a product up (host arithmetic, no GPU needed). Units are groups of 16
// columns (pairs of a gate and an up group in the fused gate/up mode); cluster c of `clusters` owns
// the units [c*units/clusters, (c+1)*units/clusters) and walks them in chunks of `upc`; the `ksplit`
// CTAs of a cluster each take one part of K. The decode kernel needs no workspace.
struct W4DecodePlan {
    int kb_total, n_tiles, gpu, units, ksplit, clusters, upc, ncg, slot_bytes, pitch, depth;
    int seg_kb, xs_off, x_pitch, ss_off, ss_pitch, alias_red, red_off, out_off, bar_off, smem_bytes, grid;
};

W4DecodePlan w4_decode_plan(int M, int N, int K, int group_size, int out_mode, int sms);
int w4_decode_launch(const W4Params& p, const W4DecodePlan& d, cudaStream_t stream);

}  // namespace wb
