// Flash-attention forward for decode shapes: a few query rows (Sq <= 16) against a long key/value
// sequence, O = softmax(scale * Q K^T [+ causal mask]) V per (batch, head).
//
// Belongs to the flash_attention entry point whose signature the reference documents
// (README.md:221-251; its implementation is not in the reference tree). The prefill kernel
// (fmha_fwd_sm100.cu) gives every CTA 128 query rows; with one to sixteen queries that wastes 7/8 or
// more of every tile and, worse, runs one CTA per head. Here the work is a single pass over K and V
// (the path is bound by their bytes, 2 * Skv * D * 2 per head), so:
//   * the key range of a head is cut into `splits` parts, one CTA each, and inside a CTA the four
//     warps take 16-key tiles round-robin; every warp keeps its own running maximum, sum and output
//     rows, so warps never wait for each other inside the stream;
//   * K and V tiles travel global -> shared with 16-byte cp.async into a two-stage ring per warp
//     (rows past the end are zero-filled), swizzled so that ldmatrix reads without bank conflicts;
//     K is read as the col operand of S = Q K^T, V through ldmatrix.trans as the col operand of
//     O += P V, and the probabilities go from the S accumulators straight into the A operand of
//     P V (no shared-memory round trip);
//   * mma.sync.m16n8k16 (the 16 query rows are the M side): the tensor work is a small fraction of
//     the time the bytes take, a tcgen05 pipeline would add set-up without moving the bound;
//   * the four warps' partial results are merged in shared memory; with more than one split the
//     CTA's (maximum, sum, unnormalised rows) go to a workspace and a second small kernel merges the
//     splits in split order (deterministic).
// No waits on other CTAs, no spin loops.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "host_common.cuh"
#include "ptx.cuh"

namespace wb {

constexpr int FD_WARPS = 4;
constexpr int FD_THREADS = FD_WARPS * 32;
constexpr int FD_TILE = 16;   // keys per tile
constexpr int FD_STAGES = 2;
constexpr int FD_MAX_SQ = 16;

struct FdParams {
    const __half* Q;
    const __half* K;
    const __half* V;
    __half* O;
    float* ws;        // [B*H][splits][Sq][D + 2]: unnormalised rows, then maximum (log2 units) and sum
    int B, H, Sq, Skv, D;
    int splits, keys_per_split;  // keys_per_split is a multiple of FD_TILE
    float scale_log2;
    int causal;
    int* status;
};

__device__ __forceinline__ void fd_mma(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                       uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void fd_ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void fd_ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}

// 16 bytes global -> shared; src_bytes = 0 writes zeros (rows past the end of the sequence)
__device__ __forceinline__ void fd_cp_async16(uint32_t dst, const void* src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void fd_cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void fd_cp_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ uint32_t fd_pack(float a, float b) {
    const __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&h);
}

// D: head dimension (64 or 128). A tile row is D halves; its 16-byte chunks are XOR-swizzled with the
// row index so that the eight rows an ldmatrix touches lie in different banks.
template <int D>
__global__ void __launch_bounds__(FD_THREADS) fmha_decode_kernel(const FdParams p) {
    constexpr int ROW_BYTES = D * 2;
    constexpr int CHUNKS = ROW_BYTES / 16;             // 16-byte chunks per row
    constexpr int TILE_BYTES = FD_TILE * ROW_BYTES;    // one K or V tile
    constexpr int DT = D / 16;                         // 16-wide tiles of the head dimension
    constexpr int MERGE_PITCH = D + 4;                 // floats per row of a warp's partial result
    extern __shared__ __align__(128) uint8_t fd_smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int bh = blockIdx.y, split = blockIdx.x;
    const int key_lo = split * p.keys_per_split;
    const int key_hi = key_lo + p.keys_per_split < p.Skv ? key_lo + p.keys_per_split : p.Skv;
    const int n_tiles = (key_hi - key_lo + FD_TILE - 1) / FD_TILE;   // of this CTA; warp w takes tiles w, w+4, ...
    const __half* Kb = p.K + static_cast<size_t>(bh) * p.Skv * D;
    const __half* Vb = p.V + static_cast<size_t>(bh) * p.Skv * D;
    const __half* Qb = p.Q + static_cast<size_t>(bh) * p.Sq * D;
    const uint32_t ring = smem_u32(fd_smem) + static_cast<uint32_t>(warp * FD_STAGES * 2 * TILE_BYTES);

    // requests tile `tile` (K then V) into stage s: each lane copies 16-byte chunks, row by row
    auto request = [&](int tile, int s) {
        const int k0 = key_lo + tile * FD_TILE;
        const uint32_t kdst = ring + static_cast<uint32_t>(s * 2 * TILE_BYTES);
        const uint32_t vdst = kdst + TILE_BYTES;
#pragma unroll
        for (int c = lane; c < FD_TILE * CHUNKS; c += 32) {
            const int row = c / CHUNKS, ch = c % CHUNKS;
            const int key = k0 + row;
            const int ok = key < key_hi ? 16 : 0;
            const size_t off = static_cast<size_t>(ok ? key : key_lo) * D + ch * 8;
            const uint32_t sw = static_cast<uint32_t>(row * ROW_BYTES + ((ch ^ (row & 7)) << 4));
            fd_cp_async16(kdst + sw, Kb + off, ok);
            fd_cp_async16(vdst + sw, Vb + off, ok);
        }
        fd_cp_commit();
    };
    const int my_tiles = n_tiles > warp ? (n_tiles - warp + FD_WARPS - 1) / FD_WARPS : 0;
    if (my_tiles > 0) request(warp, 0);
    if (my_tiles > 1) request(warp + FD_WARPS, 1);

    // Q as the A operand (rows = queries g and g + 8, 16 of the head dimension per tile): loaded once
    uint32_t qa[DT][4];
#pragma unroll
    for (int m = 0; m < DT; ++m) {
#pragma unroll
        for (int h = 0; h < 4; ++h) {
            const int row = g + 8 * (h & 1);
            const int col = 16 * m + 8 * (h >> 1) + 2 * t;
            qa[m][h] = row < p.Sq ? *reinterpret_cast<const uint32_t*>(Qb + static_cast<size_t>(row) * D + col) : 0u;
        }
    }

    float o[D / 8][4];     // output rows g ([0],[1]) and g + 8 ([2],[3]), columns 8n + 2t, 8n + 2t + 1
#pragma unroll
    for (int n = 0; n < D / 8; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};   // rows g and g + 8, log2 units
    // the last key query row r may see: all of them, or with the causal mask Skv - Sq + r
    const int lim0 = p.causal ? p.Skv - p.Sq + g : p.Skv - 1;
    const int lim1 = p.causal ? p.Skv - p.Sq + g + 8 : p.Skv - 1;

    for (int i = 0; i < my_tiles; ++i) {
        const int s = i & 1;
        if (i + 1 < my_tiles) fd_cp_wait<1>(); else fd_cp_wait<0>();
        __syncwarp();
        const uint32_t kt = ring + static_cast<uint32_t>(s * 2 * TILE_BYTES);
        const uint32_t vt = kt + TILE_BYTES;
        const int k0 = key_lo + (warp + FD_WARPS * i) * FD_TILE;

        // S = Q K^T for 16 queries x 16 keys: sc[nt] holds keys k0 + 8 nt + 2t, +1 for rows g / g + 8
        float sc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
        for (int m = 0; m < DT; ++m) {
            // four 8x8 blocks: (keys 0-7 | 8-15) x (chunk 2m | 2m + 1); lane i addresses row i % 8 of block i / 8
            const int blk = lane >> 3, r = lane & 7;
            const int key = (blk >> 1) * 8 + r, ch = 2 * m + (blk & 1);
            uint32_t b00, b01, b10, b11;
            fd_ldmatrix_x4(kt + static_cast<uint32_t>(key * ROW_BYTES + ((ch ^ (key & 7)) << 4)), b00, b01, b10, b11);
            fd_mma(sc[0], qa[m][0], qa[m][1], qa[m][2], qa[m][3], b00, b01);
            fd_mma(sc[1], qa[m][0], qa[m][1], qa[m][2], qa[m][3], b10, b11);
        }
        // scale, mask, running maximum
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int key = k0 + 8 * nt + 2 * t + (e & 1);
                const int lim = (e & 2) ? lim1 : lim0;
                const bool seen = key <= lim && key < key_hi;
                sc[nt][e] = seen ? sc[nt][e] * p.scale_log2 : -INFINITY;
                mx[e >> 1] = fmaxf(mx[e >> 1], sc[nt][e]);
            }
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
        }
        float corr[2], m_new[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            m_new[h] = fmaxf(m_run[h], mx[h]);
            // a row that has seen nothing yet keeps maximum -inf: use 0 as the reference so that exp2 stays finite
            const float ref = m_new[h] == -INFINITY ? 0.f : m_new[h];
            corr[h] = exp2f(m_run[h] - ref);      // exp2(-inf) = 0 on the first tile
            m_run[h] = m_new[h];
            m_new[h] = ref;
        }
        float rs[2] = {0.f, 0.f};
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                sc[nt][e] = exp2f(sc[nt][e] - m_new[e >> 1]);
                rs[e >> 1] += sc[nt][e];
            }
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            rs[h] += __shfl_xor_sync(0xffffffffu, rs[h], 1);
            rs[h] += __shfl_xor_sync(0xffffffffu, rs[h], 2);
            l_run[h] = l_run[h] * corr[h] + rs[h];
        }
#pragma unroll
        for (int n = 0; n < D / 8; ++n) {
            o[n][0] *= corr[0];
            o[n][1] *= corr[0];
            o[n][2] *= corr[1];
            o[n][3] *= corr[1];
        }
        // P (fp16) is the A operand of P V: rows g / g + 8, keys 2t, 2t+1 and 8 + 2t, 8 + 2t + 1
        const uint32_t pa0 = fd_pack(sc[0][0], sc[0][1]), pa1 = fd_pack(sc[0][2], sc[0][3]);
        const uint32_t pa2 = fd_pack(sc[1][0], sc[1][1]), pa3 = fd_pack(sc[1][2], sc[1][3]);
#pragma unroll
        for (int pr = 0; pr < D / 16; ++pr) {
            // V^T blocks for output columns 16 pr .. 16 pr + 15: (keys 0-7 | 8-15) x (chunk 2 pr | 2 pr + 1)
            const int blk = lane >> 3, r = lane & 7;
            const int key = (blk & 1) * 8 + r, ch = 2 * pr + (blk >> 1);
            uint32_t v00, v01, v10, v11;
            fd_ldmatrix_x4_trans(vt + static_cast<uint32_t>(key * ROW_BYTES + ((ch ^ (key & 7)) << 4)), v00, v01, v10, v11);
            fd_mma(o[2 * pr], pa0, pa1, pa2, pa3, v00, v01);
            fd_mma(o[2 * pr + 1], pa0, pa1, pa2, pa3, v10, v11);
        }
        __syncwarp();   // every lane is done with stage s before it is refilled
        if (i + 2 < my_tiles) request(warp + FD_WARPS * (i + 2), s);
    }

    // ---- merge the four warps: partial rows, maximum and sum per warp in shared memory (over the ring)
    __syncthreads();
    float* part = reinterpret_cast<float*>(fd_smem);   // [warp][16 rows][MERGE_PITCH]; maximum and sum at columns D, D + 1
    {
        float* mine = part + static_cast<size_t>(warp) * FD_MAX_SQ * MERGE_PITCH;
#pragma unroll
        for (int n = 0; n < D / 8; ++n) {
            mine[g * MERGE_PITCH + 8 * n + 2 * t] = o[n][0];
            mine[g * MERGE_PITCH + 8 * n + 2 * t + 1] = o[n][1];
            mine[(g + 8) * MERGE_PITCH + 8 * n + 2 * t] = o[n][2];
            mine[(g + 8) * MERGE_PITCH + 8 * n + 2 * t + 1] = o[n][3];
        }
        if (t == 0) {
            mine[g * MERGE_PITCH + D] = m_run[0];
            mine[g * MERGE_PITCH + D + 1] = l_run[0];
            mine[(g + 8) * MERGE_PITCH + D] = m_run[1];
            mine[(g + 8) * MERGE_PITCH + D + 1] = l_run[1];
        }
    }
    __syncthreads();
    for (int e = threadIdx.x; e < p.Sq * D; e += FD_THREADS) {
        const int row = e / D, col = e - row * D;
        float mstar = -INFINITY;
#pragma unroll
        for (int w = 0; w < FD_WARPS; ++w) mstar = fmaxf(mstar, part[(w * FD_MAX_SQ + row) * MERGE_PITCH + D]);
        const float ref = mstar == -INFINITY ? 0.f : mstar;
        float acc = 0.f, l = 0.f;
#pragma unroll
        for (int w = 0; w < FD_WARPS; ++w) {
            const float* pw = part + (w * FD_MAX_SQ + row) * MERGE_PITCH;
            const float wgt = exp2f(pw[D] - ref);
            acc += wgt * pw[col];
            l += wgt * pw[D + 1];
        }
        if (p.splits == 1) {
            const size_t idx = (static_cast<size_t>(bh) * p.Sq + row) * D + col;
            if (WB_DEBUG_INDEX(row < p.Sq && col < D, p.status, 107, row)) p.O[idx] = __float2half_rn(l > 0.f ? acc / l : 0.f);
        } else {
            float* dst = p.ws + ((static_cast<size_t>(bh) * p.splits + split) * p.Sq + row) * (D + 2);
            dst[col] = acc;
            if (col == 0) {
                dst[D] = mstar;
                dst[D + 1] = l;
            }
        }
    }
}

// Merges the splits of one (batch, head) in split order: out = sum_s w_s O_s / sum_s w_s l_s, w_s = 2^(m_s - max m).
template <int D>
__global__ void __launch_bounds__(D) fmha_decode_merge_kernel(const FdParams p) {
    // one CTA per (batch, head, query row), one thread per output column; all loads of a thread are
    // issued before the first use (the maxima first, then every split's value and sum)
    const int bh = blockIdx.x, row = blockIdx.y, col = threadIdx.x;
    const float* base = p.ws + (static_cast<size_t>(bh) * p.splits * p.Sq + row) * (D + 2);
    const size_t stride = static_cast<size_t>(p.Sq) * (D + 2);
    float mstar = -INFINITY;
    for (int s = 0; s < p.splits; ++s) mstar = fmaxf(mstar, base[s * stride + D]);
    const float ref = mstar == -INFINITY ? 0.f : mstar;
    float acc = 0.f, l = 0.f;
    for (int s = 0; s < p.splits; ++s) {
        const float wgt = exp2f(base[s * stride + D] - ref);
        acc += wgt * base[s * stride + col];
        l += wgt * base[s * stride + D + 1];
    }
    p.O[(static_cast<size_t>(bh) * p.Sq + row) * D + col] = __float2half_rn(l > 0.f ? acc / l : 0.f);
}

static void fd_plan(int BH, int Skv, int sms, int* splits, int* keys_per_split) {
    // enough CTAs for about three per SM, at least 256 keys (four tiles per warp) each
    int s = (3 * sms + BH - 1) / BH;
    const int max_s = (Skv + 255) / 256;
    if (s > max_s) s = max_s;
    if (s < 1) s = 1;
    int per = (Skv + s - 1) / s;
    per = (per + FD_TILE - 1) / FD_TILE * FD_TILE;
    s = (Skv + per - 1) / per;
    *splits = s;
    *keys_per_split = per;
}

template <int D>
static int fd_launch(const FdParams& p, cudaStream_t stream) {
    constexpr int RING = FD_WARPS * FD_STAGES * 2 * FD_TILE * D * 2;
    constexpr int MERGE = FD_WARPS * FD_MAX_SQ * (D + 4) * 4;
    constexpr int SMEM = RING > MERGE ? RING : MERGE;
    static std::atomic<bool> attr_set[64];
    int dev = 0;
    WB_CHECK_CUDA(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64 && !attr_set[dev].load(std::memory_order_acquire)) {
        WB_CHECK_CUDA(cudaFuncSetAttribute(fmha_decode_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM));
        attr_set[dev].store(true, std::memory_order_release);
    }
    dim3 grid(p.splits, p.B * p.H);
    fmha_decode_kernel<D><<<grid, FD_THREADS, SMEM, stream>>>(p);
    WB_CHECK_CUDA(cudaGetLastError());
    if (p.splits > 1) {
        fmha_decode_merge_kernel<D><<<dim3(p.B * p.H, p.Sq), D, 0, stream>>>(p);
        WB_CHECK_CUDA(cudaGetLastError());
    }
    return WMMA_OPS_OK;
}

}  // namespace wb

extern "C" size_t wmma_ops_fmha_decode_workspace_bytes(int B, int H, int Sq, int Skv, int D) {
    if (B < 1 || H < 1 || Sq < 1 || Skv < 1) return 0;
    int splits, per;
    wb::fd_plan(B * H, Skv, wb::sm_count(), &splits, &per);
    if (splits <= 1) return 0;
    return static_cast<size_t>(B) * H * splits * Sq * (D + 2) * sizeof(float);
}

extern "C" int wmma_ops_fmha_decode(const void* Q, const void* K, const void* V, void* O, int B, int H, int Sq, int Skv, int D,
                                    float scale, int causal, void* workspace, size_t workspace_bytes, int* status,
                                    void* stream) {
    using namespace wb;
    WB_REQUIRE(B >= 0 && H >= 0 && Sq >= 0 && Skv >= 0, WMMA_OPS_ERR_INVALID, "flash_attention: negative dimension");
    WB_REQUIRE(D == 64 || D == 128, WMMA_OPS_ERR_INVALID, "flash_attention: head dimension must be 64 or 128 (got %d)", D);
    WB_REQUIRE(Sq <= FD_MAX_SQ, WMMA_OPS_ERR_INVALID, "flash_attention (decode): at most %d query rows (got %d)", FD_MAX_SQ, Sq);
    WB_REQUIRE(Skv >= Sq, WMMA_OPS_ERR_INVALID, "flash_attention (decode): fewer keys (%d) than queries (%d)", Skv, Sq);
    if (B == 0 || H == 0 || Sq == 0) return WMMA_OPS_OK;
    WB_REQUIRE(Q != nullptr && K != nullptr && V != nullptr && O != nullptr, WMMA_OPS_ERR_INVALID,
               "flash_attention: null pointer");
    WB_REQUIRE(static_cast<long long>(B) * H <= 65535, WMMA_OPS_ERR_INVALID,
               "flash_attention: B*H must not exceed 65535 (got %lld)", static_cast<long long>(B) * H);
    for (const void* ptr : {Q, K, V, static_cast<const void*>(O)})
        WB_REQUIRE(reinterpret_cast<uintptr_t>(ptr) % 16 == 0, WMMA_OPS_ERR_INVALID,
                   "flash_attention: tensors must be 16-byte aligned");
    FdParams p;
    p.Q = static_cast<const __half*>(Q);
    p.K = static_cast<const __half*>(K);
    p.V = static_cast<const __half*>(V);
    p.O = static_cast<__half*>(O);
    p.B = B;
    p.H = H;
    p.Sq = Sq;
    p.Skv = Skv;
    p.D = D;
    fd_plan(B * H, Skv, sm_count(), &p.splits, &p.keys_per_split);
    if (scale < 0.f) scale = 1.0f / sqrtf(static_cast<float>(D));
    p.scale_log2 = scale * 1.4426950408889634f;
    p.causal = causal ? 1 : 0;
    p.status = status;
    p.ws = static_cast<float*>(workspace);
    if (p.splits > 1) {
        const size_t need = static_cast<size_t>(B) * H * p.splits * Sq * (D + 2) * sizeof(float);
        WB_REQUIRE(workspace != nullptr && workspace_bytes >= need, WMMA_OPS_ERR_WORKSPACE,
                   "flash_attention (decode): %d key splits need %zu bytes of workspace (got %zu); see "
                   "wmma_ops_fmha_decode_workspace_bytes",
                   p.splits, need, workspace_bytes);
    }
    if (D == 128) return fd_launch<128>(p, static_cast<cudaStream_t>(stream));
    return fd_launch<64>(p, static_cast<cudaStream_t>(stream));
}
