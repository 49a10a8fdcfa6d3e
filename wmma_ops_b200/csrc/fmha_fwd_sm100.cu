// Flash-attention forward for sm_100a: O = softmax(scale * Q K^T [+ causal mask]) V.
//
// Implements the signature the reference documents, flash_attention(Q, K, V, causal, scale) with
// Q, K, V [B,H,N,D] fp16 (README.md:221-251); the reference's own kernel is not in its tree, so
// the arithmetic follows the fp32 softmax-attention oracle.
//
// One CTA owns 128 query rows of one (batch, head) and walks the key/value sequence in tiles
// of 64 with an online softmax; two such CTAs share an SM:
//   warp 0      TMA producer: Q once, then K and V tiles into two-stage rings
//   warp 1      TMEM owner and issuer of both S = Q K^T and O += P V (fp32, TMEM)
//   warps 2..5  softmax, one thread per query row: read the row's 64 scores from TMEM, keep the
//               row's reference maximum and sum, write P (fp16) back into tensor memory over the
//               row's own scores, from where P V reads it as its A operand; rescale O in TMEM on
//               the rare tiles where the reference moves, and at the end store O / l as fp16.
// Two S accumulators let Q K^T of tile i+1 run on the tensor cores while the softmax warps
// work on tile i. K is a K-major operand; V, read as [kv, d] with d contiguous,
// is an MN-major operand, so neither is transposed.
#include "host_common.cuh"
#include "ptx.cuh"

namespace wb {

constexpr int FA_BM = 128;  // query rows per CTA
constexpr int FA_THREADS = 192;  // warp 0 producer, warp 1 MMA issuer, warps 2..5 softmax

// BN = keys per tile. BN = 64 keeps a CTA at 96 KB of shared memory and 256 TMEM columns (D = 128),
// so two CTAs share an SM and one CTA's softmax latency hides behind the other's work.
template <int D, int BN>
struct FaCfg {
    static constexpr int DB = D / 64;                   // 64-wide head-dim blocks
    static constexpr int Q_TILE_BYTES = FA_BM * D * 2;
    static constexpr int Q_BOX_BYTES = FA_BM * 64 * 2;  // one [128 rows x 64 halves] box
    static constexpr int KV_TILE_BYTES = BN * D * 2;
    static constexpr int KV_BOX_BYTES = BN * 64 * 2;    // one [BN rows x 64 halves] box
    static constexpr int SMEM_BYTES = Q_TILE_BYTES + 4 * KV_TILE_BYTES + 1024 + 256;
    static constexpr int S_COL0 = 0, S_COL1 = BN, O_COL = 2 * BN;
    static constexpr int TMEM_COLS = (2 * BN + D <= 256) ? 256 : 512;
    static constexpr int CTAS_PER_SM = (TMEM_COLS == 256 && SMEM_BYTES <= 113 * 1024) ? 2 : 1;
};

struct FaParams {
    __half* O;
    long long o_row, o_head, o_batch;  // element strides of O between tokens, heads and sequences
    int B, H, S, D;
    float scale_log2;  // scale * log2(e)
    int causal;
    int* status;
};

__device__ __forceinline__ void fa_report(int* status, int role, int detail) {
    if (status != nullptr && atomicCAS(status, 0, 3) == 0) {
        status[1] = role;
        status[2] = static_cast<int>(blockIdx.x + gridDim.x * blockIdx.y);
        status[3] = detail;
    }
}

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// three-input maximum (one instruction on sm_100)
__device__ __forceinline__ float fmax3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

__device__ __forceinline__ uint32_t pack_half2(float a, float b) {
    const __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&h);
}

template <int D, int BN>
__global__ void __launch_bounds__(FA_THREADS, (FaCfg<D, BN>::CTAS_PER_SM))
fmha_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                const __grid_constant__ CUtensorMap tmap_v, const FaParams p) {
    using Cfg = FaCfg<D, BN>;
    constexpr int FA_BN = BN;
    extern __shared__ uint8_t fa_smem_raw[];
    const uint32_t smem_base = (smem_u32(fa_smem_raw) + 1023u) & ~1023u;
    const uint32_t q_smem = smem_base;
    auto k_smem = [&](int s) { return smem_base + Cfg::Q_TILE_BYTES + s * Cfg::KV_TILE_BYTES; };
    auto v_smem = [&](int s) { return smem_base + Cfg::Q_TILE_BYTES + (2 + s) * Cfg::KV_TILE_BYTES; };
    const uint32_t bar_base = smem_base + Cfg::Q_TILE_BYTES + 4 * Cfg::KV_TILE_BYTES;
    const uint32_t q_full = bar_base;
    auto k_full = [&](int s) { return bar_base + 8u * (1 + s); };
    auto k_empty = [&](int s) { return bar_base + 8u * (3 + s); };
    auto v_full = [&](int s) { return bar_base + 8u * (5 + s); };
    auto v_empty = [&](int s) { return bar_base + 8u * (7 + s); };
    auto s_full = [&](int s) { return bar_base + 8u * (9 + s); };
    auto s_empty = [&](int s) { return bar_base + 8u * (11 + s); };
    auto p_ready = [&](int s) { return bar_base + 8u * (13 + s); };
    // P V of tile i reports to pv_done(i & 1). A softmax thread waits on it only when it has to
    // rescale O (tile i - 1's barrier, at tile i) and at the end. The parity wait is unambiguous
    // without looking at every phase: at tile i, P V of tile i - 3 (the previous phase of that
    // barrier) is known to be complete, because Q K^T of tile i - 1 could only be issued after it,
    // and P V of tile i + 1 (the next phase) cannot complete before this thread has arrived for it.
    auto pv_done = [&](int b) { return bar_base + 8u * (15 + b); };
    const uint32_t tmem_slot = bar_base + 8u * 17;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    // Heavy (late) query tiles first when causal, so the tail of the grid is made of short CTAs.
    const int q_tiles = gridDim.x;
    const int q_tile = p.causal ? (q_tiles - 1 - static_cast<int>(blockIdx.x)) : static_cast<int>(blockIdx.x);
    const int bh = blockIdx.y;
    const int b_idx = bh / p.H, h_idx = bh - b_idx * p.H;  // the tensor maps are (D, token, head, sequence)
    const int q0 = q_tile * FA_BM;
    const int kv_tiles_all = (p.S + FA_BN - 1) / FA_BN;
    const int n_tiles = p.causal ? min(kv_tiles_all, (q0 + FA_BM - 1) / FA_BN + 1) : kv_tiles_all;

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int s = 0; s < 2; ++s) {
            mbar_init(k_full(s), 1);
            mbar_init(k_empty(s), 1);
            mbar_init(v_full(s), 1);
            mbar_init(v_empty(s), 1);
            mbar_init(s_full(s), 1);
            mbar_init(s_empty(s), 1);
            mbar_init(p_ready(s), 128);
        }
        mbar_init(pv_done(0), 1);
        mbar_init(pv_done(1), 1);
        fence_barrier_init();
        fence_proxy_async_smem();
        prefetch_tmap(&tmap_q);
        prefetch_tmap(&tmap_k);
        prefetch_tmap(&tmap_v);
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

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            mbar_arrive_expect_tx(q_full, Cfg::Q_TILE_BYTES);
#pragma unroll
            for (int b = 0; b < Cfg::DB; ++b)
                tma_load_4d(q_smem + b * Cfg::Q_BOX_BYTES, &tmap_q, q_full, b * 64, q0, h_idx, b_idx);
            for (int i = 0; i < n_tiles; ++i) {
                const int s = i & 1;
                const uint32_t ph = (i >> 1) & 1;
                if (!mbar_wait(k_empty(s), ph ^ 1u)) {
                    fa_report(p.status, 0, i);
                    break;
                }
                mbar_arrive_expect_tx(k_full(s), Cfg::KV_TILE_BYTES);
#pragma unroll
                for (int b = 0; b < Cfg::DB; ++b)
                    tma_load_4d(k_smem(s) + b * Cfg::KV_BOX_BYTES, &tmap_k, k_full(s), b * 64, i * FA_BN, h_idx, b_idx);
                if (!mbar_wait(v_empty(s), ph ^ 1u)) {
                    fa_report(p.status, 0, -i - 1);
                    break;
                }
                mbar_arrive_expect_tx(v_full(s), Cfg::KV_TILE_BYTES);
#pragma unroll
                for (int b = 0; b < Cfg::DB; ++b)
                    tma_load_4d(v_smem(s) + b * Cfg::KV_BOX_BYTES, &tmap_v, v_full(s), b * 64, i * FA_BN, h_idx, b_idx);
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        // One thread issues both products, in the order Q K^T(i), P V(i-1), Q K^T(i+1), ...
        // tcgen05.mma operations of one thread execute in the order they were issued, so
        // Q K^T(i+1), which overwrites the S buffer that holds P(i-1), may be issued right after
        // P V(i-1) without waiting for it to complete. (With the two products issued by different
        // threads that wait was needed, and the chain softmax(i-1) done -> P V(i-1) issued and
        // complete -> Q K^T(i+1) issued and complete was longer than softmax(i): the softmax warps
        // stood waiting for scores.)
        if (lane == 0) {
            constexpr uint32_t idesc_s = make_idesc_f16_f32(FA_BM, FA_BN, false, false);
            constexpr uint32_t idesc_o = make_idesc_f16_f32(FA_BM, D, false, true);
            bool ok = mbar_wait(q_full, 0);
            if (!ok) fa_report(p.status, 1, -1);
            auto issue_pv = [&](int i) -> bool {
                const int s = i & 1;
                const uint32_t ph = (i >> 1) & 1;
                if (!mbar_wait(v_full(s), ph) || !mbar_wait(p_ready(s), ph)) {
                    fa_report(p.status, 1, 1000 + i);
                    return false;
                }
                tc_fence_after_sync();
#pragma unroll
                for (int kk = 0; kk < FA_BN / 16; ++kk) {
                    // P (fp16, written by the softmax warps over the start of S buffer s) is the A
                    // operand straight from tensor memory: 16 keys = 8 columns per MMA.
                    // V: MN-major, 16 keys = 2048 bytes further; 64-wide d blocks KV_BOX_BYTES apart
                    const uint64_t b_desc = make_smem_desc_sw128(v_smem(s) + kk * 2048, Cfg::KV_BOX_BYTES, 1024);
                    umma_f16_ts(tmem_base + Cfg::O_COL, tmem_base + (s ? Cfg::S_COL1 : Cfg::S_COL0) + kk * 8, b_desc,
                                idesc_o, (i > 0 || kk > 0) ? 1u : 0u);
                }
                umma_commit(v_empty(s));
                umma_commit(pv_done(s));
                return true;
            };
            for (int i = 0; ok && i < n_tiles; ++i) {
                const int s = i & 1;
                const uint32_t ph = (i >> 1) & 1;
                if (!mbar_wait(k_full(s), ph)) {
                    fa_report(p.status, 1, i);
                    ok = false;
                    break;
                }
                tc_fence_after_sync();
                const uint32_t s_tmem = tmem_base + (s ? Cfg::S_COL1 : Cfg::S_COL0);
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    const uint64_t a_desc =
                        make_smem_desc_sw128(q_smem + (kk >> 2) * Cfg::Q_BOX_BYTES + (kk & 3) * 32, 16, 1024);
                    const uint64_t b_desc =
                        make_smem_desc_sw128(k_smem(s) + (kk >> 2) * Cfg::KV_BOX_BYTES + (kk & 3) * 32, 16, 1024);
                    umma_f16(s_tmem, a_desc, b_desc, idesc_s, kk > 0 ? 1u : 0u);
                }
                umma_commit(k_empty(s));
                umma_commit(s_full(s));
                if (i > 0) ok = issue_pv(i - 1);
            }
            if (ok && n_tiles > 0) issue_pv(n_tiles - 1);
        }
    } else {
        // ------------------------------------------------------------ softmax warps (2..5)
        // One thread per query row: warp w owns the TMEM lane quadrant w & 3, i.e. rows
        // 32 (w & 3) .. + 31, and each of its threads all BN keys of a tile and all D columns of
        // O. Nothing is exchanged between threads: a row's maximum, sum and probabilities live in
        // one thread, and its P overwrites the row's own scores in tensor memory.
        const int quad = warp & 3;
        const int row = quad * 32 + lane;
        const int q = q0 + row;
        const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
        const float sl2 = fmaxf(p.scale_log2, 1e-30f);  // > 0, so that -inf * sl2 stays -inf
        float m_run = -INFINITY;  // reference (scale * log2e * s units) the probabilities are taken against
        float l_run = 0.f;        // running sum of exp2(.)
        bool ok = true;
        for (int i = 0; ok && i < n_tiles; ++i) {
            const int s = i & 1;
            const uint32_t ph = (i >> 1) & 1;
            if (!mbar_wait(s_full(s), ph)) {
                fa_report(p.status, 2, i);
                ok = false;
                break;
            }
            tc_fence_after_sync();
            const uint32_t s_addr = tmem_base + (s ? Cfg::S_COL1 : Cfg::S_COL0) + lane_addr;
            const int kv0 = i * FA_BN;
            const bool need_mask = (p.causal && i * FA_BN + FA_BN - 1 > q0) || (i * FA_BN + FA_BN > p.S);
            const int col_limit = p.causal ? min(p.S - 1, q) : p.S - 1;  // last visible key

            // the row's raw scores, kept in registers (the scale is applied inside the exponent's
            // FMA; it is positive, so the maximum can be taken on the raw scores)
            float x[FA_BN];
            {
                uint32_t v0[32], v1[32];  // both loads in flight before the one wait
                tmem_ld_32x32b_x32(s_addr, v0);
                tmem_ld_32x32b_x32(s_addr + 32, v1);
                tmem_wait_ld();
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    x[j] = __uint_as_float(v0[j]);
                    x[32 + j] = __uint_as_float(v1[j]);
                }
            }
            if (need_mask) {
#pragma unroll
                for (int j = 0; j < FA_BN; ++j)
                    if (kv0 + j > col_limit) x[j] = -INFINITY;
            }
            float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;  // four chains of three-input maxima
#pragma unroll
            for (int j = 0; j < FA_BN; j += 8) {
                mx0 = fmax3(mx0, x[j], x[j + 1]);
                mx1 = fmax3(mx1, x[j + 2], x[j + 3]);
                mx2 = fmax3(mx2, x[j + 4], x[j + 5]);
                mx3 = fmax3(mx3, x[j + 6], x[j + 7]);
            }
            const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * sl2;
            // Lazy reference: it only moves when the tile's maximum exceeds it by more than 8 (in log2
            // units), so probabilities stay below 256 (fine in fp16, sums in fp32) and O is rescaled a
            // few times per row instead of once per tile.
            const float m_cand = fmaxf(m_run, mx);
            const bool move = (m_cand - m_run) > 8.f;  // false for -inf - -inf (NaN), true for x - -inf
            const float m_new = move ? m_cand : m_run;
            const float m_safe = (m_new == -INFINITY) ? 0.f : m_new;
            const float alpha = move ? fast_exp2(m_run - m_safe) : 1.f;

            // probabilities -> fp16, written over the start of the row's own scores
            float sum0 = 0.f, sum1 = 0.f;
            uint32_t pk[FA_BN / 2];
#pragma unroll
            for (int j = 0; j < FA_BN / 2; ++j) {
                const float e0 = fast_exp2(fmaf(x[2 * j], sl2, -m_safe));
                const float e1 = fast_exp2(fmaf(x[2 * j + 1], sl2, -m_safe));
                sum0 += e0;
                sum1 += e1;
                pk[j] = pack_half2(e0, e1);
            }
            static_assert(FA_BN == 64, "the P store below is written for 64-key tiles");
            tmem_st_32x32b_x32(s_addr, pk);
            l_run = l_run * alpha + (sum0 + sum1);
            m_run = m_new;

            if (i > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
                // O holds the sum through tile i-1; bring the row to the new reference
                if (!mbar_wait(pv_done(s ^ 1), static_cast<uint32_t>((i - 1) >> 1) & 1u)) {
                    fa_report(p.status, 2, 1000 + i);
                    ok = false;
                    break;
                }
                tc_fence_after_sync();
                const uint32_t o_addr = tmem_base + Cfg::O_COL + lane_addr;
#pragma unroll 1
                for (int c = 0; c < D / 32; ++c) {
                    uint32_t v[32];
                    tmem_ld_32x32b_x32(o_addr + c * 32, v);
                    tmem_wait_ld();
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) * alpha);
                    tmem_st_32x32b_x32(o_addr + c * 32, v);
                }
            }
            tmem_wait_st();
            tc_fence_before_sync();
            mbar_arrive(p_ready(s));
        }
        if (ok) {
            if (!mbar_wait(pv_done((n_tiles - 1) & 1), static_cast<uint32_t>((n_tiles - 1) >> 1) & 1u)) {
                fa_report(p.status, 2, -1);
                ok = false;
            }
        }
        if (ok) {
            tc_fence_after_sync();
            const float inv = (l_run > 0.f) ? 1.f / l_run : 0.f;
            const uint32_t o_addr = tmem_base + Cfg::O_COL + lane_addr;
            __half* out = p.O + b_idx * p.o_batch + h_idx * p.o_head + static_cast<long long>(q) * p.o_row;
#pragma unroll 1
            for (int c = 0; c < D / 32; ++c) {
                uint32_t v[32];
                tmem_ld_32x32b_x32(o_addr + c * 32, v);
                tmem_wait_ld();
                if (q < p.S && WB_DEBUG_INDEX(q >= 0 && bh >= 0 && bh < p.B * p.H, p.status, 103, q)) {
#pragma unroll
                    for (int g = 0; g < 4; ++g) {
                        uint4 o;
                        o.x = pack_half2(__uint_as_float(v[g * 8 + 0]) * inv, __uint_as_float(v[g * 8 + 1]) * inv);
                        o.y = pack_half2(__uint_as_float(v[g * 8 + 2]) * inv, __uint_as_float(v[g * 8 + 3]) * inv);
                        o.z = pack_half2(__uint_as_float(v[g * 8 + 4]) * inv, __uint_as_float(v[g * 8 + 5]) * inv);
                        o.w = pack_half2(__uint_as_float(v[g * 8 + 6]) * inv, __uint_as_float(v[g * 8 + 7]) * inv);
                        *reinterpret_cast<uint4*>(out + c * 32 + g * 8) = o;
                    }
                }
            }
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
    }
}

// st: element strides {row, head, batch} of Q, K and V (the last dimension, D, is contiguous)
template <int D, int BN>
static int launch_fmha(const void* Q, const void* K, const void* V, const long long* st, const FaParams& p,
                       cudaStream_t stream) {
    using Cfg = FaCfg<D, BN>;
    static std::atomic<bool> attr_set[64];  // per device; setting the attribute twice is harmless
    int dev = 0;
    WB_CHECK_CUDA(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64 && !attr_set[dev].load(std::memory_order_acquire)) {
        WB_CHECK_CUDA(cudaFuncSetAttribute(fmha_fwd_kernel<D, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           Cfg::SMEM_BYTES));
        attr_set[dev].store(true, std::memory_order_release);
    }
    CUtensorMap tq, tk, tv;
    // (D, token, head, sequence): rows past the end of a sequence read as zeros whatever the layout
    const uint64_t dims[4] = {static_cast<uint64_t>(D), static_cast<uint64_t>(p.S), static_cast<uint64_t>(p.H),
                              static_cast<uint64_t>(p.B)};
    const uint32_t box_q[4] = {64, FA_BM, 1, 1};
    const uint32_t box_kv[4] = {64, BN, 1, 1};
    const void* base[3] = {Q, K, V};
    CUtensorMap* maps[3] = {&tq, &tk, &tv};
    for (int i = 0; i < 3; ++i) {
        const uint64_t strides[4] = {0, static_cast<uint64_t>(st[3 * i]) * 2, static_cast<uint64_t>(st[3 * i + 1]) * 2,
                                     static_cast<uint64_t>(st[3 * i + 2]) * 2};
        const int rc = encode_tmap(maps[i], CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, base[i], dims, strides,
                                   i == 0 ? box_q : box_kv, CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc != WMMA_OPS_OK) return rc;
    }
    dim3 grid((p.S + FA_BM - 1) / FA_BM, p.B * p.H);
    fmha_fwd_kernel<D, BN><<<grid, FA_THREADS, Cfg::SMEM_BYTES, stream>>>(tq, tk, tv, p);
    WB_CHECK_CUDA(cudaGetLastError());
    return WMMA_OPS_OK;
}

}  // namespace wb

extern "C" int wmma_ops_fmha_fwd_strided(const void* Q, const void* K, const void* V, void* O, int B, int H, int S,
                                         int D, const long long* strides, float scale, int causal, int* status,
                                         void* stream) {
    using namespace wb;
    WB_REQUIRE(B >= 0 && H >= 0 && S >= 0, WMMA_OPS_ERR_INVALID, "flash_attention: negative dimension");
    WB_REQUIRE(D == 64 || D == 128, WMMA_OPS_ERR_INVALID, "flash_attention: head dimension must be 64 or 128 (got %d)", D);
    if (B == 0 || H == 0 || S == 0) return WMMA_OPS_OK;
    WB_REQUIRE(Q != nullptr && K != nullptr && V != nullptr && O != nullptr && strides != nullptr, WMMA_OPS_ERR_INVALID,
               "flash_attention: null pointer");
    WB_REQUIRE(static_cast<long long>(B) * H <= 65535, WMMA_OPS_ERR_INVALID,
               "flash_attention: B*H must not exceed 65535 (got %lld)", static_cast<long long>(B) * H);
    for (const void* ptr : {Q, K, V, static_cast<const void*>(O)})
        WB_REQUIRE(reinterpret_cast<uintptr_t>(ptr) % 16 == 0, WMMA_OPS_ERR_INVALID,
                   "flash_attention: tensors must be 16-byte aligned");
    for (int i = 0; i < 12; ++i)
        WB_REQUIRE(strides[i] >= (i % 3 == 0 ? D : 1) && strides[i] % 8 == 0, WMMA_OPS_ERR_INVALID,
                   "flash_attention: strides must be multiples of 8 elements and rows at least D apart (stride %d is %lld)", i,
                   strides[i]);
    FaParams p;
    p.O = static_cast<__half*>(O);
    p.o_row = strides[9];
    p.o_head = strides[10];
    p.o_batch = strides[11];
    p.B = B;
    p.H = H;
    p.S = S;
    p.D = D;
    if (scale < 0.f) scale = 1.0f / sqrtf(static_cast<float>(D));
    p.scale_log2 = scale * 1.4426950408889634f;
    p.causal = causal ? 1 : 0;
    p.status = status;
    // 64-key tiles: two CTAs per SM (measured 850 vs 778 TFLOP/s with 128-key tiles at S = 4096)
    if (D == 128) return launch_fmha<128, 64>(Q, K, V, strides, p, static_cast<cudaStream_t>(stream));
    return launch_fmha<64, 64>(Q, K, V, strides, p, static_cast<cudaStream_t>(stream));
}

extern "C" int wmma_ops_fmha_fwd(const void* Q, const void* K, const void* V, void* O, int B, int H, int S,
                                 int D, float scale, int causal, int* status, void* stream) {
    // contiguous [B, H, S, D]
    const long long row = D, head = static_cast<long long>(S) * D, batch = static_cast<long long>(H) * S * D;
    const long long strides[12] = {row, head, batch, row, head, batch, row, head, batch, row, head, batch};
    return wmma_ops_fmha_fwd_strided(Q, K, V, O, B, H, S, D, strides, scale, causal, status, stream);
}
