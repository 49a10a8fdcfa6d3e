/*
 * wmma_ops_b200 — C ABI of the B200 (sm_100a) GEMM hot path.
 *
 * This is the boundary a binding of the reference's PyTorch extension module would call
 * instead of launching its HIP kernels: plain device pointers and sizes, a CUDA stream
 * passed as void*, int return codes. No torch types, no exceptions, and — except where a
 * function says otherwise — no allocation: every buffer, including scratch, is the caller's.
 *
 * Conventions
 *   - all matrix pointers are device pointers, row-major, contiguous, 16-byte aligned;
 *   - A is [M,K] fp16, B is [K,N] fp16, C is [M,N] fp32 (the reference's layouts,
 *     wmma_gemm.hip:45-60);
 *   - every function returns WMMA_OPS_OK (0) or a WMMA_OPS_ERR_* code; the message for the
 *     last failure on the calling thread is wmma_ops_last_error();
 *   - launches are asynchronous on `stream` (NULL = the legacy default stream);
 *   - `status` is an optional device pointer to 4 ints, zeroed by the caller. A kernel
 *     whose bounded wait gives up writes {code, role, block, detail} there and returns
 *     early instead of hanging; 0 in status[0] after synchronising means no kernel gave up.
 */
#ifndef WMMA_OPS_B200_H
#define WMMA_OPS_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define WMMA_OPS_OK 0
#define WMMA_OPS_ERR_INVALID 1     /* bad pointer, shape, alignment or option */
#define WMMA_OPS_ERR_CUDA 2        /* a CUDA runtime / driver call failed      */
#define WMMA_OPS_ERR_UNSUPPORTED 3 /* device is not sm_100                     */
#define WMMA_OPS_ERR_WORKSPACE 4   /* scratch buffer missing or too small      */

/* CTA tile shapes of the tcgen05 GEMM. They take the place of the reference's
 * TileConfig enum (wmma_tile_selection.hpp:17-23) and of matmul_tiled's 0..3
 * (wmma_gemm.hip:1504-1523). */
#define WMMA_OPS_TILE_AUTO (-1)
#define WMMA_OPS_TILE_128x64 0
#define WMMA_OPS_TILE_128x128 1
#define WMMA_OPS_TILE_128x256 2
#define WMMA_OPS_TILE_256x256_PAIR 3 /* two CTAs (one cluster) share one 256x256 tile */

/* Message of the last failing call on this thread ("" if none). Never NULL. */
const char* wmma_ops_last_error(void);

/* Library version: major * 10000 + minor * 100 + patch. */
int wmma_ops_version(void);

/* Leaves `sms` SMs (0..64, default 0) unoccupied by this library's persistent kernels, so that
 * kernels of other libraries launched on other streams (a collective that should overlap a
 * GEMM) find room to run. Process-wide; no counterpart in the reference (it is single-GPU). */
int wmma_ops_set_sm_margin(int sms);

/* Tile shape and split-K factor for an M x N x K product on a device with num_sms SMs
 * (num_sms <= 0: 148). Replaces select_optimal_tile (wmma_tile_selection.hpp:30-66) and
 * split_k::compute_config (wmma_xor_swizzle.hpp:293-332). Pure host arithmetic. */
int wmma_ops_select_tile(int M, int N, int K, int num_sms, int* tile_cfg, int* split_k);

/* Installs a measured tile table (process-wide; n_rows = 0 removes it). rows is n_rows x 6 ints
 * {M, N, K, num_sms, tile_cfg, split_k}: wmma_ops_select_tile, and every AUTO launch, then return
 * tile_cfg / split_k for any product in the same shape bucket (ceil(M/128), ceil(N/64), ceil(K/64))
 * on a device with num_sms SMs, and fall back to the built-in cost model otherwise. The table is
 * what the tuner (wmma_ops_b200/tune.py) measures and stores; it takes the place of the reference's
 * generated select_tuned_tile (autotune.py:131-283). */
int wmma_ops_set_tile_table(const int* rows, int n_rows);

/* Bytes of scratch wmma_ops_gemm_f16f32 needs for this split_k (0 when split_k <= 1):
 * split_k fp32 partial products of M x N, the layout of the reference's split-K
 * workspace (wmma_xor_swizzle.hpp:1196-1210). */
size_t wmma_ops_gemm_workspace_bytes(int M, int N, int K, int split_k);

/* C_out = alpha * (A . B) + beta * C_in, fp16 inputs, fp32 accumulate and output.
 * Replaces the launches in wmma_matmul (wmma_gemm.hip:1432-1470), wmma_matmul_tiled
 * (:1473-1528), wmma_matmul_adaptive (:1197-1263), wmma_gemm / _inplace / _adaptive
 * (:1891-2078) and the unbound split-K path (wmma_xor_swizzle.hpp:1172-1219).
 *   C_in   read only when beta != 0 and C_in != NULL (wmma_gemm.hip:653-660); may equal C_out.
 *   tile_cfg  WMMA_OPS_TILE_* ; AUTO picks tile and split_k with wmma_ops_select_tile.
 *   split_k   <= 1: one pass. > 1: K is cut into split_k slices, partials go to
 *             `workspace` ([split_k][M][N] fp32) and are summed in ascending slice order.
 *             With tile_cfg AUTO, pass split_k = 0 to let the table decide (the workspace
 *             must then hold wmma_ops_gemm_workspace_bytes(M, N, K, chosen split_k)).
 * Requirements: M >= 1, N % 8 == 0, K % 8 == 0 (16-byte row pitch for TMA). */
int wmma_ops_gemm_f16f32(const void* A, const void* B, const void* C_in, void* C_out, int M, int N,
                         int K, float alpha, float beta, int tile_cfg, int split_k, void* workspace,
                         size_t workspace_bytes, int* status, void* stream);

/* Split-K GEMM that allocates nothing and needs no workspace argument. It has no counterpart
 * in the reference. It is for callers that cannot call cudaMalloc where they need the product:
 * code living inside another framework's memory pool, plugins that are handed only their input
 * and output buffers, loops that must not risk the device-wide synchronisation an allocation
 * can cause. Same arithmetic and arguments as wmma_ops_gemm_f16f32; the partial products go to
 * a fixed 8 MiB array in device memory that belongs to the library (each GPU that loads the
 * library holds it until the process exits; wmma_ops_gemm_static_scratch_bytes() returns its
 * size). Limits and rules:
 *   - split_k * M * N * 4 bytes must fit in the array, otherwise WMMA_OPS_ERR_WORKSPACE with a
 *     message that names both sizes (with tile_cfg AUTO and split_k 0 the library's own choice
 *     of split_k is what is checked);
 *   - the first call on each device looks up the array's device address; make that call
 *     before any stream capture begins on that device;
 *   - every call on a device shares the one array: two calls whose kernels can overlap on the
 *     GPU (different streams, no ordering between them) race on it. Calls on one stream are
 *     safe. Nothing in the array has to be zero: each call overwrites every partial it reads. */
size_t wmma_ops_gemm_static_scratch_bytes(void);
int wmma_ops_gemm_f16f32_splitk_static(const void* A, const void* B, const void* C_in, void* C_out, int M,
                                       int N, int K, float alpha, float beta, int tile_cfg, int split_k,
                                       int* status, void* stream);

/* INT4 weight prepack ("W4-B200-v1"; the reference snapshot has no INT4 code, so the
 * format is defined here and restated in oracle/int4.py):
 *   codes    [K,N] uint8, values 0..15 (weight k,n = (code - 8) * scale[k / group][n])
 *   qweight  uint32 [K/64][ceil(N/128)][128][8]. Block (kb, nt) is 4 KB: for the 128 columns
 *            n = 128 nt + r (zero codes where n >= N) the codes k = 64 kb .. 64 kb + 63 as 8
 *            words per column; word j, nibble p (bits 4p..4p+3) holds
 *            k = 64 kb + 8 j + {0,2,4,6,1,3,5,7}[p].
 * Requirements: K % 64 == 0, N % 8 == 0. */
int wmma_ops_int4_prepack(const void* codes_u8, void* qweight, int K, int N, void* stream);

/* Inverse of wmma_ops_int4_prepack: qweight -> codes [K,N] uint8. */
int wmma_ops_int4_unpack(const void* qweight, void* codes_u8, int K, int N, void* stream);

/* W[k][n] = fp16(code - 8) * scales[k / group_size][n] (one fp16 multiply, round to nearest
 * even), written as [K,N] fp16. scales is [K/group_size, N] fp16. */
int wmma_ops_int4_dequant(const void* qweight, const void* scales, void* W_f16, int K, int N,
                          int group_size, void* stream);

/* Overlapped decode launches (off by default; process-wide). When on, the decode kernel
 * (M <= 16, split_k = 0) is launched as a programmatic dependent launch: its CTAs may start, and
 * load their scales and request their packed-weight segments, while the previous kernel of the
 * stream is still finishing; they wait for that kernel to complete before they read the
 * activations or touch the output. The caller promises that neither qweight nor scales is written
 * by the kernels queued just before the call (weights are static in decode). No counterpart in the
 * reference. */
int wmma_ops_set_w4a16_overlap(int enable);

/* The decode kernel's launch plan for an M x N x K product (M <= 16), host arithmetic only:
 * plan[0..13] = {grid, clusters, ksplit, units, groups_per_unit, units_per_chunk, ring_depth,
 * slot_bytes, reduction_pitch, shared_memory_bytes, groups_per_chunk_of_the_kernel_variant,
 * reduction_tiles_over_the_ring, k_blocks_per_segment, staged_row_pitch}. Columns are dealt in
 * units of 16 (pairs of a gate and an up group with WMMA_OPS_W4_OUT_F16_SILU_MUL) to `clusters`
 * clusters of `ksplit` CTAs; the CTAs of a cluster split K; activations and scales are staged in
 * shared memory one segment of K at a time. num_sms <= 0: 148. No counterpart in the reference. */
int wmma_ops_w4a16_decode_plan(int M, int N, int K, int group_size, int out_mode, int num_sms, int* plan);

/* Bytes of scratch wmma_ops_w4a16_gemm needs for this shape and split_k (partial sums + arrival
 * counters of the tcgen05 kernel's split plans); 0 when the plan has no partial sums, which includes
 * every product the decode kernel takes (M <= 16, split_k = 0). The buffer must be zero-filled
 * once: the kernels leave the counters (its first 64 KB) at zero, so one buffer can serve calls of
 * any shape; after a non-zero status word, zero it again before the next call. */
size_t wmma_ops_w4a16_workspace_bytes(int M, int N, int K, int split_k);

/* Split-K factor wmma_ops_w4a16_gemm picks when split_k == 0 and M > 16. */
int wmma_ops_w4a16_select_split(int M, int N, int K, int num_sms);

/* C[M,N] fp32 = A[M,K] fp16 . W, W dequantised on the fly from qweight / scales inside the
 * kernel, never materialised in global memory.
 * Requirements: K % 64 == 0, K % group_size == 0, group_size % 64 == 0, N % 8 == 0.
 * split_k: 0 = the library's plan, 1 = none, > 1 = that many K slices (needs workspace).
 * Arithmetic contract: weight[k][n] = (code - 8) * scale[k / group_size][n] exactly, fp16
 * activations, fp32 accumulation; the result is within 1e-3 (relative Frobenius) of that product.
 * Two kernels implement it and differ in where the fp16 scale is applied:
 *   M > 16 or split_k != 0  the tcgen05 kernel multiplies by the fp16-rounded weights of
 *          wmma_ops_int4_dequant (one rounding per weight, about 2e-4 relative);
 *   M <= 16 and split_k == 0  the decode kernel multiplies by the exact integers code - 8 and
 *          applies the scale to the fp32 sum of each 64-deep block (no weight rounding; half of
 *          the zero points are removed by a constant-operand MMA chain, 5e-7 relative). Every CTA
 *          owns a range of columns and walks all of K, sums are added in a fixed order
 *          (deterministic), and no workspace is needed. */
int wmma_ops_w4a16_gemm(const void* A, const void* qweight, const void* scales, void* C, int M,
                        int N, int K, int group_size, int split_k, void* workspace,
                        size_t workspace_bytes, int* status, void* stream);

/* wmma_ops_w4a16_gemm with a fused output stage (no counterpart in the reference):
 *   WMMA_OPS_W4_OUT_F32           C fp32 [M,N] = acc                      (what wmma_ops_w4a16_gemm does)
 *   WMMA_OPS_W4_OUT_F16           C fp16 [M,N] = half(alpha * acc)
 *   WMMA_OPS_W4_OUT_F16_SILU_MUL  C fp16 [M,N/2] = half(alpha * silu(in_scale * gate) * (in_scale * up)), where in every
 *                                 128-column tile of the weight the first 64 columns are gate columns
 *                                 and the last 64 the up columns of the same 64 outputs (N % 128 == 0).
 * in_scale (used by the last mode only; pass 1 otherwise) stands for a scale of the activations
 * that the caller did not apply: A may then be the unscaled tensor.
 * With M > 16 the fp16 modes run without partial sums (split_k 0 or 1). */
#define WMMA_OPS_W4_OUT_F32 0
#define WMMA_OPS_W4_OUT_F16 1
#define WMMA_OPS_W4_OUT_F16_SILU_MUL 2
int wmma_ops_w4a16_gemm_ex(const void* A, const void* qweight, const void* scales, void* C, int M, int N,
                           int K, int group_size, int split_k, int out_mode, float alpha, float in_scale,
                           void* workspace, size_t workspace_bytes, int* status, void* stream);

/* wmma_ops_w4a16_gemm_ex that tells a consumer how far it has got (no counterpart in the reference).
 * M > 16, split_k 0 or 1. The output is produced token block by token block (blocks of
 * wmma_ops_w4a16_token_block(M) rows, all column tiles of a block before the next block), and
 * block_done[b] (device memory, zero before the call, one int per token block) is incremented, after a
 * system-scope fence, each time one 128-column tile of block b has been written: block b is complete
 * when block_done[b] == ceil(N_out / 128), N_out = N. A kernel that runs beside this one (the sum over
 * the ranks, wmma_ops_switch_allreduce_following) can then consume the output while later blocks are
 * still being computed. block_done may be NULL (then this is wmma_ops_w4a16_gemm_ex). */
int wmma_ops_w4a16_gemm_blocks(const void* A, const void* qweight, const void* scales, void* C, int M, int N,
                               int K, int group_size, int split_k, int out_mode, float alpha, float in_scale,
                               void* workspace, size_t workspace_bytes, int* block_done, int* status,
                               void* stream);
int wmma_ops_w4a16_token_block(int M);

/* Sum of an fp16 buffer over the ranks of one NVSwitch domain, in place, for the row-parallel
 * outputs of the sharded layer (no counterpart in the reference, which is single-GPU).
 * multicast_ptr is the NVLink multicast address of a buffer of n_halves fp16 values that every
 * rank holds in symmetric memory (torch.distributed._symmetric_memory gives both). The caller
 * makes sure, with a barrier across the ranks on `stream`, that every rank's values are written
 * before any rank calls this, and that every rank's call has finished before the sums are read.
 * Rank `rank` reduces the rank-th of `world` slices through the switch (multimem.ld_reduce, fp32
 * accumulation) and stores the result to all ranks (multimem.st). max_ctas <= 0: all SMs. */
int wmma_ops_multimem_allreduce_f16(void* multicast_ptr, size_t n_halves, int rank, int world, int max_ctas,
                                    void* stream);

/* The same sum as one self-contained launch: the rank barriers before and after the reduction are
 * made inside the kernel with flags in symmetric memory (no counterpart in the reference).
 *   mc_in / mc_out  multicast addresses of buffers every rank holds in symmetric memory. With
 *                   in_is_f32 = 0, mc_in holds n_values fp16 partial outputs and is summed in
 *                   place (mc_out == mc_in). With in_is_f32 = 1, mc_in holds n_values fp32
 *                   partials and the sums are written as fp16 to mc_out.
 *   flag_ptrs_dev   device array of `world` pointers, entry r being rank r's copy of a
 *                   zero-initialised symmetric buffer of wmma_ops_switch_allreduce_flag_bytes()
 *                   bytes that is used for nothing else.
 *   channel         0..3; calls that may be in flight at the same time need different channels.
 *   max_ctas        CTAs (of 192 threads) per rank (<= 0: 128); all ranks must pass the same value.
 * Every rank calls it with the same arguments on a stream on which its partial outputs have been
 * written; when the call has completed on a rank, that rank's copy of the output holds all sums.
 * A rank that does not arrive within about a second makes the others record {5, rank, block,
 * missing rank} in `status` and finish with an incomplete sum instead of hanging. */
size_t wmma_ops_switch_allreduce_flag_bytes(void);
int wmma_ops_switch_allreduce(const void* mc_in, void* mc_out, size_t n_values, int in_is_f32, int rank, int world,
                              const void* flag_ptrs_dev, int channel, int max_ctas, int* status, void* stream);

/* wmma_ops_switch_allreduce for a [rows, cols] buffer that a GEMM of this rank is still writing, on another
 * stream, token block by token block (wmma_ops_w4a16_gemm_blocks): each block of block_rows rows is summed
 * as soon as every rank's block_done[] entry for it has reached tiles_per_block, so the exchange runs beside
 * the GEMM and only the last block's sum remains after it.
 *   mc_in / mc_out  multicast addresses of the first of the `rows` rows (cols % 8 == 0), as above.
 *   block_done      the counters given to the GEMM; seen: as many zero-initialised ints of device memory.
 *                   Both are zero again when the call has completed.
 *   max_ctas        <= 0: 32. Up to eight CTAs share a token block when there are fewer blocks than CTAs.
 * Launch the GEMM first and leave it room to become resident: either as many SMs free as this call has
 * CTAs (wmma_ops_set_sm_margin), or a product with more than 128 rows, whose kernel leaves room for one
 * CTA of this one on every SM. A CTA whose GEMM does not finish a block within about a second records
 * {6, rank, CTA, token block} in `status` and carries on. */
int wmma_ops_switch_allreduce_following(const void* mc_in, void* mc_out, int rows, int cols, int in_is_f32,
                                        int block_rows, int* block_done, int* seen, int tiles_per_block, int rank,
                                        int world, const void* flag_ptrs_dev, int channel, int max_ctas, int* status,
                                        void* stream);

/* Flash-attention forward: O = softmax(scale * Q K^T [+ causal mask]) V per (b,h).
 * Q, K, V, O are [B,H,S,D] fp16 contiguous; the signature documented in the reference's
 * README.md:221-251 (its implementation is not in the reference tree).
 * scale < 0 means 1/sqrt(D). Requirements: D == 128 or D == 64, S >= 1. */
int wmma_ops_fmha_fwd(const void* Q, const void* K, const void* V, void* O, int B, int H, int S,
                      int D, float scale, int causal, int* status, void* stream);

/* The same for tensors that are not contiguous [B,H,S,D]: D is contiguous, and `strides` holds, in elements,
 * the distances between consecutive tokens, heads and sequences of Q, then K, V and O (12 values; multiples
 * of 8, token rows at least D apart). E.g. the Q section of a packed projection output [tokens, 3, H, D]
 * has strides {3 H D, D, S 3 H D}. Nothing is copied: the kernel's tensor maps are (D, token, head, sequence). */
int wmma_ops_fmha_fwd_strided(const void* Q, const void* K, const void* V, void* O, int B, int H, int S, int D,
                              const long long* strides, float scale, int causal, int* status, void* stream);

/* The same attention for decode shapes: Sq <= 16 query rows per (b,h) against Skv >= Sq keys and
 * values (Q, O [B,H,Sq,D]; K, V [B,H,Skv,D]; fp16, contiguous). With causal != 0 query row i sees
 * the keys 0 .. Skv - Sq + i. The key range is cut into splits over the SMs; with more than one
 * split the partial results go through `workspace` (wmma_ops_fmha_decode_workspace_bytes, any
 * contents) and are merged in split order by a second launch on the same stream. Extends the
 * signature of README.md:221-251 to a key/value cache; no counterpart in the reference tree. */
size_t wmma_ops_fmha_decode_workspace_bytes(int B, int H, int Sq, int Skv, int D);
int wmma_ops_fmha_decode(const void* Q, const void* K, const void* V, void* O, int B, int H, int Sq, int Skv, int D,
                         float scale, int causal, void* workspace, size_t workspace_bytes, int* status, void* stream);

/* On-disk container for prepacked INT4 weights (written and read by wmma_ops_b200/w4file.py; no
 * counterpart in the reference, which has no INT4 code). Little endian; every payload starts on a
 * 256-byte boundary, so a file mapped at a page boundary can be copied to the device block by
 * block. A file is: one header, n_entries entries, then the payloads.
 *   qweight payload  uint32 [K/64][ceil(N/128)][128][8], the device layout of wmma_ops_int4_prepack
 *   scales payload   fp16 [K/group_size][N]
 * A reader must refuse a version it does not know: the packed block layout is part of the version.
 * Checksums are CRC-32 (IEEE 802.3, as zlib computes it). */
#define WMMA_OPS_W4_FILE_MAGIC "W4B200\0\0"
#define WMMA_OPS_W4_FILE_VERSION 1u
typedef struct wmma_ops_w4_file_header {
    char magic[8];          /* WMMA_OPS_W4_FILE_MAGIC */
    uint32_t version;       /* WMMA_OPS_W4_FILE_VERSION */
    uint32_t header_bytes;  /* 64 */
    uint32_t entry_bytes;   /* 128 */
    uint32_t n_entries;
    uint32_t table_crc32;   /* of the n_entries entries that follow the header */
    uint8_t reserved[36];
} wmma_ops_w4_file_header;
typedef struct wmma_ops_w4_file_entry {
    char name[64];          /* UTF-8, zero padded */
    uint32_t K, N, group_size, zero_point; /* zero_point is 8 */
    uint64_t qweight_offset, qweight_bytes, scales_offset, scales_bytes; /* offsets from the start of the file */
    uint32_t qweight_crc32, scales_crc32;
    uint8_t reserved[8];
} wmma_ops_w4_file_entry;

/* Self-tests of the failure reporting (no counterpart in the reference, whose kernels have no
 * bounded waits). wmma_ops_selftest_wait_expiry launches one tiny kernel whose only wait is on a
 * barrier nobody arrives at; after limit_cycles SM cycles (1e3 .. 4e9) the wait gives up, the
 * kernel returns normally and status reads {7, 77, 0, detail}. wmma_ops_selftest_debug_index
 * evaluates the debug build's index check on `index` against a buffer of n ints: in range, the
 * kernel writes out[index] = 1; out of range, the store is skipped and, in the debug build only,
 * status reads {9, 104, 0, index}. wmma_ops_debug_checks_enabled returns 1 for the library built
 * with -DWMMA_OPS_DEBUG_CHECKS (device-side index checks that write the status word), else 0. */
int wmma_ops_selftest_wait_expiry(long long limit_cycles, int detail, int* status, void* stream);
int wmma_ops_selftest_debug_index(int index, int n, int* out, int* status, void* stream);
int wmma_ops_debug_checks_enabled(void);

#ifdef __cplusplus
}
#endif
#endif /* WMMA_OPS_B200_H */
