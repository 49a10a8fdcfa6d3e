// Host-side helpers shared by the C-ABI entry points: last-error string, status codes,
// tensor-map (TMA descriptor) encoding through the driver entry point, per-device facts.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <atomic>
#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "../../include/wmma_ops_b200.h"

namespace wb {

void set_error(const char* fmt, ...);  // stores a thread-local message for wmma_ops_last_error()

#define WB_CHECK_CUDA(expr)                                                               \
    do {                                                                                  \
        cudaError_t _e = (expr);                                                          \
        if (_e != cudaSuccess) {                                                          \
            wb::set_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), __FILE__, \
                          __LINE__);                                                      \
            return WMMA_OPS_ERR_CUDA;                                                     \
        }                                                                                 \
    } while (0)

#define WB_REQUIRE(cond, code, ...)  \
    do {                             \
        if (!(cond)) {               \
            wb::set_error(__VA_ARGS__); \
            return (code);           \
        }                            \
    } while (0)

// Number of SMs the persistent kernels may occupy on the current device: the device's SM count
// (cached per device index) minus the margin set with wmma_ops_set_sm_margin.
int sm_count();
extern std::atomic<int> g_sm_margin;  // process-wide switch, read once per launch

// Encodes a tiled tensor map. dims/strides are innermost first; strides[0] is implied
// (element size) and strides[i>0] are in bytes. Returns 0 or WMMA_OPS_ERR_*.
int encode_tmap(CUtensorMap* out, CUtensorMapDataType dtype, int rank, const void* base,
                const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box,
                CUtensorMapSwizzle swizzle,
                CUtensorMapL2promotion promo = CU_TENSOR_MAP_L2_PROMOTION_L2_256B);

inline int encode_tmap_2d(CUtensorMap* out, CUtensorMapDataType dtype, const void* base,
                          uint64_t inner, uint64_t outer, uint64_t row_stride_bytes,
                          uint32_t box_inner, uint32_t box_outer, CUtensorMapSwizzle swizzle) {
    uint64_t dims[2] = {inner, outer};
    uint64_t strides[2] = {0, row_stride_bytes};
    uint32_t box[2] = {box_inner, box_outer};
    return encode_tmap(out, dtype, 2, base, dims, strides, box, swizzle);
}

}  // namespace wb
