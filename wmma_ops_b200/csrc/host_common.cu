// Host-side helpers shared by the C-ABI entry points (see host_common.cuh).
#include "host_common.cuh"

#include <cstring>
#include <mutex>

namespace wb {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

std::atomic<int> g_sm_margin{0};

int sm_count() {
    static int cached[64];
    static std::mutex mu;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    std::lock_guard<std::mutex> lock(mu);
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
            n = 148;
        cached[dev] = n;
    }
    // SMs left free for other kernels (collectives) that must run beside the persistent ones
    const int usable = cached[dev] - g_sm_margin.load(std::memory_order_relaxed);
    return usable > 8 ? usable : 8;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
                cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

int encode_tmap(CUtensorMap* out, CUtensorMapDataType dtype, int rank, const void* base,
                const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box,
                CUtensorMapSwizzle swizzle, CUtensorMapL2promotion promo) {
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) {
        set_error("cuTensorMapEncodeTiled is not available from this driver");
        return WMMA_OPS_ERR_CUDA;
    }
    cuuint64_t gdims[5];
    cuuint64_t gstrides[4];
    cuuint32_t gbox[5];
    cuuint32_t estr[5];
    for (int i = 0; i < rank; ++i) {
        gdims[i] = dims[i];
        gbox[i] = box[i];
        estr[i] = 1;
        if (i > 0) gstrides[i - 1] = strides_bytes[i];
    }
    CUresult r = fn(out, dtype, static_cast<cuuint32_t>(rank), const_cast<void*>(base), gdims,
                    gstrides, gbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, promo,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_error("cuTensorMapEncodeTiled failed with CUresult %d (rank %d, dims %llu x %llu, box %u x %u)",
                  static_cast<int>(r), rank, static_cast<unsigned long long>(dims[0]),
                  static_cast<unsigned long long>(rank > 1 ? dims[1] : 1), box[0],
                  rank > 1 ? box[1] : 1);
        return WMMA_OPS_ERR_CUDA;
    }
    return WMMA_OPS_OK;
}

}  // namespace wb

extern "C" const char* wmma_ops_last_error(void) { return wb::g_err; }

extern "C" int wmma_ops_version(void) { return 100; }

extern "C" int wmma_ops_set_sm_margin(int sms) {
    if (sms < 0 || sms > 64) {
        wb::set_error("sm margin must be in 0..64 (got %d)", sms);
        return WMMA_OPS_ERR_INVALID;
    }
    wb::g_sm_margin.store(sms, std::memory_order_relaxed);
    return WMMA_OPS_OK;
}
