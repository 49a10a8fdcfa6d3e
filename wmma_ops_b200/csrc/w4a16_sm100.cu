// placeholder until the fused kernel lands
#include "host_common.cuh"
extern "C" int wmma_ops_int4_prepack(const void*, void*, int, int, void*) { wb::set_error("not built"); return WMMA_OPS_ERR_UNSUPPORTED; }
extern "C" int wmma_ops_int4_unpack(const void*, void*, int, int, void*) { wb::set_error("not built"); return WMMA_OPS_ERR_UNSUPPORTED; }
extern "C" int wmma_ops_int4_dequant(const void*, const void*, void*, int, int, int, void*) { wb::set_error("not built"); return WMMA_OPS_ERR_UNSUPPORTED; }
extern "C" size_t wmma_ops_w4a16_workspace_bytes(int, int, int, int) { return 0; }
extern "C" int wmma_ops_w4a16_select_split(int, int, int, int) { return 1; }
extern "C" int wmma_ops_w4a16_gemm(const void*, const void*, const void*, void*, int, int, int, int, int, void*, size_t, int*, void*) { wb::set_error("not built"); return WMMA_OPS_ERR_UNSUPPORTED; }
