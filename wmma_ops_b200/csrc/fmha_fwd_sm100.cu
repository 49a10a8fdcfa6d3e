// placeholder until the attention kernel lands
#include "host_common.cuh"
extern "C" int wmma_ops_fmha_fwd(const void*, const void*, const void*, void*, int, int, int, int, float, int, int*, void*) { wb::set_error("not built"); return WMMA_OPS_ERR_UNSUPPORTED; }
