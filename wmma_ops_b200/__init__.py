"""wmma_ops_b200 — the GEMM hot path of wmma_ops, written for B200 (sm_100a).

Same function names and argument meaning as the reference's extension module
(wmma_gemm.hip:2120-2156) plus the flash-attention signature its README documents
(README.md:221-251) and the INT4 prepack / W4A16 pair. Every function runs hand-written
CUDA through libwmma_ops_b200.so; there is no CPU or library fallback.
"""
from . import _lib
from .ops import (  # noqa: F401
    check_status,
    reset_workspaces,
    gemm,
    gemm_adaptive,
    gemm_inplace,
    matmul,
    matmul_adaptive,
    matmul_asmOpt,
    matmul_coop,
    matmul_highOcc,
    matmul_hilbert,
    matmul_kunroll,
    matmul_native,
    matmul_noPrefetch,
    matmul_opt,
    matmul_pingpong,
    matmul_quad,
    matmul_host,
    matmul_splitk,
    matmul_swizzled,
    matmul_tiled,
    matmul_xor_optimized,
    matmul_zerocopy,
    select_tile,
    set_sm_margin,
)

from .attention import flash_attention  # noqa: F401,E402
from .quant import (int4_dequant, int4_prepack, int4_unpack, interleave_gate_up, matmul_w4a16,  # noqa: F401,E402
                    set_w4a16_overlap, w4a16_token_block)

from .w4file import load_w4, read_w4_index, save_w4  # noqa: F401,E402

__version__ = "0.2.0"
