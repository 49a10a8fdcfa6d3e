"""ctypes binding of libwmma_ops_b200.so (declared in include/wmma_ops_b200.h).

There is no fallback: if the library is missing or a call fails, a RuntimeError is raised.
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path

_PKG = Path(__file__).resolve().parent
LIB_PATH = _PKG / "libwmma_ops_b200.so"
# the same sources built with -DWMMA_OPS_DEBUG_CHECKS: device-side index checks that record a
# fault in the status word and skip the access (loaded when WMMA_OPS_DEBUG=1)
DEBUG_LIB_PATH = _PKG / "libwmma_ops_b200_debug.so"

OK = 0
ERR_INVALID = 1
ERR_CUDA = 2
ERR_UNSUPPORTED = 3
ERR_WORKSPACE = 4

TILE_AUTO = -1
TILE_128x64 = 0
TILE_128x128 = 1
TILE_128x256 = 2
TILE_256x256_PAIR = 3

_c_int = ctypes.c_int
_c_float = ctypes.c_float
_c_size_t = ctypes.c_size_t
_vp = ctypes.c_void_p

# name -> (restype, argtypes); one entry per function declared in include/wmma_ops_b200.h
SIGNATURES = {
    "wmma_ops_last_error": (ctypes.c_char_p, []),
    "wmma_ops_version": (_c_int, []),
    "wmma_ops_set_sm_margin": (_c_int, [_c_int]),
    "wmma_ops_select_tile": (_c_int, [_c_int, _c_int, _c_int, _c_int, ctypes.POINTER(_c_int), ctypes.POINTER(_c_int)]),
    "wmma_ops_set_tile_table": (_c_int, [ctypes.POINTER(_c_int), _c_int]),
    "wmma_ops_gemm_workspace_bytes": (_c_size_t, [_c_int, _c_int, _c_int, _c_int]),
    "wmma_ops_gemm_f16f32": (_c_int, [_vp, _vp, _vp, _vp, _c_int, _c_int, _c_int, _c_float, _c_float,
                                      _c_int, _c_int, _vp, _c_size_t, _vp, _vp]),
    "wmma_ops_gemm_static_scratch_bytes": (_c_size_t, []),
    "wmma_ops_gemm_f16f32_splitk_static": (_c_int, [_vp, _vp, _vp, _vp, _c_int, _c_int, _c_int, _c_float, _c_float,
                                                    _c_int, _c_int, _vp, _vp]),
    "wmma_ops_int4_prepack": (_c_int, [_vp, _vp, _c_int, _c_int, _vp]),
    "wmma_ops_int4_unpack": (_c_int, [_vp, _vp, _c_int, _c_int, _vp]),
    "wmma_ops_int4_dequant": (_c_int, [_vp, _vp, _vp, _c_int, _c_int, _c_int, _vp]),
    "wmma_ops_set_w4a16_overlap": (_c_int, [_c_int]),
    "wmma_ops_w4a16_decode_plan": (_c_int, [_c_int, _c_int, _c_int, _c_int, _c_int, _c_int, ctypes.POINTER(_c_int)]),
    "wmma_ops_w4a16_workspace_bytes": (_c_size_t, [_c_int, _c_int, _c_int, _c_int]),
    "wmma_ops_w4a16_select_split": (_c_int, [_c_int, _c_int, _c_int, _c_int]),
    "wmma_ops_w4a16_gemm": (_c_int, [_vp, _vp, _vp, _vp, _c_int, _c_int, _c_int, _c_int, _c_int, _vp,
                                     _c_size_t, _vp, _vp]),
    "wmma_ops_w4a16_gemm_ex": (_c_int, [_vp, _vp, _vp, _vp, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float,
                                        _c_float, _vp, _c_size_t, _vp, _vp]),
    "wmma_ops_w4a16_gemm_blocks": (_c_int, [_vp, _vp, _vp, _vp, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float,
                                            _c_float, _vp, _c_size_t, _vp, _vp, _vp]),
    "wmma_ops_w4a16_token_block": (_c_int, [_c_int]),
    "wmma_ops_fmha_fwd": (_c_int, [_vp, _vp, _vp, _vp, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int,
                                   _vp, _vp]),
    "wmma_ops_fmha_fwd_strided": (_c_int, [_vp, _vp, _vp, _vp, _c_int, _c_int, _c_int, _c_int, ctypes.POINTER(ctypes.c_longlong),
                                           _c_float, _c_int, _vp, _vp]),
    "wmma_ops_fmha_decode_workspace_bytes": (_c_size_t, [_c_int, _c_int, _c_int, _c_int, _c_int]),
    "wmma_ops_fmha_decode": (_c_int, [_vp, _vp, _vp, _vp, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int, _vp,
                                      _c_size_t, _vp, _vp]),
    "wmma_ops_multimem_allreduce_f16": (_c_int, [_vp, _c_size_t, _c_int, _c_int, _c_int, _vp]),
    "wmma_ops_switch_allreduce_flag_bytes": (_c_size_t, []),
    "wmma_ops_switch_allreduce": (_c_int, [_vp, _vp, _c_size_t, _c_int, _c_int, _c_int, _vp, _c_int, _c_int, _vp, _vp]),
    "wmma_ops_switch_allreduce_following": (_c_int, [_vp, _vp, _c_int, _c_int, _c_int, _c_int, _vp, _vp, _c_int, _c_int, _c_int,
                                                     _vp, _c_int, _c_int, _vp, _vp]),
    "wmma_ops_selftest_wait_expiry": (_c_int, [ctypes.c_longlong, _c_int, _vp, _vp]),
    "wmma_ops_selftest_debug_index": (_c_int, [_c_int, _c_int, _vp, _vp, _vp]),
    "wmma_ops_debug_checks_enabled": (_c_int, []),
}

_lib = None


def load() -> ctypes.CDLL:
    """Loads the library once; raises RuntimeError with build instructions if it is absent."""
    global _lib
    if _lib is not None:
        return _lib
    debug = os.environ.get("WMMA_OPS_DEBUG", "0") not in ("", "0")
    path = Path(os.environ.get("WMMA_OPS_B200_LIB", DEBUG_LIB_PATH if debug else LIB_PATH))
    if not path.exists():
        raise RuntimeError(
            f"{path} not found: the CUDA library is not built. Run `python -m wmma_ops_b200.csrc.build` "
            "(needs nvcc; there is no CPU fallback)."
        )
    lib = ctypes.CDLL(str(path))
    for name, (res, args) in SIGNATURES.items():
        try:
            fn = getattr(lib, name)
        except AttributeError as e:  # a stale build
            raise RuntimeError(f"{path} does not export {name}; rebuild it") from e
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def last_error() -> str:
    return load().wmma_ops_last_error().decode("utf-8", "replace")


def check(rc: int) -> None:
    """Turns a non-zero return code into RuntimeError carrying the library's message."""
    if rc != OK:
        raise RuntimeError(last_error() or f"wmma_ops_b200 call failed with code {rc}")
