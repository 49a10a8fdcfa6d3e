"""The C-ABI library without a GPU: it loads, exports what include/*.h declares, and its
host-only entry points (tile table, workspace sizes, argument checks) behave."""
import ctypes
import re
from pathlib import Path

import pytest

from wmma_ops_b200 import _lib

ROOT = Path(__file__).resolve().parents[1]


def _declared_functions():
    names = []
    for hdr in sorted((ROOT / "include").glob("*.h")):
        text = re.sub(r"/\*.*?\*/", "", hdr.read_text(), flags=re.S)
        names += re.findall(r"\b(wmma_ops_[a-z0-9_]+)\s*\(", text)
    return sorted(set(names))


def test_every_declared_symbol_is_exported_and_bound(lib):
    declared = _declared_functions()
    assert len(declared) >= 10
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in include/ but not exported"
        assert name in _lib.SIGNATURES, f"{name} has no ctypes signature"
    assert sorted(_lib.SIGNATURES) == declared


def test_version_and_error_string(lib):
    assert lib.wmma_ops_version() >= 100
    assert isinstance(_lib.last_error(), str)


@pytest.mark.parametrize("shape", [(8192, 8192, 8192), (512, 512, 512), (256, 256, 16384), (1, 11008, 4096),
                                   (4096, 4096, 2048), (130, 72, 200), (1, 8, 8)])
def test_select_tile_invariants(lib, shape):
    M, N, K = shape
    cfg, sk = ctypes.c_int(-5), ctypes.c_int(-5)
    assert lib.wmma_ops_select_tile(M, N, K, 148, ctypes.byref(cfg), ctypes.byref(sk)) == 0
    assert cfg.value in (_lib.TILE_128x64, _lib.TILE_128x128, _lib.TILE_128x256, _lib.TILE_256x256_PAIR)
    kb = -(-K // 64)
    assert 1 <= sk.value <= 32
    if sk.value > 1:
        # the limits the reference's plan also keeps (wmma_xor_swizzle.hpp:311-317):
        # at most 32 slices, at least 256 of K per slice, no empty slice
        per = -(-kb // sk.value)
        assert per >= 4 and per * (sk.value - 1) < kb


def test_select_tile_expected_choices(lib):
    def sel(M, N, K, sms=148):
        cfg, sk = ctypes.c_int(), ctypes.c_int()
        assert lib.wmma_ops_select_tile(M, N, K, sms, ctypes.byref(cfg), ctypes.byref(sk)) == 0
        return cfg.value, sk.value
    assert sel(8192, 8192, 8192)[1] == 1 and sel(8192, 8192, 8192)[0] in (_lib.TILE_128x256, _lib.TILE_256x256_PAIR)
    assert sel(256, 256, 16384)[1] > 1          # the split-K shape is split
    assert sel(4096, 4096, 4096)[1] == 1
    assert sel(64, 64, 64) == (sel(64, 64, 64)[0], 1)  # K too short to split


def test_select_tile_rejects_bad_arguments(lib):
    cfg, sk = ctypes.c_int(), ctypes.c_int()
    assert lib.wmma_ops_select_tile(0, 8, 8, 148, ctypes.byref(cfg), ctypes.byref(sk)) == _lib.ERR_INVALID
    assert "positive" in _lib.last_error()
    assert lib.wmma_ops_select_tile(8, 8, 8, 148, None, None) == _lib.ERR_INVALID


def test_workspace_bytes(lib):
    assert lib.wmma_ops_gemm_workspace_bytes(256, 256, 16384, 1) == 0
    assert lib.wmma_ops_gemm_workspace_bytes(256, 256, 16384, 32) == 32 * 256 * 256 * 4
    assert lib.wmma_ops_gemm_workspace_bytes(8192, 8192, 8192, 2) == 2 * 8192 * 8192 * 4  # > 2^31: size_t


def test_gemm_argument_checks_need_no_gpu(lib):
    # these are rejected before any CUDA call
    rc = lib.wmma_ops_gemm_f16f32(None, None, None, 16, 8, 12, 8, 1.0, 0.0, 0, 1, None, 0, None, None)
    assert rc == _lib.ERR_INVALID and "N must be a multiple of 8" in _lib.last_error()
    rc = lib.wmma_ops_gemm_f16f32(None, None, None, 16, 8, 8, 4, 1.0, 0.0, 0, 1, None, 0, None, None)
    assert rc == _lib.ERR_INVALID and "K must be a multiple of 8" in _lib.last_error()
    rc = lib.wmma_ops_gemm_f16f32(None, None, None, None, 8, 8, 8, 1.0, 0.0, 0, 1, None, 0, None, None)
    assert rc == _lib.ERR_INVALID and "C_out" in _lib.last_error()
    rc = lib.wmma_ops_gemm_f16f32(None, None, None, 24, 8, 8, 8, 1.0, 0.0, 0, 1, None, 0, None, None)
    assert rc == _lib.ERR_INVALID and "16-byte aligned" in _lib.last_error()
    # empty output: nothing to do, no launch
    assert lib.wmma_ops_gemm_f16f32(None, None, None, None, 0, 8, 8, 1.0, 0.0, 0, 1, None, 0, None, None) == 0


def test_w4a16_workspace_plan_of_the_streaming_decode_kernel():
    # Pure host arithmetic (148 SMs assumed without a GPU): products with up to 16 rows and no explicit
    # split get 64 KB of arrival counters plus, per 128-column tile, one 16 x 128 fp32 part for every
    # CTA that can share the tile: ceil(k_blocks / shortest_run) + 1, shortest_run = blocks // CTAs.
    lib = _lib.load()

    def expect(N, K, sms=148):
        n_tiles, kbt = -(-N // 128), K // 64
        blocks = n_tiles * kbt
        grid = min(sms, blocks)
        per = blocks // grid
        max_slices = -(-kbt // per) + 1
        return 65536 + n_tiles * max_slices * 16 * 128 * 4

    for (M, N, K) in [(1, 11008, 4096), (16, 11008, 4096), (16, 128, 64), (4, 4096, 11008), (8, 136, 512)]:
        assert lib.wmma_ops_w4a16_workspace_bytes(M, N, K, 0) == expect(N, K)
    # more rows, or an explicit split of 1: the tcgen05 kernel without partial sums
    assert lib.wmma_ops_w4a16_workspace_bytes(17, 11008, 4096, 0) == 0
    assert lib.wmma_ops_w4a16_workspace_bytes(16, 11008, 4096, 1) == 0
    # the overlap switch is a plain setter
    assert lib.wmma_ops_set_w4a16_overlap(1) == 0 and lib.wmma_ops_set_w4a16_overlap(0) == 0
