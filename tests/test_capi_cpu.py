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


def _decode_plan(lib, M, N, K, mode=0, sms=148, group=128):
    out = (ctypes.c_int * 14)()
    assert lib.wmma_ops_w4a16_decode_plan(M, N, K, group, mode, sms, out) == 0, _lib.last_error()
    keys = ("grid", "clusters", "ksplit", "units", "gpu", "upc", "depth", "slot_bytes", "pitch", "smem_bytes", "ncg", "alias_red",
            "seg_kb", "x_pitch")
    return dict(zip(keys, list(out)))


def _group_col(gu, v0, j):
    # column of group j of a chunk that starts at unit v0 (the kernel's sc_group_col)
    if not gu:
        return (v0 + j) * 16
    v = v0 + j // 2
    return (v // 4) * 128 + (v % 4) * 16 + (j % 2) * 64


@pytest.mark.parametrize("case", [
    (1, 11008, 4096, 0), (16, 11008, 4096, 0), (8, 4096, 11008, 0), (16, 4096, 4096, 0), (3, 22016, 4096, 0),
    (16, 128, 64, 0), (2, 8, 64, 0), (5, 136, 512, 0), (16, 11008, 11008, 0), (8, 256, 16384, 0), (16, 40000, 64, 0), (9, 1000, 2048, 0), (1, 12288, 4096, 0),
    (8, 1280, 1024, 2), (16, 1280, 1024, 2), (1, 22016, 4096, 2), (12, 2816, 4096, 2),
])
def test_w4a16_decode_plan_covers_every_block_once(lib, case):
    # Host arithmetic of the decode kernel, walked the way the kernel walks it: every (k-block,
    # 16-column group) of the packed matrix is read by exactly one warp of one CTA, ring slots are
    # reused only after they were consumed, and the plan fits in shared memory.
    M, N, K, mode = case
    group = 128 if K % 128 == 0 else 64
    pl = _decode_plan(lib, M, N, K, mode, group=group)
    gu = mode == 2
    kbt = K // 64
    ncg_max = pl["ncg"]
    assert ncg_max == 6 if M > 8 else ncg_max in (5, 8)
    assert pl["gpu"] == (2 if gu else 1)
    assert pl["units"] == (N // 32 if gu else -(-N // 16))
    assert pl["grid"] == pl["clusters"] * pl["ksplit"] and pl["grid"] <= 148
    assert pl["ksplit"] in (1, 2, 4) and pl["upc"] * pl["gpu"] <= ncg_max
    groups = pl["upc"] * pl["gpu"]
    assert pl["slot_bytes"] == groups * 512 and pl["depth"] >= 1
    # activations and scales are staged one K segment at a time: whole rounds of the 16 warps and whole
    # scale groups, rows 16 bytes longer than their data
    assert pl["seg_kb"] % 16 == 0 and pl["seg_kb"] % (group // 64) == 0 and pl["x_pitch"] == pl["seg_kb"] * 128 + 16
    assert pl["pitch"] >= pl["upc"] * pl["gpu"] * 16 and pl["pitch"] % 32 in (4, 20)
    assert pl["smem_bytes"] <= 227 * 1024
    ring, tiles = 16 * pl["depth"] * pl["slot_bytes"], 16 * M * pl["pitch"] * 4
    staged = M * pl["x_pitch"] + -(-pl["seg_kb"] // (group // 64)) * groups * 32
    assert (max(ring, tiles) if pl["alias_red"] else ring + tiles) + staged + M * pl["pitch"] * 4 <= pl["smem_bytes"]
    # a whole block of groups is read past a chunk's last group: it must stay inside the allocation
    assert 16 * pl["depth"] * pl["slot_bytes"] - pl["slot_bytes"] + ncg_max * 512 <= pl["smem_bytes"]
    seen = {}
    n_groups_total = -(-N // 16)
    for cluster in range(pl["clusters"]):
        u0 = cluster * pl["units"] // pl["clusters"]
        u1 = (cluster + 1) * pl["units"] // pl["clusters"]
        assert u1 > u0
        n_chunks = -(-(u1 - u0) // pl["upc"])
        for rank in range(pl["ksplit"]):
            k0 = rank * kbt // pl["ksplit"]
            k1 = (rank + 1) * kbt // pl["ksplit"]
            for warp in range(16):
                nkb = -(-(k1 - k0 - warp) // 16) if k1 - k0 > warp else 0
                for it in range(nkb * n_chunks):
                    ci = it // nkb
                    kb = k0 + warp + 16 * (it - ci * nkb)
                    assert k0 <= kb < k1
                    v0 = u0 + ci * pl["upc"]
                    nun = min(u1 - v0, pl["upc"])
                    assert nun >= 1
                    for j in range(nun * pl["gpu"]):
                        col = _group_col(gu, v0, j)
                        assert col % 16 == 0 and col // 16 < -(-N // 128) * 8
                        key = (kb, col // 16)
                        assert key not in seen, key
                        seen[key] = True
    assert len(seen) == kbt * n_groups_total


def test_w4a16_decode_plan_choices(lib):
    # 11008 columns: 688 groups on 148 CTAs, whole K per CTA, everything requested at once
    pl = _decode_plan(lib, 1, 11008, 4096)
    assert (pl["ksplit"], pl["clusters"], pl["upc"], pl["depth"], pl["alias_red"], pl["seg_kb"]) == (1, 148, 5, 4, 0, 64)
    # 16 rows: all of X (128 KB) beside the ring would leave one slot per warp, so K is staged in two halves
    pl = _decode_plan(lib, 16, 11008, 4096)
    assert pl["depth"] >= 2 and pl["alias_red"] == 1
    # a long K with 16 rows does not fit at once: it is staged in segments
    pl = _decode_plan(lib, 16, 11008, 11008)
    assert pl["seg_kb"] < 172 and pl["depth"] >= 2
    # 4096 columns: 256 groups would leave 148 CTAs with 1 or 2 each; clusters of 4 split K instead
    pl = _decode_plan(lib, 4, 4096, 11008)
    assert pl["ksplit"] == 4 and pl["clusters"] == 37 and pl["upc"] == 7
    # the decode kernel needs no workspace; more rows or an explicit split use the tcgen05 kernel
    assert lib.wmma_ops_w4a16_workspace_bytes(16, 11008, 4096, 0) == 0
    assert lib.wmma_ops_w4a16_workspace_bytes(17, 11008, 4096, 0) == 0
    assert lib.wmma_ops_w4a16_workspace_bytes(16, 11008, 4096, 4) > 0
    out = (ctypes.c_int * 14)()
    assert lib.wmma_ops_w4a16_decode_plan(17, 128, 64, 64, 0, 148, out) == _lib.ERR_INVALID
    assert lib.wmma_ops_w4a16_decode_plan(4, 192, 64, 64, 2, 148, out) == _lib.ERR_INVALID
    assert lib.wmma_ops_w4a16_decode_plan(4, 128, 256, 96, 0, 148, out) == _lib.ERR_INVALID
    # plain setters
    assert lib.wmma_ops_set_w4a16_overlap(1) == 0 and lib.wmma_ops_set_w4a16_overlap(0) == 0


def test_reset_hooks_follow_reset_workspaces():
    """Objects that own device-side counters (the switch all-reduce) register for reset_workspaces: the call
    reaches the objects of that device while they live, and no others."""
    import torch
    from wmma_ops_b200 import ops

    class Owner:
        def __init__(self, device):
            self.device, self.resets = device, 0

        def reset(self):
            self.resets += 1

    a, b = Owner(torch.device("cuda", 0)), Owner(torch.device("cuda", 1))
    ops._register_reset(a)
    ops._register_reset(b)
    ops.reset_workspaces(torch.device("cuda", 0))
    assert (a.resets, b.resets) == (1, 0)
    ops.reset_workspaces("cuda:1")
    assert (a.resets, b.resets) == (1, 1)
    del a
    ops.reset_workspaces(torch.device("cuda", 0))   # a dead owner is dropped silently
    assert b.resets == 1
