"""The tile-table cache and its installation into the library, without a GPU: keys, candidate
lists, JSON round trip, lookup through wmma_ops_select_tile, the environment-variable route."""
import ctypes
import json
import os
import subprocess
import sys
from pathlib import Path

import pytest

from wmma_ops_b200 import _lib, tune

ROOT = Path(__file__).resolve().parents[1]


def _select(lib, M, N, K, sms=148):
    cfg, sk = ctypes.c_int(), ctypes.c_int()
    assert lib.wmma_ops_select_tile(M, N, K, sms, ctypes.byref(cfg), ctypes.byref(sk)) == 0
    return cfg.value, sk.value


def test_shape_lists_and_keys():
    assert len(tune.REFERENCE_TUNE_SHAPES) == 13 and len(tune.REFERENCE_REPORT_SHAPES) == 8
    assert (8192, 8192, 8192) in tune.TUNE_SHAPES and (256, 256, 16384) in tune.TUNE_SHAPES
    assert len(set(tune.TUNE_SHAPES)) == len(tune.TUNE_SHAPES)
    assert tune.shape_bucket(4096, 11008, 4096) == (32, 172, 64)
    assert tune.shape_bucket(4000, 11000, 4090) == (32, 172, 64)       # same grid of smallest tiles
    assert tune.cache_key("gemm", 256, 256, 16384, 148) == "gemm:2x4x256:sm148"


def test_candidates_respect_the_kernel_limits():
    for (M, N, K) in tune.TUNE_SHAPES + [(1, 8, 8), (130, 72, 200)]:
        cands = tune.candidates(M, N, K)
        assert len(set(cands)) == len(cands) and (_lib.TILE_128x128, 1) in cands
        for tile, split in cands:
            assert tile in tune.TILE_NAMES and split >= 1
            if tile == _lib.TILE_256x256_PAIR:
                assert split == 1 and M > 128 and N > 128
            if split > 1:
                assert (-(-K // 64)) // split >= 4 and split <= 32
    assert any(s == 32 for _, s in tune.candidates(256, 256, 16384))


def test_table_round_trip_install_and_lookup(lib, tmp_path):
    before = _select(lib, 2048, 2048, 512), _select(lib, 256, 256, 16384)
    table = tune.new_table("test device", 148)
    table["entries"][tune.cache_key("gemm", 2048, 2048, 512, 148)] = {
        "M": 2048, "N": 2048, "K": 512, "sms": 148, "tile": _lib.TILE_128x64, "split_k": 2, "us": 1.0}
    table["entries"][tune.cache_key("gemm", 256, 256, 16384, 148)] = {
        "M": 256, "N": 256, "K": 16384, "sms": 148, "tile": _lib.TILE_128x256, "split_k": 16, "us": 1.0}
    path = tmp_path / "table.json"
    tune.save_table(path, table)
    assert tune.load_table(path) == table
    try:
        assert tune.install_table(tune.load_table(path)) == 2
        assert _select(lib, 2048, 2048, 512) == (_lib.TILE_128x64, 2)
        assert _select(lib, 2000, 2040, 500) == (_lib.TILE_128x64, 2)          # same bucket
        assert _select(lib, 256, 256, 16384) == (_lib.TILE_128x256, 16)
        assert _select(lib, 2048, 2048, 512, sms=132) == _select(lib, 2048, 2048, 512, sms=132)  # other SM count: model
        assert _select(lib, 4096, 4096, 4096)[1] == 1                          # not in the table: cost model
    finally:
        assert tune.install_table(None) == 0
    assert (_select(lib, 2048, 2048, 512), _select(lib, 256, 256, 16384)) == before


def test_bad_tables_are_refused(lib, tmp_path):
    p = tmp_path / "bad.json"
    p.write_text(json.dumps({"version": 99, "entries": {}}))
    with pytest.raises(RuntimeError, match="not a tile table"):
        tune.load_table(p)
    p.write_text(json.dumps({"version": 1, "entries": {"gemm:1x1x1:sm148": {"M": 8, "N": 8}}}))
    with pytest.raises(RuntimeError, match="lacks the integer field"):
        tune.load_table(p)
    rows = (ctypes.c_int * 6)(256, 256, 256, 148, 7, 1)                        # no such tile
    assert lib.wmma_ops_set_tile_table(rows, 1) == _lib.ERR_INVALID
    rows = (ctypes.c_int * 6)(256, 256, 256, 148, _lib.TILE_256x256_PAIR, 2)   # the pair tile cannot split
    assert lib.wmma_ops_set_tile_table(rows, 1) == _lib.ERR_INVALID
    rows = (ctypes.c_int * 6)(256, 256, 256, 148, _lib.TILE_128x64, 9)         # more slices than k-blocks
    assert lib.wmma_ops_set_tile_table(rows, 1) == _lib.ERR_INVALID


def test_environment_variable_installs_the_table(tmp_path):
    table = tune.new_table("test device", 148)
    table["entries"][tune.cache_key("gemm", 768, 768, 768, 148)] = {
        "M": 768, "N": 768, "K": 768, "sms": 148, "tile": _lib.TILE_128x64, "split_k": 2, "us": 1.0}
    path = tmp_path / "env_table.json"
    tune.save_table(path, table)
    code = ("import sys; sys.path.insert(0, %r)\n"
            "import wmma_ops_b200 as w\n"
            "print('CHOICE', w.select_tile(768, 768, 768, 148))\n") % str(ROOT)
    res = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=300,
                         env={**os.environ, tune.ENV_VAR: str(path)})
    assert res.returncode == 0 and f"CHOICE ({_lib.TILE_128x64}, 2)" in res.stdout, res.stdout + res.stderr
    res = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=300,
                         env={**os.environ, tune.ENV_VAR: "none"})
    assert res.returncode == 0 and f"CHOICE ({_lib.TILE_128x64}, 2)" not in res.stdout, res.stdout + res.stderr
