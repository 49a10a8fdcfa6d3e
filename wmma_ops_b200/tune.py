"""Tile-table tuner: measures every tile shape and split-K factor on a list of shapes, stores the
winners in a JSON cache, installs a cache into the library, and prints a shape report.

This takes the place of the reference's search that justifies its tile table (autotune.py:131-283:
per-shape search over matmul_tiled 0..3, a JSON cache :134-149, a generated select_tuned_tile :261)
and of its shape report (benchmark_summary.py:10-19), without Optuna: the space is four tiles times
a handful of split factors, so it is measured exhaustively with CUDA events.

    python -m wmma_ops_b200.tune --out tile_table.json        # measure TUNE_SHAPES, write the cache
    python -m wmma_ops_b200.tune --report [--table tile_table.json]
    WMMA_OPS_TILE_TABLE=tile_table.json python my_program.py  # matmul_adaptive / gemm_adaptive use it

A cache entry is keyed by (op, shape bucket, SM count): the bucket is (ceil(M/128), ceil(N/64),
ceil(K/64)), i.e. all shapes with the same grid of smallest tiles and the same number of k-blocks.
Shapes that are not in the installed table fall back to the library's built-in cost model.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import sys
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

import torch

from . import _lib

CACHE_VERSION = 1
ENV_VAR = "WMMA_OPS_TILE_TABLE"
TILE_NAMES = {_lib.TILE_128x64: "128x64", _lib.TILE_128x128: "128x128", _lib.TILE_128x256: "128x256",
              _lib.TILE_256x256_PAIR: "256x256 pair"}

# The shapes the reference tunes and reports on (autotune.py:64-82, benchmark_summary.py:10-19) and the
# shapes of this repository's benchmark configurations (squares up to 8192, 4096x4096x2048, the
# split-K shape 256x256x16384).
REFERENCE_TUNE_SHAPES = [(256, 256, 256), (512, 512, 512), (768, 768, 768), (1024, 1024, 1024), (2048, 2048, 512),
                         (2048, 2048, 1024), (2048, 2048, 2048), (4096, 4096, 1024), (4096, 4096, 2048),
                         (4096, 4096, 4096), (8192, 1024, 2048), (1024, 8192, 2048), (4096, 11008, 4096)]
REFERENCE_REPORT_SHAPES = [(256, 256, 256), (512, 512, 512), (768, 768, 768), (1024, 1024, 1024), (1536, 1536, 1536),
                           (2048, 2048, 2048), (4096, 4096, 4096), (4096, 11008, 4096)]
CONFIG_SHAPES = [(8192, 8192, 8192), (256, 256, 16384)]


def _unique(shapes: Iterable[Tuple[int, int, int]]) -> List[Tuple[int, int, int]]:
    out, seen = [], set()
    for s in shapes:
        if s not in seen:
            seen.add(s)
            out.append(s)
    return out


TUNE_SHAPES = _unique(REFERENCE_TUNE_SHAPES + REFERENCE_REPORT_SHAPES + CONFIG_SHAPES)


# ----------------------------------------------------------------------------- keys and cache files
def shape_bucket(M: int, N: int, K: int) -> Tuple[int, int, int]:
    return (-(-M // 128), -(-N // 64), -(-K // 64))


def cache_key(op: str, M: int, N: int, K: int, sms: int) -> str:
    mb, nb, kb = shape_bucket(M, N, K)
    return f"{op}:{mb}x{nb}x{kb}:sm{sms}"


def candidates(M: int, N: int, K: int) -> List[Tuple[int, int]]:
    """(tile_cfg, split_k) pairs worth measuring: every tile without a split, the 1-CTA tiles with
    power-of-two splits that keep at least 256 of K per slice (the limit the built-in plan keeps, as
    the reference's plan does: wmma_xor_swizzle.hpp:311-317), and no split for the CTA-pair tile."""
    kb = -(-K // 64)
    out = [(t, 1) for t in (_lib.TILE_128x64, _lib.TILE_128x128, _lib.TILE_128x256)]
    if M > 128 and N > 128:
        out.append((_lib.TILE_256x256_PAIR, 1))
    for tile in (_lib.TILE_128x64, _lib.TILE_128x128, _lib.TILE_128x256):
        tiles = -(-M // 128) * -(-N // {0: 64, 1: 128, 2: 256}[tile])
        s = 2
        while s <= 32 and kb // s >= 4 and tiles * s <= 4 * 148:
            out.append((tile, s))
            s *= 2
    return out


def new_table(device_name: str, sms: int) -> dict:
    return {"version": CACHE_VERSION, "device": device_name, "sms": sms, "entries": {}}


def save_table(path, table: dict) -> None:
    tmp = f"{os.fspath(path)}.tmp{os.getpid()}"
    with open(tmp, "w") as f:
        json.dump(table, f, indent=1, sort_keys=True)
    os.replace(tmp, path)


def load_table(path) -> dict:
    with open(path) as f:
        table = json.load(f)
    if not isinstance(table, dict) or table.get("version") != CACHE_VERSION or not isinstance(table.get("entries"), dict):
        raise RuntimeError(f"{path}: not a tile table of version {CACHE_VERSION}")
    for key, e in table["entries"].items():
        for field in ("M", "N", "K", "sms", "tile", "split_k"):
            if not isinstance(e.get(field), int):
                raise RuntimeError(f"{path}: entry {key} lacks the integer field {field}")
    return table


_env_done = False


def install_table(table: Optional[dict]) -> int:
    """Hands the table's GEMM entries to the library (None or an empty table removes the installed
    one). Returns the number of rows installed. Needs no GPU."""
    global _env_done
    _env_done = True   # an explicit installation is not replaced by the automatic one later
    lib = _lib.load()
    rows: List[int] = []
    if table:
        for key, e in sorted(table["entries"].items()):
            if key.startswith("gemm:"):
                rows += [e["M"], e["N"], e["K"], e["sms"], e["tile"], e["split_k"]]
    arr = (ctypes.c_int * max(1, len(rows)))(*rows)
    _lib.check(lib.wmma_ops_set_tile_table(arr, len(rows) // 6))
    return len(rows) // 6


DEFAULT_TABLE = os.path.join(os.path.dirname(os.path.abspath(__file__)), "tile_table_b200.json")


def install_from_env(force: bool = False) -> Optional[str]:
    """Installs the table named by WMMA_OPS_TILE_TABLE, once per process; when the variable is
    unset, the table measured on B200 that ships with the package (its rows only match devices with
    the SM count they were measured on); "none" installs nothing. Called by the host layer before
    its first adaptive launch. Returns the path used, or None."""
    if _env_done and not force:
        return None
    path = os.environ.get(ENV_VAR, "")
    if path.lower() == "none":
        install_table(None)
        return None
    if not path:
        if not os.path.exists(DEFAULT_TABLE):
            return None
        path = DEFAULT_TABLE
    install_table(load_table(path))
    return path


# ----------------------------------------------------------------------------- measurement
def _time_us(fn, iters: int, warmup: int = 3) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    best = float("inf")
    for _ in range(3):
        e0 = torch.cuda.Event(enable_timing=True)
        e1 = torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1) * 1e3 / iters)
    return best


def _operands(M: int, N: int, K: int, device, sets: int):
    g = torch.Generator(device=device).manual_seed(M * 7 + N * 3 + K)
    return [((torch.randn(M, K, generator=g, device=device) * K ** -0.5).half(),
             torch.randn(K, N, generator=g, device=device).half()) for _ in range(sets)]


def measure_shape(M: int, N: int, K: int, device=None, iters: Optional[int] = None) -> Dict[str, float]:
    """Microseconds per product for every candidate of one shape, launched through the C ABI with a
    preallocated output (so the host path is the same for all candidates). Operand sets are rotated
    so that products smaller than the L2 do not run entirely out of it."""
    from .ops import _launch_gemm
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    bytes_per = 2 * (M * K + K * N) + 4 * M * N
    sets = max(1, min(8, int(256e6 // bytes_per)))
    ops_ = _operands(M, N, K, device, sets)
    outs = [torch.empty((M, N), dtype=torch.float32, device=device) for _ in range(sets)]
    flops = 2.0 * M * N * K
    if iters is None:
        iters = int(max(4, min(200, 2e11 // flops)))
    res = {}
    for tile, split in candidates(M, N, K):
        state = {"i": 0}

        def fn(tile=tile, split=split):
            i = state["i"] % sets
            state["i"] += 1
            A, B = ops_[i]
            _launch_gemm(A, B, None, outs[i], M, N, K, 1.0, 0.0, tile, split)

        res[f"{tile}:{split}"] = _time_us(fn, iters)
    return res


def tune(shapes: Sequence[Tuple[int, int, int]] = tuple(TUNE_SHAPES), device=None, table: Optional[dict] = None,
         verbose: bool = True) -> dict:
    """Measures `shapes`, records the fastest (tile, split_k) of each in `table` (a new one if None)
    and returns it. Entries already present for a bucket are overwritten."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    props = torch.cuda.get_device_properties(device)
    if table is None:
        table = new_table(props.name, props.multi_processor_count)
    for (M, N, K) in shapes:
        res = measure_shape(M, N, K, device)
        best = min(res, key=res.get)
        tile, split = (int(v) for v in best.split(":"))
        table["entries"][cache_key("gemm", M, N, K, props.multi_processor_count)] = {
            "M": M, "N": N, "K": K, "sms": props.multi_processor_count, "tile": tile, "split_k": split,
            "us": round(res[best], 3), "tflops": round(2.0 * M * N * K / res[best] / 1e6, 1),
            "all_us": {k: round(v, 3) for k, v in sorted(res.items())}}
        if verbose:
            print(f"{M:6d} x {N:6d} x {K:6d}: {TILE_NAMES[tile]:>13s} split {split:2d}  {res[best]:9.2f} us  "
                  f"{2.0 * M * N * K / res[best] / 1e6:7.1f} TFLOP/s", flush=True)
    return table


def report(shapes: Sequence[Tuple[int, int, int]] = tuple(_unique(REFERENCE_REPORT_SHAPES + REFERENCE_TUNE_SHAPES + CONFIG_SHAPES)),
           device=None, peak_tflops: Optional[float] = None) -> List[dict]:
    """The shape report: per shape the TFLOP/s of matmul_adaptive, of the best fixed candidate, their
    ratio, and torch's fp16 matmul (cuBLAS) on the same operands for context."""
    from . import ops
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    rows = []
    print(f"{'shape':>22s}  {'adaptive':>9s}  {'choice':>20s}  {'best fixed':>10s}  {'adaptive/best':>13s}  {'torch fp16':>10s}")
    for (M, N, K) in shapes:
        res = measure_shape(M, N, K, device)
        best = min(res, key=res.get)
        A, B = _operands(M, N, K, device, 1)[0]
        flops = 2.0 * M * N * K
        iters = int(max(4, min(200, 2e11 // flops)))
        t_ad = _time_us(lambda: ops.matmul_adaptive(A, B), iters)
        t_lib = _time_us(lambda: torch.matmul(A, B), iters)
        tile, split = ops.select_tile(M, N, K, torch.cuda.get_device_properties(device).multi_processor_count)
        row = {"M": M, "N": N, "K": K, "adaptive_tflops": flops / t_ad / 1e6, "adaptive_choice": [tile, split],
               "best_fixed": best, "best_fixed_tflops": flops / res[best] / 1e6, "adaptive_over_best": res[best] / t_ad,
               "torch_fp16_tflops": flops / t_lib / 1e6}
        if peak_tflops:
            row["adaptive_frac_of_peak"] = row["adaptive_tflops"] / peak_tflops
        rows.append(row)
        print(f"{M:6d}x{N:6d}x{K:6d}  {row['adaptive_tflops']:9.1f}  {TILE_NAMES[tile] + ' /' + str(split):>20s}  "
              f"{row['best_fixed_tflops']:10.1f}  {row['adaptive_over_best']:13.3f}  {row['torch_fp16_tflops']:10.1f}", flush=True)
    return rows


def main(argv: Optional[Sequence[str]] = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--out", help="write the measured table to this JSON file")
    ap.add_argument("--table", help="install this table before --report (default: $WMMA_OPS_TILE_TABLE)")
    ap.add_argument("--report", action="store_true", help="print the shape report")
    ap.add_argument("--json", help="also write the report rows to this file")
    args = ap.parse_args(argv)
    if not torch.cuda.is_available():
        print("the tuner measures on a GPU; none is visible", file=sys.stderr)
        return 2
    if args.out:
        table = tune()
        save_table(args.out, table)
        print(f"wrote {len(table['entries'])} entries to {args.out}")
        install_table(table)
    elif args.table:
        install_table(load_table(args.table))
    else:
        install_from_env(force=True)
    if args.report:
        rows = report()
        if args.json:
            with open(args.json, "w") as f:
                json.dump(rows, f, indent=1)
    return 0


if __name__ == "__main__":
    sys.exit(main())
