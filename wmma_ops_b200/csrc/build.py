"""Builds libwmma_ops_b200.so (the C-ABI library) in-tree with nvcc for sm_100a.

Takes the place of the reference's setup.py (setup.py:6-36, hipcc for gfx1151). Run as
``python -m wmma_ops_b200.csrc.build`` or call :func:`build`. Only nvcc is needed; no GPU.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

CSRC = Path(__file__).resolve().parent
PKG = CSRC.parent
LIB_PATH = PKG / "libwmma_ops_b200.so"
DEBUG_LIB_PATH = PKG / "libwmma_ops_b200_debug.so"   # same sources with -DWMMA_OPS_DEBUG_CHECKS
OBJ_DIR = CSRC / "build"

SOURCES = [
    "host_common.cu",
    "gemm_sm100.cu",
    "w4a16_sm100.cu",
    "w4a16_decode_sm100.cu",
    "fmha_fwd_sm100.cu",
    "fmha_decode_sm100.cu",
    "allreduce_sm100.cu",
    "selftest_sm100.cu",
]

NVCC_FLAGS = [
    "-std=c++17",
    "-O3",
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-Xcompiler",
    "-fPIC",
    "--expt-relaxed-constexpr",
    "-Xptxas",
    "-v",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; cannot build libwmma_ops_b200.so")
    return exe


def _digest(path: Path, extra: str = "") -> str:
    h = hashlib.sha256()
    h.update((" ".join(NVCC_FLAGS) + extra).encode())
    h.update(path.read_bytes())
    for hdr in sorted(CSRC.glob("*.cuh")) + sorted((PKG.parent / "include").glob("*.h")):
        h.update(hdr.read_bytes())
    return h.hexdigest()


def _compile_one(src: str, verbose: bool, debug: bool = False) -> Path:
    path = CSRC / src
    tag = ".debug" if debug else ""
    extra = ["-DWMMA_OPS_DEBUG_CHECKS"] if debug else []
    obj = OBJ_DIR / (src + tag + ".o")
    stamp = OBJ_DIR / (src + tag + ".sha")
    dig = _digest(path, " ".join(extra))
    if obj.exists() and stamp.exists() and stamp.read_text() == dig:
        return obj
    cmd = [_nvcc(), *NVCC_FLAGS, *extra, "-c", str(path), "-o", str(obj)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    (OBJ_DIR / (src + tag + ".log")).write_text(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{res.stdout}\n{res.stderr}")
    if verbose:
        sys.stderr.write(res.stderr)
    stamp.write_text(dig)
    return obj


def _link(objs, out: Path, force: bool) -> None:
    newest = max(o.stat().st_mtime for o in objs)
    if force or not out.exists() or out.stat().st_mtime < newest:
        cmd = [_nvcc(), "-shared", "-o", str(out), *map(str, objs), "-cudart", "static"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")


def build(verbose: bool = False, force: bool = False, debug: bool = True) -> Path:
    """Compile every CUDA source for sm_100a and link the shared library (and, with debug=True,
    the variant with device-side index checks). Returns the path of the normal library."""
    OBJ_DIR.mkdir(exist_ok=True)
    if force:
        for f in OBJ_DIR.glob("*.sha"):
            f.unlink()
    sources = [s for s in SOURCES if (CSRC / s).exists()]
    jobs = [(s, False) for s in sources] + ([(s, True) for s in sources] if debug else [])
    with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
        objs = list(ex.map(lambda j: _compile_one(j[0], verbose, j[1]), jobs))
    _link(objs[:len(sources)], LIB_PATH, force)
    if debug:
        _link(objs[len(sources):], DEBUG_LIB_PATH, force)
    return LIB_PATH


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force="-f" in sys.argv))
