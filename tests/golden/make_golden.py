"""Generates the fixtures in this directory. Run from the repository root in a container that
has the reference tree (needed only for tile_selection.json):

    make -C oracle && python tests/golden/make_golden.py

tile_selection.json  outputs of the reference's own select_optimal_tile, produced by running the
                     reference header compiled by oracle/Makefile (oracle/_ref/tile_select).
gemm_golden.npz      the reference's closed-form known-answer case (test_fragment_loading.py:225-274)
                     and small seeded cases whose outputs come from the reference's oracle
                     computation (torch fp32 matmul on the host).
int4_golden.npz      a small code matrix with its packed words and dequantised weights under the
                     W4-B200-v1 format (the repository's own specification; parity unpinned).
attention_golden.npz a small fp32 softmax-attention case (parity unpinned).
"""
import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
from oracle import attention, gemm, int4  # noqa: E402

HERE = Path(__file__).resolve().parent

TILE_SHAPES = [
    (512, 512, 512), (1024, 1024, 1024), (2048, 2048, 2048), (4096, 4096, 4096), (8192, 8192, 8192),
    (4096, 4096, 2048), (256, 256, 16384), (256, 256, 256), (8192, 1024, 2048), (4096, 11008, 4096),
    (1, 11008, 4096), (16, 11008, 4096), (128, 11008, 4096), (8192, 12288, 4096), (8192, 4096, 4096),
    (8192, 22016, 4096), (8192, 4096, 11008), (768, 768, 512), (1536, 1536, 511), (1537, 64, 4096),
    (511, 511, 64), (16385, 4096, 64), (2048, 8192, 64), (2047, 8192, 64),
]


def tile_selection():
    exe = ROOT / "oracle" / "_ref" / "tile_select"
    if not exe.exists():
        raise SystemExit("oracle/_ref/tile_select missing: run `make -C oracle` where the reference tree is mounted")
    inp = "".join(f"{m} {n} {k}\n" for m, n, k in TILE_SHAPES)
    out = subprocess.run([str(exe)], input=inp, capture_output=True, text=True, check=True).stdout
    rows = [list(map(int, line.split())) for line in out.strip().splitlines()]
    (HERE / "tile_selection.json").write_text(json.dumps(
        {"source": "reference wmma_tile_selection.hpp:30-66 compiled with g++ -D__host__=", "rows": rows}, indent=1))


def gemm_cases():
    A, B, C = gemm.known_answer_case()
    data = {"ka_A": A.numpy(), "ka_B": B.numpy(), "ka_C": C.numpy()}
    for i, (M, N, K) in enumerate([(64, 96, 80), (130, 72, 200), (1, 8, 8)]):
        a, b = gemm.seeded_ab(M, N, K, seed=42 + i)
        c_in = gemm.seeded_c(M, N, seed=142 + i)
        data[f"s{i}_A"] = a.numpy()
        data[f"s{i}_B"] = b.numpy()
        data[f"s{i}_Cin"] = c_in.numpy()
        data[f"s{i}_C"] = gemm.gemm_ref(a, b).numpy()
        data[f"s{i}_C_a2b05"] = gemm.gemm_alphabeta_ref(a, b, 2.0, 0.5, c_in).numpy()
    np.savez_compressed(HERE / "gemm_golden.npz", **data)


def int4_cases():
    codes, scales = int4.seeded_w4(128, 136, 64, seed=5)
    q = int4.pack_ref(codes)
    w = int4.dequant_ref(codes, scales, 64)
    np.savez_compressed(HERE / "int4_golden.npz", codes=codes.numpy(), scales=scales.numpy(),
                        qweight=q.numpy(), W=w.numpy(), group=np.int32(64))


def attention_cases():
    Q, K, V = attention.seeded_qkv(1, 2, 80, 64, seed=3)
    np.savez_compressed(
        HERE / "attention_golden.npz", Q=Q.numpy(), K=K.numpy(), V=V.numpy(),
        O=attention.attention_ref(Q, K, V, False).numpy(),
        O_causal=attention.attention_ref(Q, K, V, True).numpy())


if __name__ == "__main__":
    tile_selection()
    gemm_cases()
    int4_cases()
    attention_cases()
    print("golden fixtures written to", HERE)
