"""The oracle against the reference's golden vectors and the committed fixtures (CPU only)."""
import json
import os
import subprocess
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import attention, gemm, int4, tile_plan

ROOT = Path(__file__).resolve().parents[1]


def test_known_answer_closed_form(golden_dir):
    # test_fragment_loading.py:225-274: C[i,k] = (i % 16) * 120, max error <= 0.01
    A, B, C = gemm.known_answer_case()
    out = gemm.gemm_ref(A, B)
    assert (out - C).abs().max().item() == 0.0
    g = np.load(golden_dir / "gemm_golden.npz")
    assert np.array_equal(g["ka_C"], out.numpy())
    assert np.array_equal(g["ka_A"], A.numpy()) and np.array_equal(g["ka_B"], B.numpy())


def test_seeded_gemm_matches_fixture(golden_dir):
    g = np.load(golden_dir / "gemm_golden.npz")
    for i, (M, N, K) in enumerate([(64, 96, 80), (130, 72, 200), (1, 8, 8)]):
        a, b = gemm.seeded_ab(M, N, K, seed=42 + i)
        assert np.array_equal(a.numpy(), g[f"s{i}_A"]), "seeded generator drifted"
        assert np.array_equal(b.numpy(), g[f"s{i}_B"])
        c = gemm.gemm_ref(a, b)
        assert gemm.rel_frobenius(c, torch.from_numpy(g[f"s{i}_C"])) < 1e-6
        c2 = gemm.gemm_alphabeta_ref(a, b, 2.0, 0.5, torch.from_numpy(g[f"s{i}_Cin"]))
        assert gemm.rel_frobenius(c2, torch.from_numpy(g[f"s{i}_C_a2b05"])) < 1e-6


def test_gemm_oracle_against_float64():
    a, b = gemm.seeded_ab(96, 80, 256, seed=1)
    ref64 = a.double() @ b.double()
    assert gemm.rel_frobenius(gemm.gemm_ref(a, b), ref64) < 1e-6


def test_alphabeta_semantics():
    a, b = gemm.seeded_ab(32, 16, 64, seed=2)
    c = gemm.seeded_c(32, 16)
    base = gemm.gemm_ref(a, b)
    assert torch.equal(gemm.gemm_alphabeta_ref(a, b, 1.0, 0.0, c), base)        # beta == 0: C ignored
    assert torch.equal(gemm.gemm_alphabeta_ref(a, b, 2.0, 0.5, None), 2.0 * base)  # C missing: alpha*AB


def test_tile_selection_matches_reference_run(golden_dir):
    rows = json.loads((golden_dir / "tile_selection.json").read_text())["rows"]
    assert len(rows) >= 20
    for M, N, K, cfg in rows:
        assert tile_plan.select_optimal_tile_ref(M, N, K) == cfg, (M, N, K)


def test_tile_selection_against_live_reference_binary(golden_dir):
    exe = ROOT / "oracle" / "_ref" / "tile_select"
    if not exe.exists():
        pytest.skip("oracle/_ref/tile_select not built (needs the reference tree)")
    rng = np.random.default_rng(0)
    shapes = [(int(rng.integers(1, 20000)), int(rng.integers(1, 20000)), int(rng.integers(1, 20000))) for _ in range(500)]
    inp = "".join(f"{m} {n} {k}\n" for m, n, k in shapes)
    out = subprocess.run([str(exe)], input=inp, capture_output=True, text=True, check=True).stdout
    for line in out.strip().splitlines():
        M, N, K, cfg = map(int, line.split())
        assert tile_plan.select_optimal_tile_ref(M, N, K) == cfg, (M, N, K)


def test_split_k_plan_restatement():
    # worked by hand from wmma_xor_swizzle.hpp:293-332 for 256x256x16384 on 40 CUs
    p = tile_plan.split_k_config_ref(256, 256, 16384)
    assert (p.split_factor, p.k_per_split, p.workspace_size) == (32, 512, 8 * 1024 * 1024)
    p = tile_plan.split_k_config_ref(4096, 4096, 4096)
    assert (p.split_factor, p.k_per_split, p.workspace_size) == (1, 4096, 0)
    p = tile_plan.split_k_config_ref(128, 64, 1024)   # one tile, K/256 = 4 caps the factor
    assert p.split_factor == 4 and p.k_per_split == 256


def test_int4_pack_roundtrip_and_fixture(golden_dir):
    g = np.load(golden_dir / "int4_golden.npz")
    codes = torch.from_numpy(g["codes"])
    q = int4.pack_ref(codes)
    assert np.array_equal(q.numpy(), g["qweight"])
    assert torch.equal(int4.unpack_ref(q, *codes.shape), codes)
    w = int4.dequant_ref(codes, torch.from_numpy(g["scales"]), int(g["group"]))
    assert np.array_equal(w.numpy().view(np.uint16), g["W"].view(np.uint16))


def test_int4_nibble_order_by_hand():
    codes = torch.zeros(64, 8, dtype=torch.uint8)
    codes[8:16, 3] = torch.tensor([1, 2, 3, 4, 5, 6, 7, 9], dtype=torch.uint8)
    q = int4.pack_ref(codes)
    assert q.shape == (1, 1, 128, 8)  # [K/64, ceil(N/128), 128, 8]
    # column 3, word 1 (k = 8..15): nibbles p=0..7 hold k = 8+{0,2,4,6,1,3,5,7} -> 1,3,5,7,2,4,6,9
    assert (q[0, 0, 3, 1].item() & 0xFFFFFFFF) == 0x96427531
    assert int(q.abs().sum()) == abs(q[0, 0, 3, 1].item())


def test_int4_dequant_is_single_rounded_fp16_product():
    codes, scales = int4.seeded_w4(256, 16, 128, seed=9)
    w = int4.dequant_ref(codes, scales, 128)
    q16 = (codes.to(torch.int32) - 8).to(torch.float16)
    s16 = scales.repeat_interleave(128, dim=0)
    assert torch.equal(w, q16 * s16)  # torch's CPU fp16 multiply rounds once as well


def test_attention_oracle_fixture_and_properties(golden_dir):
    g = np.load(golden_dir / "attention_golden.npz")
    Q, K, V = (torch.from_numpy(g[k]) for k in ("Q", "K", "V"))
    o = attention.attention_ref(Q, K, V, False)
    oc = attention.attention_ref(Q, K, V, True)
    assert np.array_equal(o.numpy().view(np.uint16), g["O"].view(np.uint16))
    assert np.array_equal(oc.numpy().view(np.uint16), g["O_causal"].view(np.uint16))
    # causal row 0 attends only to key 0
    assert torch.allclose(oc[:, :, 0].float(), V[:, :, 0].float(), atol=1e-3)
    # against torch's own SDPA in fp32
    ref = torch.nn.functional.scaled_dot_product_attention(Q.float(), K.float(), V.float())
    assert (o.float() - ref).abs().max().item() < 2e-3
