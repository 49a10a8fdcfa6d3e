"""GEMM oracle: the computation the reference's tests compare against, on the host in fp32.

TEST INFRASTRUCTURE. Follows test_fragment_loading.py:93 (`torch.matmul(A.float(), B.float())`)
and the fused epilogue of wmma_gemm.hip:653-660 (`alpha * acc + beta * C_in`, C_in read only
when beta != 0 and a C was given).
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch


def gemm_ref(A: torch.Tensor, B: torch.Tensor) -> torch.Tensor:
    """C = A.float() @ B.float() on the CPU (test_fragment_loading.py:93)."""
    return torch.matmul(A.detach().cpu().float(), B.detach().cpu().float())


def gemm_alphabeta_ref(A, B, alpha: float = 1.0, beta: float = 0.0, C: Optional[torch.Tensor] = None) -> torch.Tensor:
    """alpha * (A @ B) + beta * C with alpha, beta rounded to fp32 first (wmma_gemm.hip:1941,
    :653-660). beta != 0 with C=None degrades to alpha * A @ B, as in the reference (:1913)."""
    a32 = torch.tensor(alpha, dtype=torch.float32)
    b32 = torch.tensor(beta, dtype=torch.float32)
    out = a32 * gemm_ref(A, B)
    if float(beta) != 0.0 and C is not None:
        out = out + b32 * C.detach().cpu().float()
    return out


def rel_frobenius(C: torch.Tensor, C_ref: torch.Tensor) -> float:
    """||C - C_ref||_F / ||C_ref||_F in float64 (the relative L2 error the reference prints,
    test_fragment_loading.py:122-125)."""
    c = C.detach().cpu().double()
    r = C_ref.detach().cpu().double()
    denom = r.norm().item()
    num = (c - r).norm().item()
    if denom == 0.0:
        return 0.0 if num == 0.0 else math.inf
    return num / denom


def reference_pass(C: torch.Tensor, C_ref: torch.Tensor) -> bool:
    """The reference's own pass rule: max-rel < 1e-2 or max-abs < 1.0 (test_fragment_loading.py:127-130)."""
    err = (C.detach().cpu().float() - C_ref).abs().max().item()
    ref_max = C_ref.abs().max().item()
    rel = err / ref_max if ref_max > 0 else (math.inf if err > 0 else 0.0)
    return rel < 1e-2 or err < 1.0


def known_answer_case() -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """M=N=64, K=16, A[i,j] = i % 16, B[j,k] = j  =>  C[i,k] = (i % 16) * 120 exactly
    (test_fragment_loading.py:225-274)."""
    M, N, K = 64, 64, 16
    A = (torch.arange(M) % 16).to(torch.float16)[:, None].expand(M, K).contiguous()
    B = torch.arange(K).to(torch.float16)[:, None].expand(K, N).contiguous()
    C = ((torch.arange(M) % 16).float() * 120.0)[:, None].expand(M, N).contiguous()
    return A, B, C


# The seven seeded shapes of test_fragment_loading.py:67-75.
REFERENCE_SEEDED_SHAPES = [
    (512, 512, 64), (512, 512, 128), (1024, 1024, 256), (2048, 2048, 512),
    (4096, 4096, 1024), (2048, 1024, 512), (1024, 2048, 512),
]


def seeded_ab(M: int, N: int, K: int, seed: int = 42, scale_by_k: bool = False):
    """fp16 N(0,1) A [M,K] and B [K,N] from a CPU generator (the reference seeds with 42,
    test_fragment_loading.py:87-89; it draws on the GPU, so only the procedure carries over).
    scale_by_k multiplies by K^-1/2, the sweep's input scaling."""
    g = torch.Generator().manual_seed(seed)
    A = torch.randn(M, K, generator=g, dtype=torch.float32)
    B = torch.randn(K, N, generator=g, dtype=torch.float32)
    if scale_by_k:
        A = A * (K ** -0.5)
    return A.to(torch.float16), B.to(torch.float16)


def seeded_c(M: int, N: int, seed: int = 43) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    return torch.randn(M, N, generator=g, dtype=torch.float32)
