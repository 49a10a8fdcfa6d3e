"""Attention oracle: O = softmax(scale * Q K^T [+ causal mask]) V in fp32 on the CPU.
TEST INFRASTRUCTURE.

PARITY UNPINNED: the reference tree holds only the documented signature
flash_attention(Q, K, V, causal=False, scale=-1.0) with Q, K, V [B,H,N,D] fp16 and the default
scale 1/sqrt(D) (README.md:221-251); its implementation and tests are not in the tree.
"""
from __future__ import annotations

import math

import torch


def attention_ref(Q: torch.Tensor, K: torch.Tensor, V: torch.Tensor, causal: bool = False,
                  scale: float = -1.0, out_dtype=torch.float16) -> torch.Tensor:
    q = Q.detach().cpu().float()
    k = K.detach().cpu().float()
    v = V.detach().cpu().float()
    B, H, S, D = q.shape
    if scale < 0:
        scale = 1.0 / math.sqrt(D)
    out = torch.empty_like(q)
    mask = None
    if causal:
        Sk = k.shape[2]
        mask = torch.ones(S, Sk, dtype=torch.bool).tril(diagonal=Sk - S)
    for b in range(B):
        for h in range(H):
            s = (q[b, h] @ k[b, h].T) * scale
            if mask is not None:
                s = s.masked_fill(~mask, float("-inf"))
            p = torch.softmax(s, dim=-1)
            out[b, h] = p @ v[b, h]
    return out.to(out_dtype)


def seeded_qkv(B: int, H: int, S: int, D: int, seed: int = 11):
    g = torch.Generator().manual_seed(seed)
    mk = lambda: torch.randn(B, H, S, D, generator=g, dtype=torch.float32).to(torch.float16)
    return mk(), mk(), mk()


def fmha_flops(B: int, H: int, S: int, D: int, causal: bool) -> float:
    return 4.0 * B * H * D * (S * (S + 1) / 2 if causal else S * S)
