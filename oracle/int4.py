"""INT4 weight format "W4-B200-v1" and W4A16 arithmetic on the CPU. TEST INFRASTRUCTURE.

PARITY UNPINNED: the reference tree contains no INT4 / W4A16 code, so there is nothing of the
reference to check this against; this file is the written specification the CUDA prepack,
unpack and dequant kernels must match bit for bit.

Format
  codes    uint8 [K, N], values 0..15; weight[k, n] = (code[k, n] - 8) * scale[k // g, n]
  scales   fp16 [K // g, N] (g = group size along K, 128 in the configs)
  qweight  uint32 [K // 64, ceil(N/128), 128, 8]: block (kb, nt) is 4 KB and holds, for the 128
           columns n = 128 nt + r (zero codes where n >= N), the codes k = 64 kb .. 64 kb + 63 as
           8 words per column; word j, nibble p (bits 4p .. 4p+3) holds
           k = 64 kb + 8 j + NIBBLE_K[p], NIBBLE_K = (0, 2, 4, 6, 1, 3, 5, 7).
           With this nibble order `(word >> 4i) & 0x000F000F` yields the adjacent pair
           (k = 8j+2i, 8j+2i+1) in the low / high half-word, which is what a half2 dequant wants;
           blocks are ordered k-block major, so CTAs that walk K in step read one contiguous window.
"""
from __future__ import annotations

import numpy as np
import torch

NIBBLE_K = (0, 2, 4, 6, 1, 3, 5, 7)
ZERO_POINT = 8


def pack_ref(codes: torch.Tensor) -> torch.Tensor:
    """codes uint8 [K,N] -> qweight int32 [K//64, ceil(N/128), 128, 8] (bit pattern of uint32 words)."""
    c = codes.detach().cpu().numpy().astype(np.uint32)
    K, N = c.shape
    assert K % 64 == 0 and c.max(initial=0) <= 15
    n_pad = -(-N // 128) * 128
    cp = np.zeros((K, n_pad), dtype=np.uint32)
    cp[:, :N] = c
    # [kb, j, kk, nt, r] -> [kb, nt, r, j, kk]
    t = cp.reshape(K // 64, 8, 8, n_pad // 128, 128).transpose(0, 3, 4, 1, 2)
    words = np.zeros(t.shape[:4], dtype=np.uint32)
    for p, kk in enumerate(NIBBLE_K):
        words |= t[..., kk] << np.uint32(4 * p)
    return torch.from_numpy(np.ascontiguousarray(words).view(np.int32))


def unpack_ref(qweight: torch.Tensor, K: int, N: int) -> torch.Tensor:
    """qweight int32 [K//64, ceil(N/128), 128, 8] -> codes uint8 [K,N]."""
    n_tiles = -(-N // 128)
    w = qweight.detach().cpu().numpy().view(np.uint32).reshape(K // 64, n_tiles, 128, 8)
    t = np.zeros((K // 64, n_tiles, 128, 8, 8), dtype=np.uint8)
    for p, kk in enumerate(NIBBLE_K):
        t[..., kk] = ((w >> np.uint32(4 * p)) & np.uint32(0xF)).astype(np.uint8)
    # [kb, nt, r, j, kk] -> [kb, j, kk, nt, r]
    c = t.transpose(0, 3, 4, 1, 2).reshape(K, n_tiles * 128)
    return torch.from_numpy(np.ascontiguousarray(c[:, :N]))


def dequant_ref(codes: torch.Tensor, scales: torch.Tensor, group_size: int = 128) -> torch.Tensor:
    """W fp16 [K,N] = fp16(code - 8) * scale[k // g, n], a single fp16 multiply rounded to
    nearest even (computed in fp32 and rounded once: the product of two fp16 values is exact in
    fp32, so one rounding to fp16 equals the IEEE fp16 multiply)."""
    K, N = codes.shape
    q = (codes.detach().cpu().to(torch.int32) - ZERO_POINT).to(torch.float32)
    s = scales.detach().cpu().to(torch.float32).repeat_interleave(group_size, dim=0)[:K]
    return (q * s).to(torch.float16)


def w4a16_ref(A: torch.Tensor, codes: torch.Tensor, scales: torch.Tensor, group_size: int = 128) -> torch.Tensor:
    """C fp32 [M,N] = A.float() @ dequant(codes, scales).float()."""
    W = dequant_ref(codes, scales, group_size)
    return torch.matmul(A.detach().cpu().float(), W.float())


def w4a16_block_scaled_ref(A: torch.Tensor, codes: torch.Tensor, scales: torch.Tensor, group_size: int = 128) -> torch.Tensor:
    """The decode kernel's own definition of the product (M <= 16, library-chosen plan): no weight
    is rounded; C[m, n] = sum over 64-deep blocks b of scale[b*64 // g, n] * sum_{k in b} A[m, k] *
    (code[k, n] - 8). Evaluated in float64 (the integer-weighted block sums are exact there), returned
    as fp32. It differs from w4a16_ref, which rounds every (code - 8) * scale product to fp16 first,
    by that rounding (about 2e-4 relative)."""
    K, N = codes.shape
    a = A.detach().cpu().to(torch.float64)
    q = (codes.detach().cpu().to(torch.int32) - ZERO_POINT).to(torch.float64)
    s = scales.detach().cpu().to(torch.float64)
    out = torch.zeros(a.shape[0], N, dtype=torch.float64)
    for b in range(K // 64):
        blk = a[:, 64 * b:64 * b + 64] @ q[64 * b:64 * b + 64]
        out += blk * s[(64 * b) // group_size][None, :]
    return out.to(torch.float32)


def seeded_w4(K: int, N: int, group_size: int = 128, seed: int = 7):
    """codes uniform in [0,15], scales fp16 uniform in [0.001, 0.02] (the W4A16 config)."""
    g = torch.Generator().manual_seed(seed)
    codes = torch.randint(0, 16, (K, N), generator=g, dtype=torch.uint8)
    scales = (torch.rand(K // group_size, N, generator=g) * (0.02 - 0.001) + 0.001).to(torch.float16)
    return codes, scales


def w4a16_bytes(M: int, N: int, K: int, group_size: int = 128) -> int:
    """Algorithmic bytes of one W4A16 product: packed weights + scales + activations + fp32 output."""
    return K * N // 2 + 2 * (K // group_size) * N + 2 * M * K + 4 * M * N
