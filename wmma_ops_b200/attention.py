"""flash_attention: the signature the reference documents (README.md:221-251),
flash_attention(Q, K, V, causal=False, scale=-1.0) with Q, K, V [B, H, N, D] fp16 on one CUDA
device and scale < 0 meaning 1/sqrt(D). Returns O with Q's shape and dtype."""
from __future__ import annotations

import torch

from . import _lib
from .ops import _device_guard, _post, _require, _status_word, _stream


def flash_attention(Q: torch.Tensor, K: torch.Tensor, V: torch.Tensor, causal: bool = False,
                    scale: float = -1.0) -> torch.Tensor:
    for t in (Q, K, V):
        _require(isinstance(t, torch.Tensor) and t.is_cuda, "Inputs must be CUDA tensors")
    _require(Q.device == K.device and Q.device == V.device, "Inputs must be on same device")
    _require(Q.dtype == torch.float16 and K.dtype == torch.float16 and V.dtype == torch.float16,
             "Inputs must be float16")
    _require(Q.dim() == 4 and K.dim() == 4 and V.dim() == 4, "Inputs must be 4D [B, H, N, D]")
    _require(K.shape == Q.shape and V.shape == Q.shape, "Q, K and V must have the same shape")
    B, H, S, D = Q.shape
    _require(D in (64, 128), f"head dimension must be 64 or 128 (got {D})")
    Q, K, V = Q.contiguous(), K.contiguous(), V.contiguous()
    O = torch.empty_like(Q)
    if Q.numel() == 0:
        return O
    dev = Q.device
    with _device_guard(dev):
        rc = _lib.load().wmma_ops_fmha_fwd(Q.data_ptr(), K.data_ptr(), V.data_ptr(), O.data_ptr(), B, H, S, D,
                                           float(scale), 1 if causal else 0, _status_word(dev).data_ptr(), _stream(dev))
        _lib.check(rc)
        _post(dev)
    return O
