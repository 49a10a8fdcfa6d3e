"""flash_attention: the signature the reference documents (README.md:221-251),
flash_attention(Q, K, V, causal=False, scale=-1.0) with Q, K, V [B, H, N, D] fp16 on one CUDA
device and scale < 0 meaning 1/sqrt(D). Returns O with Q's shape and dtype.

Decode shapes: K and V may hold more rows than Q when Q has at most 16 (a few new tokens against a
cache of keys and values, Q [B, H, Nq, D], K and V [B, H, Nkv, D], Nkv >= Nq). The causal mask then
lets query row i see the keys up to Nkv - Nq + i. These calls, and any call with Nq <= 16, run on a
kernel that splits the key range over the SMs instead of giving one CTA 128 query rows."""
from __future__ import annotations

import ctypes

import torch

from . import _lib
from .ops import _device_guard, _post, _require, _status_word, _stream, _workspace

DECODE_MAX_QUERIES = 16


def _strided_ok(t: torch.Tensor) -> bool:
    """A [B, H, N, D] view the prefill kernel can read in place: D contiguous, the other strides multiples of
    8 elements (16 bytes) and rows at least D apart, 16-byte aligned."""
    sb, sh, ss, sd = t.stride()
    return (sd == 1 and ss >= t.size(3) and all(v > 0 and v % 8 == 0 for v in (sb, sh, ss))
            and t.data_ptr() % 16 == 0)


def flash_attention(Q: torch.Tensor, K: torch.Tensor, V: torch.Tensor, causal: bool = False,
                    scale: float = -1.0, out: torch.Tensor = None) -> torch.Tensor:
    """See the module text. Beyond the documented signature: with more than 16 query rows Q, K and V may be
    views with a contiguous last dimension (e.g. the Q, K and V sections of a packed [tokens, 3, heads, D]
    projection output, permuted to [B, H, N, D]), which are read in place, and `out` may be such a view of the
    caller's buffer (e.g. [B, N, H, D] storage seen as [B, H, N, D]); nothing is copied then."""
    for t in (Q, K, V):
        _require(isinstance(t, torch.Tensor) and t.is_cuda, "Inputs must be CUDA tensors")
    _require(Q.device == K.device and Q.device == V.device, "Inputs must be on same device")
    _require(Q.dtype == torch.float16 and K.dtype == torch.float16 and V.dtype == torch.float16,
             "Inputs must be float16")
    _require(Q.dim() == 4 and K.dim() == 4 and V.dim() == 4, "Inputs must be 4D [B, H, N, D]")
    _require(K.shape == V.shape, "K and V must have the same shape")
    B, H, S, D = Q.shape
    Skv = K.size(2)
    _require(K.size(0) == B and K.size(1) == H and K.size(3) == D and (Skv == S or (S <= DECODE_MAX_QUERIES and Skv >= S)),
             "Q, K and V must have the same shape (K and V may be longer than Q when Q has at most 16 rows)")
    _require(D in (64, 128), f"head dimension must be 64 or 128 (got {D})")
    prefill = not (S <= DECODE_MAX_QUERIES and Skv >= 1)
    if not (prefill and all(_strided_ok(t) for t in (Q, K, V))):
        Q, K, V = Q.contiguous(), K.contiguous(), V.contiguous()
    if out is not None:
        _require(out.is_cuda and out.device == Q.device and out.dtype == torch.float16 and tuple(out.shape) == (B, H, S, D)
                 and (out.is_contiguous() or (prefill and _strided_ok(out))),
                 "out must be a float16 CUDA tensor [B, H, N, D], contiguous or with a contiguous last dimension")
        O = out
    else:
        O = torch.empty((B, H, S, D), dtype=torch.float16, device=Q.device)
    if Q.numel() == 0:
        return O
    dev = Q.device
    lib = _lib.load()
    with _device_guard(dev):
        if S <= DECODE_MAX_QUERIES and Skv >= 1:
            need = lib.wmma_ops_fmha_decode_workspace_bytes(B, H, S, Skv, D)
            ws_ptr, ws_bytes = None, 0
            if need > 0:
                ws = _workspace(dev, need)
                ws_ptr, ws_bytes = ws.data_ptr(), ws.numel()
            rc = lib.wmma_ops_fmha_decode(Q.data_ptr(), K.data_ptr(), V.data_ptr(), O.data_ptr(), B, H, S, Skv, D, float(scale),
                                          1 if causal else 0, ws_ptr, ws_bytes, _status_word(dev).data_ptr(), _stream(dev))
        else:
            strides = []
            for t in (Q, K, V, O):
                sb, sh, ss, _ = t.stride()
                strides += [ss, sh, sb]      # between tokens, heads, sequences (elements)
            rc = lib.wmma_ops_fmha_fwd_strided(Q.data_ptr(), K.data_ptr(), V.data_ptr(), O.data_ptr(), B, H, S, D,
                                               (ctypes.c_longlong * 12)(*strides), float(scale), 1 if causal else 0,
                                               _status_word(dev).data_ptr(), _stream(dev))
        _lib.check(rc)
        _post(dev)
    return O
