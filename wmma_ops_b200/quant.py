"""INT4 prepack and W4A16 matmul entry points.

The reference snapshot has neither (its README and sources contain no INT4 code), so names,
packed format ("W4-B200-v1", described in include/wmma_ops_b200.h) and arithmetic are defined
by this package:  weight[k, n] = (code[k, n] - 8) * scale[k // group_size, n],  C = A @ weight
with fp16 operands and fp32 accumulation.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _lib
from .ops import _device_guard, _post, _require, _sm_count, _status_word, _stream, _workspace

ZERO_POINT = 8


def _check_codes(codes: torch.Tensor, scales: torch.Tensor, group_size: int) -> Tuple[int, int]:
    _require(codes.is_cuda and scales.is_cuda, "Inputs must be CUDA tensors")
    _require(codes.device == scales.device, "Inputs must be on same device")
    _require(codes.dtype == torch.uint8, "codes must be uint8 with values 0..15")
    _require(scales.dtype == torch.float16, "scales must be float16")
    _require(codes.dim() == 2 and scales.dim() == 2, "codes and scales must be 2D")
    K, N = codes.shape
    _require(group_size > 0 and K % group_size == 0, f"group_size must divide K (got group_size={group_size}, K={K})")
    _require(tuple(scales.shape) == (K // group_size, N),
             f"scales must have shape [K/group_size, N] = [{K // group_size}, {N}]")
    return K, N


def int4_prepack(codes: torch.Tensor, scales: torch.Tensor, group_size: int = 128,
                 zero_point: int = ZERO_POINT) -> Tuple[torch.Tensor, torch.Tensor]:
    """Packs uint8 codes [K,N] (0..15) into the kernel's layout.

    Returns (qweight int32 [K/64, ceil(N/128), 128, 8], scales fp16 [K/group_size, N] contiguous)."""
    _require(zero_point == ZERO_POINT, "only zero_point=8 is supported")
    K, N = _check_codes(codes, scales, group_size)
    codes = codes.contiguous()
    dev = codes.device
    q = torch.empty((K // 64, (N + 127) // 128, 128, 8), dtype=torch.int32, device=dev)
    with _device_guard(dev):
        _lib.check(_lib.load().wmma_ops_int4_prepack(codes.data_ptr(), q.data_ptr(), K, N, _stream(dev)))
    return q, scales.contiguous()


def _qshape(qweight: torch.Tensor, N: int) -> Tuple[int, int]:
    _require(qweight.is_cuda and qweight.dtype == torch.int32 and qweight.dim() == 4
             and qweight.size(2) == 128 and qweight.size(3) == 8 and qweight.is_contiguous(),
             "qweight must be a contiguous CUDA int32 tensor [K/64, ceil(N/128), 128, 8] from int4_prepack")
    _require(qweight.size(1) == (N + 127) // 128, "qweight does not match N")
    return qweight.size(0) * 64, N


def int4_unpack(qweight: torch.Tensor, N: int) -> torch.Tensor:
    """Inverse of int4_prepack: codes uint8 [K,N]."""
    K, N = _qshape(qweight, N)
    dev = qweight.device
    out = torch.empty((K, N), dtype=torch.uint8, device=dev)
    with _device_guard(dev):
        _lib.check(_lib.load().wmma_ops_int4_unpack(qweight.data_ptr(), out.data_ptr(), K, N, _stream(dev)))
    return out


def int4_dequant(qweight: torch.Tensor, scales: torch.Tensor, group_size: int = 128) -> torch.Tensor:
    """fp16 weights [K,N] = fp16(code - 8) * scale, one fp16 multiply per element."""
    _require(scales.is_cuda and scales.dtype == torch.float16 and scales.dim() == 2, "scales must be CUDA float16 2D")
    K, N = _qshape(qweight, scales.size(1))
    _require(scales.size(0) * group_size == K, "scales do not match K / group_size")
    dev = qweight.device
    out = torch.empty((K, N), dtype=torch.float16, device=dev)
    with _device_guard(dev):
        _lib.check(_lib.load().wmma_ops_int4_dequant(qweight.data_ptr(), scales.contiguous().data_ptr(),
                                                     out.data_ptr(), K, N, group_size, _stream(dev)))
    return out


OUT_F32, OUT_F16, OUT_F16_SILU_MUL = 0, 1, 2


def set_w4a16_overlap(enable: bool) -> None:
    """Switches overlapped decode launches on or off (off by default, process-wide): with it on,
    matmul_w4a16 products with up to 16 rows start fetching their packed weights while the previous
    kernel of the stream is still finishing (programmatic dependent launch) and wait for it before
    reading the activations. Only for weights and scales that are not produced by the kernels queued
    just before the call, which is the case in decode."""
    _lib.check(_lib.load().wmma_ops_set_w4a16_overlap(1 if enable else 0))


def interleave_gate_up(codes: torch.Tensor, scales: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Reorders the columns of a [K, 2F] gate|up weight (gate columns first, then up columns) so that
    every 128-column tile holds 64 gate columns followed by the 64 up columns of the same outputs,
    the layout the fused silu(gate) * up epilogue of matmul_w4a16 expects. F must be a multiple of 64."""
    K, N2 = codes.shape
    F = N2 // 2
    _require(N2 % 2 == 0 and F % 64 == 0, "gate/up width must be a multiple of 64")
    idx = torch.arange(F, device=codes.device).view(F // 64, 1, 64)
    order = torch.cat([idx, idx + F], dim=1).reshape(-1)
    return codes[:, order].contiguous(), scales[:, order].contiguous()


def w4a16_token_block(M: int) -> int:
    """Rows per token block of the tcgen05 W4A16 kernel for a product with M rows (see block_done)."""
    return int(_lib.load().wmma_ops_w4a16_token_block(int(M)))


def matmul_w4a16(A: torch.Tensor, qweight: torch.Tensor, scales: torch.Tensor, group_size: int = 128,
                 split_k: int = 0, out_dtype: torch.dtype = torch.float32, alpha: float = 1.0,
                 epilogue: str = "none", out: Optional[torch.Tensor] = None, in_scale: float = 1.0,
                 block_done: Optional[torch.Tensor] = None) -> torch.Tensor:
    """C [M,N] = A fp16 [M,K] @ dequant(qweight, scales); the weights are expanded inside the kernel,
    never written to memory. split_k=0 lets the library choose: up to 16 rows go to the decode
    kernel (every CTA owns a range of columns and streams their packed weights over all of K; exact
    integer weights, the group scale applied to fp32 block sums), more rows to the tcgen05 kernel
    (weights rounded to fp16 as int4_dequant does).

    out_dtype=torch.float32 (default) returns the fp32 accumulators. out_dtype=torch.float16 returns
    half(alpha * acc). epilogue="silu_mul" (weights prepared with interleave_gate_up) returns
    half(alpha * silu(in_scale * gate) * (in_scale * up)) of shape [M, N/2]; in_scale stands for a scale
    of A that the caller left out (A @ W is linear in A). `out`, if given, is the contiguous tensor of that
    shape and dtype the result is written to (for example a buffer in symmetric memory).

    block_done (M > 16, no K split): int32 CUDA tensor, zero before the call, one entry per block of
    w4a16_token_block(M) rows. The kernel then works through the rows block by block and adds one to
    block_done[b] whenever a 128-column tile of block b is in memory, so that a kernel running beside it
    can consume finished blocks (a block is complete at ceil(N / 128))."""
    _require(A.is_cuda and qweight.is_cuda and scales.is_cuda, "Inputs must be CUDA tensors")
    _require(A.device == qweight.device and A.device == scales.device, "Inputs must be on same device")
    _require(A.dtype == torch.float16, "Inputs must be float16")
    _require(scales.dtype == torch.float16 and scales.dim() == 2, "scales must be float16 [K/group_size, N]")
    _require(A.dim() == 2, "Inputs must be 2D")
    _require(epilogue in ("none", "silu_mul"), "epilogue must be 'none' or 'silu_mul'")
    _require(float(in_scale) == 1.0 or epilogue == "silu_mul", "in_scale is only used by the silu_mul epilogue")
    _require(out_dtype in (torch.float32, torch.float16), "out_dtype must be float32 or float16")
    N = scales.size(1)
    K, N = _qshape(qweight, N)
    _require(A.size(1) == K, "Inner dimensions must match")
    _require(scales.size(0) * group_size == K, "scales do not match K / group_size")
    A = A.contiguous()
    scales = scales.contiguous()
    _require(A.data_ptr() % 16 == 0, "A must be 16-byte aligned")
    M = A.size(0)
    dev = A.device
    lib = _lib.load()
    if epilogue == "silu_mul":
        _require(N % 128 == 0, "the fused gate/up epilogue needs N to be a multiple of 128")
        mode, C = OUT_F16_SILU_MUL, torch.empty((M, N // 2), dtype=torch.float16, device=dev)
    elif out_dtype == torch.float16:
        mode, C = OUT_F16, torch.empty((M, N), dtype=torch.float16, device=dev)
    else:
        _require(float(alpha) == 1.0, "alpha is only applied to float16 outputs")
        mode, C = OUT_F32, torch.empty((M, N), dtype=torch.float32, device=dev)
    if out is not None:
        _require(out.is_cuda and out.device == dev and out.dtype == C.dtype and tuple(out.shape) == tuple(C.shape)
                 and out.is_contiguous(), "out must be a contiguous CUDA tensor of the result's shape and dtype")
        C = out
    if M == 0:
        return C
    done_ptr = None
    if block_done is not None:
        _require(M > 16 and split_k in (0, 1), "block_done needs more than 16 rows and no K split")
        _require(block_done.is_cuda and block_done.device == dev and block_done.dtype == torch.int32
                 and block_done.is_contiguous() and block_done.numel() * w4a16_token_block(M) >= M,
                 "block_done must be a contiguous int32 CUDA tensor with one entry per token block")
        done_ptr = block_done.data_ptr()
    with _device_guard(dev):
        ws_ptr, ws_bytes = None, 0
        need = lib.wmma_ops_w4a16_workspace_bytes(M, N, K, split_k)   # split_k = 0: the library's own plan
        if need > 0:
            ws = _workspace(dev, need, zero_init=True)
            ws_ptr, ws_bytes = ws.data_ptr(), ws.numel()
        rc = lib.wmma_ops_w4a16_gemm_blocks(A.data_ptr(), qweight.data_ptr(), scales.data_ptr(), C.data_ptr(), M, N, K,
                                            group_size, split_k, mode, float(alpha), float(in_scale), ws_ptr, ws_bytes,
                                            done_ptr, _status_word(dev).data_ptr(), _stream(dev))
        _lib.check(rc)
        _post(dev)
    return C
