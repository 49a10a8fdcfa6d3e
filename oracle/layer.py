"""Single-process oracle of the sharded decoder-layer linears. TEST INFRASTRUCTURE.

The reference has no multi-GPU code; the workload is the Llama-7B-shaped set of W4A16
projections on 8192 tokens: QKV 4096->12288, O 4096->4096, gate/up 4096->2x11008,
down 11008->4096. The glue between the GEMMs is fixed here and used identically by the
sharded implementation: O's input is the first 4096 columns of the QKV output (config 5 of the
benchmark is the linears alone) or, with seq_len given, the output of softmax attention over the
Q, K and V sections (32 heads of 128, sequences of seq_len tokens); the MLP input is the O output,
act = silu(gate) * up. Each
intermediate is multiplied by GLUE_SCALE = 1/4 (exact in binary) before it is rounded to fp16, which
keeps the random-weight activations of this synthetic layer inside fp16 range.
"""
from __future__ import annotations

import torch

from . import attention, int4

HIDDEN = 4096
QKV_OUT = 12288
FFN = 11008
GROUP = 128
GLUE_SCALE = 0.25


def make_layer_weights(seed: int = 21, hidden: int = HIDDEN, qkv_out: int = QKV_OUT, ffn: int = FFN,
                       group: int = GROUP):
    """codes/scales for the four projections: name -> (codes [K,N] uint8, scales [K/g,N] fp16)."""
    shapes = {"qkv": (hidden, qkv_out), "o": (hidden, hidden), "gate_up": (hidden, 2 * ffn), "down": (ffn, hidden)}
    out = {}
    for i, (name, (K, N)) in enumerate(shapes.items()):
        out[name] = int4.seeded_w4(K, N, group, seed + i)
    return out


HEAD_DIM = 128


def attention_block_ref(qkv16: torch.Tensor, seq_len: int, causal: bool, head_dim: int = HEAD_DIM) -> torch.Tensor:
    """qkv16 fp16 [T, 3 * hidden] with columns [Q | K | V], heads contiguous inside each section,
    T = batch * seq_len tokens (sequence-major within a batch entry) -> attention output fp16 [T, hidden]."""
    T, three_h = qkv16.shape
    hidden = three_h // 3
    heads = hidden // head_dim
    batch = T // seq_len
    assert batch * seq_len == T and heads * head_dim == hidden
    q, k, v = (qkv16[:, i * hidden:(i + 1) * hidden].reshape(batch, seq_len, heads, head_dim).permute(0, 2, 1, 3).contiguous()
               for i in range(3))
    o = attention.attention_ref(q, k, v, causal)                       # fp16 [batch, heads, seq_len, head_dim]
    return o.permute(0, 2, 1, 3).reshape(T, hidden).contiguous()


def layer_ref(x: torch.Tensor, weights, group: int = GROUP, seq_len=None, causal: bool = True):
    """x fp16 [T, hidden] -> (attn_out fp32 [T, hidden], mlp_out fp32 [T, hidden]). With seq_len the
    attention core runs between the QKV and the O projection; without it O's input is the Q section."""
    hidden = x.shape[1]
    qkv = int4.w4a16_ref(x, *weights["qkv"], group)
    if seq_len is None:
        o_in = (qkv[:, :hidden] * GLUE_SCALE).to(torch.float16)
    else:
        o_in = attention_block_ref((qkv * GLUE_SCALE).to(torch.float16), seq_len, causal)
    attn_out = int4.w4a16_ref(o_in, *weights["o"], group)
    h = (attn_out * GLUE_SCALE).to(torch.float16)
    gu = int4.w4a16_ref(h, *weights["gate_up"], group)
    ffn = gu.shape[1] // 2
    act = (torch.nn.functional.silu(gu[:, :ffn]) * gu[:, ffn:] * GLUE_SCALE).to(torch.float16)
    mlp_out = int4.w4a16_ref(act, *weights["down"], group)
    return attn_out, mlp_out


def attention_flops(tokens: int, seq_len: int, causal: bool, hidden: int = HIDDEN) -> float:
    """Flops of the attention core over `tokens` tokens in sequences of seq_len (all heads)."""
    per_seq = 4.0 * hidden * (seq_len * (seq_len + 1) / 2 if causal else seq_len * seq_len)
    return per_seq * (tokens // seq_len)


def layer_flops(tokens: int, hidden: int = HIDDEN, qkv_out: int = QKV_OUT, ffn: int = FFN) -> float:
    return 2.0 * tokens * hidden * (qkv_out + hidden + 2 * ffn + ffn)
