"""Column/row-sharded decoder-layer linears over 1/2/4/8 GPUs (one process per GPU).

The reference is single-GPU; this is the layer-shaped workload built from its GEMM path:
W4A16 projections QKV (hidden -> 3*hidden), O (hidden -> hidden), gate/up (hidden -> 2*ffn) and
down (ffn -> hidden) on a block of tokens. QKV and gate/up are column-parallel (output columns
sharded, no communication), O and down are row-parallel (K sharded) and end in the only
collective of the project, an all-reduce (sum) of the partial outputs through
torch.distributed (NCCL on GPUs).

Sharding rules
  * shard boundaries fall on multiples of 128 columns / rows, which are both the quantisation
    group size and the kernel's column-tile width, so scales and packed blocks are never split;
    11008 = 86 groups is cut as evenly as 86 allows (tp=4: 22,22,21,21; tp=8: 11 x6, 10 x2);
  * the Q, K and V sections of the QKV weight are each cut by rank, so rank r's slice of the Q
    section is exactly the K-shard of O it owns (no exchange between QKV and O);
  * gate and up are cut with the same partition as down's rows, so silu(gate) * up is local.
Every rank packs its own shard after slicing (the packed layout is tile-major along K).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Tuple

import torch

GROUP = 128
# Every intermediate is scaled by 1/4 (exact) before its fp16 rounding so that the random-weight
# activations of the synthetic layer stay inside fp16 range; the oracle uses the same constant.
GLUE_SCALE = 0.25


def split_units(total_units: int, parts: int) -> List[Tuple[int, int]]:
    """Cuts `total_units` into `parts` contiguous ranges as evenly as possible (the first
    total_units % parts ranges get one more). Returns [(start, stop)] in units."""
    if parts < 1 or total_units < parts:
        raise ValueError(f"cannot cut {total_units} units into {parts} non-empty parts")
    base, extra = divmod(total_units, parts)
    out, start = [], 0
    for r in range(parts):
        n = base + (1 if r < extra else 0)
        out.append((start, start + n))
        start += n
    return out


def shard_range(size: int, rank: int, world: int, unit: int = GROUP) -> Tuple[int, int]:
    """[start, stop) of rank's shard of a dimension of `size` cut on multiples of `unit`."""
    if size % unit != 0:
        raise ValueError(f"dimension {size} is not a multiple of {unit}")
    a, b = split_units(size // unit, world)[rank]
    return a * unit, b * unit


@dataclass
class LayerShapes:
    hidden: int = 4096
    qkv_out: int = 12288
    ffn: int = 11008
    group: int = GROUP


def shard_layer_weights(weights: Dict[str, Tuple[torch.Tensor, torch.Tensor]], rank: int, world: int,
                        shapes: LayerShapes = LayerShapes()) -> Dict[str, Tuple[torch.Tensor, torch.Tensor]]:
    """Slices full (codes [K,N] uint8, scales [K/g,N] fp16) pairs into this rank's shards.
    Pure tensor slicing; works on any device."""
    g = shapes.group
    h, f = shapes.hidden, shapes.ffn
    sec = shapes.qkv_out // 3
    out = {}

    def cols(pair, ranges):
        codes, scales = pair
        return (torch.cat([codes[:, a:b] for a, b in ranges], dim=1).contiguous(),
                torch.cat([scales[:, a:b] for a, b in ranges], dim=1).contiguous())

    def rows(pair, a, b):
        codes, scales = pair
        return codes[a:b].contiguous(), scales[a // g:b // g].contiguous()

    qa, qb = shard_range(sec, rank, world, g)
    out["qkv"] = cols(weights["qkv"], [(s * sec + qa, s * sec + qb) for s in range(3)])
    out["o"] = rows(weights["o"], qa, qb)
    fa, fb = shard_range(f, rank, world, g)
    out["gate_up"] = cols(weights["gate_up"], [(fa, fb), (f + fa, f + fb)])
    out["down"] = rows(weights["down"], fa, fb)
    return out


class ShardedDecoderLinears:
    """One rank's part of the layer. `matmul(x_fp16, name) -> fp32` computes x @ W_local[name];
    by default it is the fused W4A16 kernel on prepacked shards. `all_reduce(t)` sums a tensor
    over the ranks in place (torch.distributed by default; a no-op for world size 1)."""

    def __init__(self, local_weights: Dict[str, Tuple[torch.Tensor, torch.Tensor]], world: int = 1,
                 group: int = GROUP, matmul: Optional[Callable] = None, all_reduce: Optional[Callable] = None,
                 reduce_dtype: torch.dtype = torch.float32, chunks: int = 1, switch=None,
                 attention: Optional[Tuple[int, bool]] = None, head_dim: int = 128,
                 attention_fn: Optional[Callable] = None, follow: bool = False):
        self.world = world
        # with a switch: the sum of a row-parallel output runs beside the GEMM that produces it, token block
        # by token block, on a helper stream (SwitchAllReduce.reduce_following)
        self.follow = bool(follow) and switch is not None and world > 1
        self._helpers: Dict[int, torch.cuda.Stream] = {}
        # (seq_len, causal): run the attention core between QKV and O on this rank's heads (the Q, K
        # and V sections are cut by rank, so a rank holds whole heads and attention needs no exchange);
        # None keeps the linears-only workload, where O's input is the rank's slice of the Q section
        self.attention = attention
        self.head_dim = head_dim
        self._attention_fn = attention_fn    # (Q, K, V, causal) -> O on [batch, heads, seq, D]; default flash_attention
        # optional collective.SwitchAllReduce: the row-parallel GEMMs then write fp16 partial outputs
        # into its symmetric buffers and the sum is done through the NVSwitch by the library's own
        # kernel; forward() then returns views of those buffers (valid until the next forward)
        self.switch = switch if world > 1 else None
        if self.switch is not None and reduce_dtype != self.switch.partial_dtype:
            raise ValueError("reduce_dtype must be the dtype of the switch's partial-output buffers")
        self.group = group
        self.reduce_dtype = reduce_dtype
        self.chunks = max(1, chunks)
        self.q_cols = local_weights["qkv"][0].shape[1] // 3
        self.ffn_local = local_weights["gate_up"][0].shape[1] // 2
        self.fused = matmul is None
        if matmul is None:
            # Product path: prepacked shards, fused output stages (fp16 activations written by the
            # GEMM epilogue, silu(gate) * up inside the gate/up GEMM).
            from .quant import int4_prepack, interleave_gate_up, matmul_w4a16
            prepared = dict(local_weights)
            prepared["gate_up"] = interleave_gate_up(*local_weights["gate_up"])
            packed = {k: int4_prepack(c, s, group) for k, (c, s) in prepared.items()}
            self.packed = packed
            self._w4 = lambda x, name, **kw: matmul_w4a16(x, packed[name][0], packed[name][1], group, **kw)  # noqa: E731
            matmul = lambda x, name: self._w4(x, name)  # noqa: E731
        self._matmul = matmul
        if all_reduce is None:
            all_reduce = self._dist_all_reduce
        self._all_reduce = all_reduce

    def _dist_all_reduce(self, t: torch.Tensor, async_op: bool = False):
        if self.world == 1:
            return None
        import torch.distributed as dist
        return dist.all_reduce(t, op=dist.ReduceOp.SUM, async_op=async_op)

    def _switch_row_parallel(self, a: torch.Tensor, name: str, slot: int, row0: int = 0,
                             channel: Optional[int] = None) -> torch.Tensor:
        """a @ W_local written into rows [row0, row0 + len(a)) of the switch's buffer `slot` and summed over the
        ranks; returns the fp16 sums. With follow, the sum kernel is launched on a helper stream right after the
        GEMM and consumes finished token blocks while the GEMM computes the next ones."""
        from .quant import w4a16_token_block
        sw, rows = self.switch, a.shape[0]
        out = sw.buffer(slot)[row0:row0 + rows]
        if not (self.follow and rows > 128 and row0 % 32 == 0):
            self._w4(a, name, out_dtype=self.reduce_dtype, out=out)
            return sw.reduce(slot, rows, row0=row0, channel=channel)
        cur = torch.cuda.current_stream(a.device)
        helper = self._helpers.get(cur.cuda_stream)
        if helper is None:
            helper = self._helpers[cur.cuda_stream] = torch.cuda.Stream(device=a.device)
        helper.wait_stream(cur)      # the sum may not overtake earlier readers of the buffer
        self._w4(a, name, out_dtype=self.reduce_dtype, out=out, block_done=sw.counters(slot, row0))
        tiles = (out.shape[1] + 127) // 128
        with torch.cuda.stream(helper):
            part = sw.reduce_following(slot, rows, w4a16_token_block(rows), tiles, row0=row0, channel=channel)
        cur.wait_stream(helper)
        return part

    def _row_parallel(self, x: torch.Tensor, name: str) -> torch.Tensor:
        """x @ W_local (K-sharded) summed over ranks. Token chunks let the all-reduce of one
        chunk overlap the GEMM of the next (NCCL runs on its own stream)."""
        T = x.shape[0]
        if self.world == 1:
            return self._matmul(x, name)
        n_chunks = min(self.chunks, max(1, T // 256))
        bounds = [(i * T // n_chunks, (i + 1) * T // n_chunks) for i in range(n_chunks)]
        parts, handles = [], []
        for a, b in bounds:
            part = self._matmul(x[a:b], name)
            if self.reduce_dtype != part.dtype:
                part = part.to(self.reduce_dtype)
            handles.append(self._all_reduce(part, True) if n_chunks > 1 else self._all_reduce(part))
            parts.append(part)
        for h in handles:
            if h is not None and hasattr(h, "wait"):
                h.wait()
        return parts[0] if n_chunks == 1 else torch.cat(parts, dim=0)

    def _o_input(self, qkv16: torch.Tensor) -> torch.Tensor:
        """O's input from this rank's fp16 QKV output [T, 3 * q_cols] (columns Q | K | V)."""
        if self.attention is None:
            return qkv16[:, :self.q_cols].contiguous()
        fn = self._attention_fn
        if fn is None:
            from .attention import flash_attention as fn
        seq_len, causal = self.attention
        T = qkv16.shape[0]
        heads = self.q_cols // self.head_dim
        if T % seq_len != 0 or heads * self.head_dim != self.q_cols:
            raise ValueError(f"{T} tokens are not whole sequences of {seq_len}, or the shard does not hold whole heads")
        batch = T // seq_len
        qkv = qkv16.view(batch, seq_len, 3, heads, self.head_dim)
        if self._attention_fn is None:
            # the library's kernel reads the Q, K and V sections of the projection output where they lie and
            # writes token-major, which is what the O projection reads: no copies either side
            o = torch.empty((batch, seq_len, heads, self.head_dim), dtype=torch.float16, device=qkv16.device)
            q, k, v = (qkv[:, :, i].permute(0, 2, 1, 3) for i in range(3))
            fn(q, k, v, causal, out=o.permute(0, 2, 1, 3))
            return o.view(T, self.q_cols)
        # a caller's attention function: [3, batch, heads, seq, D] contiguous in, [batch, heads, seq, D] out
        qkv = qkv.permute(2, 0, 3, 1, 4).contiguous()
        o = fn(qkv[0], qkv[1], qkv[2], causal)
        return o.permute(0, 2, 1, 3).reshape(T, self.q_cols)     # a copy: [batch, seq, heads, D] row-major

    def forward(self, x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """x fp16 [T, hidden] (replicated) -> (attn_out, mlp_out), both [T, hidden], replicated,
        in reduce_dtype. The glue is the oracle's: O's input is this rank's slice of the Q section
        of the QKV output; the MLP input is attn_out; act = silu(gate) * up; each scaled by GLUE_SCALE, fp16 between GEMMs."""
        if self.fused:
            return self._forward_fused(x)
        qkv = self._matmul(x, "qkv")
        if self.attention is None:
            o_in = (qkv[:, :self.q_cols] * GLUE_SCALE).to(torch.float16)
        else:
            o_in = self._o_input((qkv * GLUE_SCALE).to(torch.float16))
        attn_out = self._row_parallel(o_in, "o")
        h = (attn_out * GLUE_SCALE).to(torch.float16)
        gu = self._matmul(h, "gate_up")
        f = self.ffn_local
        act = (torch.nn.functional.silu(gu[:, :f]) * gu[:, f:] * GLUE_SCALE).to(torch.float16)
        mlp_out = self._row_parallel(act, "down")
        return attn_out, mlp_out

    def _forward_fused(self, x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """Same arithmetic with the glue inside the GEMM epilogues: QKV writes half(GLUE_SCALE * acc),
        gate/up writes half(GLUE_SCALE * silu(gate) * up); only the slice copy and the scaling of the
        all-reduced attention output remain as separate (small) kernels."""
        if self.world > 1 and self.chunks > 1 and x.shape[0] >= 512 * self.chunks and (
                self.attention is None or (x.shape[0] // self.chunks) % self.attention[0] == 0):
            return self._forward_pipelined(x)
        out_dt = self.reduce_dtype
        qkv16 = self._w4(x, "qkv", out_dtype=torch.float16, alpha=GLUE_SCALE)
        o_in = self._o_input(qkv16)
        if self.switch is not None:
            # partial outputs (fp16, or the fp32 accumulators) go straight into symmetric memory and are
            # summed through the switch by one launch; the sums are fp16, so the 1/4 scaling of the MLP
            # input is exact and is folded into the gate/up GEMM instead of a pass over the tensor
            attn_out = self._switch_row_parallel(o_in, "o", 0)
            act = self._w4(attn_out, "gate_up", epilogue="silu_mul", alpha=GLUE_SCALE, in_scale=GLUE_SCALE)
            mlp_out = self._switch_row_parallel(act, "down", 1)
            return attn_out, mlp_out
        self._matmul = lambda a, name: self._w4(a, name, out_dtype=out_dt)  # noqa: E731
        attn_out = self._row_parallel(o_in, "o")
        h = (attn_out * GLUE_SCALE).to(torch.float16)
        act = self._w4(h, "gate_up", epilogue="silu_mul", alpha=GLUE_SCALE)
        mlp_out = self._row_parallel(act, "down")
        return attn_out, mlp_out

    def _forward_pipelined(self, x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """The fused forward on token chunks, alternating between two side streams: while one
        chunk's partial outputs are being all-reduced (NCCL runs on its own stream), the other
        chunk's GEMMs run. The GEMM kernels are persistent and would fill every SM, so the caller
        should leave a few SMs free for the collective (wmma_ops_b200.set_sm_margin)."""
        import torch.distributed as dist
        out_dt = self.reduce_dtype
        T = x.shape[0]
        n = self.chunks
        bounds = [(i * T // n, (i + 1) * T // n) for i in range(n)]
        main = torch.cuda.current_stream(x.device)
        if getattr(self, "_streams", None) is None:
            self._streams = [torch.cuda.Stream(device=x.device) for _ in range(2)]
        if self.switch is not None:
            attn_out = mlp_out = None   # views of the summed buffers, taken from the last chunk's reduce
        else:
            attn_out = torch.empty((T, self.packed["o"][1].shape[1]), dtype=out_dt, device=x.device)
            mlp_out = torch.empty_like(attn_out)
        for st in self._streams:
            st.wait_stream(main)
        keep, stage1, stage2 = [], [], []
        for c, (a, b) in enumerate(bounds):
            with torch.cuda.stream(self._streams[c % 2]):
                qkv16 = self._w4(x[a:b], "qkv", out_dtype=torch.float16, alpha=GLUE_SCALE)
                o_in = self._o_input(qkv16)
                if self.switch is not None:
                    # partial output into the symmetric buffer, summed through the switch by the
                    # library's kernel on this side stream (a few CTAs; the other stream's GEMM
                    # keeps the remaining SMs busy)
                    part = self._switch_row_parallel(o_in, "o", 0, row0=a, channel=c % 2)
                    work = None
                else:
                    part = self._w4(o_in, "o", out_dtype=out_dt)
                    work = dist.all_reduce(part, op=dist.ReduceOp.SUM, async_op=True)
                stage1.append((part, work))
                keep += [qkv16, o_in]
        for c, (a, b) in enumerate(bounds):
            with torch.cuda.stream(self._streams[c % 2]):
                part, work = stage1[c]
                if work is not None:
                    work.wait()
                    attn_out[a:b].copy_(part)
                if self.switch is not None:
                    h = part       # fp16 sums: the 1/4 scaling is exact and rides in the gate/up GEMM
                    act = self._w4(h, "gate_up", epilogue="silu_mul", alpha=GLUE_SCALE, in_scale=GLUE_SCALE)
                else:
                    h = (part * GLUE_SCALE).to(torch.float16)
                    act = self._w4(h, "gate_up", epilogue="silu_mul", alpha=GLUE_SCALE)
                if self.switch is not None:
                    part2 = self._switch_row_parallel(act, "down", 1, row0=a, channel=2 + c % 2)
                    work2 = None
                else:
                    part2 = self._w4(act, "down", out_dtype=out_dt)
                    work2 = dist.all_reduce(part2, op=dist.ReduceOp.SUM, async_op=True)
                stage2.append((part2, work2))
                keep += [h, act]
        for c, (a, b) in enumerate(bounds):
            with torch.cuda.stream(self._streams[c % 2]):
                part2, work2 = stage2[c]
                if work2 is not None:
                    work2.wait()
                    mlp_out[a:b].copy_(part2)
        for st in self._streams:
            main.wait_stream(st)
        # the intermediates were allocated on the side streams: tell the allocator the main stream
        # (which now depends on them) may still be using them
        if self.switch is None:
            keep += [p for p, _ in stage1] + [p for p, _ in stage2]
        else:
            attn_out, mlp_out = self.switch.summed(0, T), self.switch.summed(1, T)
        for t in keep:
            t.record_stream(main)
        return attn_out, mlp_out

    def capture(self, x: torch.Tensor):
        """Captures forward(x) (GEMMs, glue and the NCCL all-reduces) into a CUDA graph and returns
        (replay, attn_out, mlp_out): calling replay() re-runs the layer on the current contents of
        `x` and refreshes the two output tensors. At 8 GPUs the per-rank kernels take tens of
        microseconds, less than the host needs to launch them one by one."""
        for _ in range(2):     # warm-up outside capture: lazy initialisation, workspaces, NCCL set-up
            self.forward(x)
        torch.cuda.synchronize(x.device)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            attn_out, mlp_out = self.forward(x)
        return graph.replay, attn_out, mlp_out

    __call__ = forward
