"""All-reduce of the sharded layer's row-parallel outputs through the NVSwitch.

The reference is single-GPU; this module belongs to the layer-shaped multi-GPU workload
(sharded.py). `SwitchAllReduce` owns buffers in symmetric memory (mapped on every rank and bound to
an NVLink multicast object by torch.distributed._symmetric_memory). A row-parallel GEMM writes its
partial output straight into such a buffer; `reduce()` then sums it over the ranks with ONE launch
of the library's kernel per rank: the rank barriers before and after the reduction are flags in
symmetric memory that the kernel itself writes and polls (bounded), the sum is done by the switch
(multimem.ld_reduce, fp32 accumulation) and stored to all ranks (multimem.st).
torch.distributed is used for the plumbing only (rendezvous, one barrier at set-up).

Two forms of partial output:
  fp16  the GEMM writes half(acc); the buffer is summed in place. Cheapest on the links (the buffer
        once out and once in per GPU), costs one fp16 rounding of every partial output.
  fp32  the GEMM writes its fp32 accumulators; the sums are written as fp16 to a second buffer.
        Twice the bytes on the way in, no rounding before the sum.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch

from . import _lib
from .ops import _register_reset, _status_word


class SwitchAllReduce:
    """`slots` buffers of `rows` x `cols` partial outputs in symmetric memory, summed over `group`
    on demand. Raises RuntimeError if symmetric memory or NVLink multicast is not available (the
    caller then keeps torch.distributed.all_reduce)."""

    def __init__(self, rows: int, cols: int, device: torch.device, group=None, slots: int = 2,
                 max_ctas: int = 0, partial_dtype: torch.dtype = torch.float16):
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm

        if not dist.is_initialized():
            raise RuntimeError("SwitchAllReduce needs an initialised torch.distributed process group")
        if partial_dtype not in (torch.float16, torch.float32):
            raise RuntimeError("SwitchAllReduce: partial outputs are float16 or float32")
        self.group = group if group is not None else dist.group.WORLD
        self.rank = dist.get_rank(self.group)
        self.world = dist.get_world_size(self.group)
        self.rows, self.cols = rows, cols
        self.device = device
        self.max_ctas = max_ctas
        self.partial_dtype = partial_dtype
        if (rows * cols) % 8 != 0 or cols % 8 != 0:
            raise RuntimeError("SwitchAllReduce: cols must be a multiple of 8")
        self._lib = _lib.load()

        def shared(shape, dtype):
            t = symm.empty(shape, dtype=dtype, device=device)
            try:
                hdl = symm.rendezvous(t, self.group)
            except TypeError:
                hdl = symm.rendezvous(t, self.group.group_name)
            return t, hdl

        # arrival flags and per-CTA epochs of the kernel's rank barriers: zero once, never reset
        n_flag = self._lib.wmma_ops_switch_allreduce_flag_bytes() // 4
        self._flags, self._flag_hdl = shared((n_flag,), torch.int32)
        self._flags.zero_()
        self._partial: List[Tuple[torch.Tensor, object]] = []
        self._summed: List[Tuple[torch.Tensor, object]] = []
        for _ in range(slots):
            t, hdl = shared((rows, cols), partial_dtype)
            if not getattr(hdl, "multicast_ptr", 0):
                raise RuntimeError("SwitchAllReduce: this system gives no NVLink multicast address")
            self._partial.append((t, hdl))
            self._summed.append(shared((rows, cols), torch.float16) if partial_dtype == torch.float32 else (t, hdl))
        # per slot: tile counters a GEMM advances per token block, and how many CTAs of the following sum
        # have seen a block complete; both return to zero by themselves (see reduce_following)
        self._blocks = torch.zeros((slots, 2, rows // 32 + 2), dtype=torch.int32, device=device)
        _register_reset(self)
        torch.cuda.synchronize(device)
        dist.barrier(self.group)      # every rank's flags are zero before any peer writes to them

    def buffer(self, slot: int, rows: Optional[int] = None) -> torch.Tensor:
        """The first `rows` rows of the partial-output buffer `slot`: what a GEMM writes to."""
        t = self._partial[slot][0]
        return t if rows is None else t[:rows]

    def summed(self, slot: int, rows: Optional[int] = None) -> torch.Tensor:
        """The first `rows` rows of the fp16 sums of buffer `slot` (what reduce() last produced there)."""
        t = self._summed[slot][0]
        return t if rows is None else t[:rows]

    def reduce(self, slot: int, rows: Optional[int] = None, row0: int = 0, channel: Optional[int] = None) -> torch.Tensor:
        """Sums rows [row0, row0 + rows) of buffer `slot` over the ranks on the current stream and
        returns the fp16 sums (a view of symmetric memory, valid until the slot is written again).
        All ranks must call it with the same arguments. Calls that may be in flight at the same
        time on different streams need different channels (0..3)."""
        part, phdl = self._partial[slot]
        out, ohdl = self._summed[slot]
        rows = self.rows - row0 if rows is None else rows
        n = rows * self.cols
        if row0 < 0 or rows < 0 or row0 + rows > self.rows:
            raise RuntimeError("SwitchAllReduce.reduce: row range outside the buffer")
        channel = slot if channel is None else channel
        stream = torch.cuda.current_stream(self.device).cuda_stream
        f32 = self.partial_dtype == torch.float32
        off = row0 * self.cols
        rc = self._lib.wmma_ops_switch_allreduce(
            phdl.multicast_ptr + off * (4 if f32 else 2), ohdl.multicast_ptr + off * 2, n, 1 if f32 else 0, self.rank,
            self.world, self._flag_hdl.buffer_ptrs_dev, channel, self.max_ctas, _status_word(self.device).data_ptr(), stream)
        _lib.check(rc)
        return out[row0:row0 + rows]

    def counters(self, slot: int, row0: int = 0) -> torch.Tensor:
        """Tile counters for a GEMM that writes rows [row0, ...) of buffer `slot` and is to be followed by
        reduce_following: pass them as matmul_w4a16(..., block_done=...)."""
        if row0 % 32 != 0:
            raise RuntimeError("SwitchAllReduce.counters: row0 must be a multiple of 32")
        return self._blocks[slot, 0, row0 // 32:]

    def reduce_following(self, slot: int, rows: int, token_block: int, tiles_per_block: int, row0: int = 0,
                         channel: Optional[int] = None) -> torch.Tensor:
        """reduce() for a buffer that a GEMM of this rank is still writing on ANOTHER stream, token block by
        token block (matmul_w4a16 with block_done=counters(slot, row0)): on the current stream, sums each
        block of `token_block` rows as soon as every rank's GEMM has counted `tiles_per_block` column tiles
        for it. The caller launches the GEMM first, then this, and joins the two streams afterwards."""
        part, phdl = self._partial[slot]
        out, ohdl = self._summed[slot]
        if row0 < 0 or rows < 1 or row0 + rows > self.rows or row0 % 32 != 0:
            raise RuntimeError("SwitchAllReduce.reduce_following: row range outside the buffer or row0 not a multiple of 32")
        channel = slot if channel is None else channel
        stream = torch.cuda.current_stream(self.device).cuda_stream
        f32 = self.partial_dtype == torch.float32
        off = row0 * self.cols
        done = self._blocks[slot, 0, row0 // 32:]
        seen = self._blocks[slot, 1, row0 // 32:]
        rc = self._lib.wmma_ops_switch_allreduce_following(
            phdl.multicast_ptr + off * (4 if f32 else 2), ohdl.multicast_ptr + off * 2, rows, self.cols, 1 if f32 else 0,
            token_block, done.data_ptr(), seen.data_ptr(), tiles_per_block, self.rank, self.world,
            self._flag_hdl.buffer_ptrs_dev, channel, self.max_ctas, _status_word(self.device).data_ptr(), stream)
        _lib.check(rc)
        return out[row0:row0 + rows]

    def reset(self) -> None:
        """After a non-zero status word: the tile counters may have been left behind."""
        self._blocks.zero_()
