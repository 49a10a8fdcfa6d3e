"""All-reduce of the sharded layer's row-parallel outputs through the NVSwitch.

The reference is single-GPU; this module belongs to the layer-shaped multi-GPU workload
(sharded.py). `SwitchAllReduce` owns a few fp16 buffers in symmetric memory (mapped on every rank
and bound to an NVLink multicast object by torch.distributed._symmetric_memory). A row-parallel
GEMM writes its partial output straight into such a buffer; `reduce()` then sums it over the ranks
in place with one launch of the library's multimem kernel per rank, bracketed by the symmetric
memory barrier. torch.distributed is used for the plumbing only (rendezvous, barrier).
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch

from . import _lib


class SwitchAllReduce:
    """`slots` buffers of `rows` x `cols` fp16 in symmetric memory, summed over `group` on demand.

    Raises RuntimeError if symmetric memory or NVLink multicast is not available (the caller then
    keeps torch.distributed.all_reduce)."""

    def __init__(self, rows: int, cols: int, device: torch.device, group=None, slots: int = 2,
                 max_ctas: int = 0):
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm

        if not dist.is_initialized():
            raise RuntimeError("SwitchAllReduce needs an initialised torch.distributed process group")
        self.group = group if group is not None else dist.group.WORLD
        self.rank = dist.get_rank(self.group)
        self.world = dist.get_world_size(self.group)
        self.rows, self.cols = rows, cols
        self.device = device
        self.max_ctas = max_ctas
        if (rows * cols) % 8 != 0:
            raise RuntimeError("SwitchAllReduce: rows * cols must be a multiple of 8")
        self._bufs: List[Tuple[torch.Tensor, object]] = []
        for _ in range(slots):
            t = symm.empty((rows, cols), dtype=torch.float16, device=device)
            try:
                hdl = symm.rendezvous(t, self.group)
            except TypeError:
                hdl = symm.rendezvous(t, self.group.group_name)
            if not getattr(hdl, "multicast_ptr", 0):
                raise RuntimeError("SwitchAllReduce: this system gives no NVLink multicast address")
            self._bufs.append((t, hdl))
        self._lib = _lib.load()

    def buffer(self, slot: int, rows: Optional[int] = None) -> torch.Tensor:
        """The first `rows` rows of buffer `slot`: the tensor a GEMM writes its partial output to."""
        t = self._bufs[slot][0]
        return t if rows is None else t[:rows]

    def reduce(self, slot: int, rows: Optional[int] = None, row0: int = 0, channel: Optional[int] = None) -> torch.Tensor:
        """Sums rows [row0, row0 + rows) of buffer `slot` over the ranks, in place on every rank, on
        the current stream. All ranks must call it with the same arguments. Calls that may be in
        flight at the same time on different streams need different barrier channels."""
        t, hdl = self._bufs[slot]
        rows = self.rows - row0 if rows is None else rows
        n = rows * self.cols
        if n % 8 != 0 or (row0 * self.cols) % 8 != 0:
            raise RuntimeError("SwitchAllReduce.reduce: the row range must be a multiple of 8 values")
        if row0 < 0 or row0 + rows > self.rows:
            raise RuntimeError("SwitchAllReduce.reduce: row range outside the buffer")
        channel = slot if channel is None else channel
        stream = torch.cuda.current_stream(self.device).cuda_stream
        hdl.barrier(channel=channel)     # every rank's partial output is written
        rc = self._lib.wmma_ops_multimem_allreduce_f16(hdl.multicast_ptr + row0 * self.cols * 2, n, self.rank,
                                                       self.world, self.max_ctas, stream)
        _lib.check(rc)
        hdl.barrier(channel=channel)     # every rank's slice is stored everywhere
        return t[row0:row0 + rows]
