"""Worker for tests/test_sharded_multi_gpu.py: run under torch.distributed.run with one rank per
GPU (NCCL). Every rank computes the sharded layer on 1024 tokens with full layer shapes; EVERY rank
compares its own copy of the all-reduced outputs with the single-process CPU oracle (rank 0
computes it and broadcasts it). The accuracy gate is the workload's, for every variant: relative
Frobenius error <= 1e-3 against the fp32 oracle (measured at 2 ranks: 5e-5 with fp32 sums, 3.0e-4 to
3.6e-4 with fp16 partial outputs, 2.1e-4 with fp32 partials and fp16 sums); the number is printed
either way.

A failure on one rank is recorded, not raised: every rank still reaches the final collectives and
releases its symmetric-memory buffers before the process group is destroyed, so that no rank exits
while its memory is bound to the multicast object and its peers wait on it."""
import os
import sys
import traceback
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

import wmma_ops_b200 as w  # noqa: E402
from oracle import gemm as og  # noqa: E402
from oracle import layer as olayer  # noqa: E402
from wmma_ops_b200 import sharded  # noqa: E402

GATE = 1e-3           # the workload's tolerance (attn_out and mlp_out)
FP16_PARTIALS = 1e-3  # partial outputs rounded to fp16 before the sum: measured 3.0e-4 .. 3.6e-4


def main():
    rank, local_rank, world = int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"]), int(os.environ["WORLD_SIZE"])
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    ok = True
    layer = sw16 = sw32 = None
    try:
        weights = olayer.make_layer_weights(seed=21)
        g = torch.Generator().manual_seed(5)
        T = 1024
        x = torch.randn(T, 4096, generator=g).to(torch.float16)
        refs = torch.empty((2, T, 4096), dtype=torch.float32, device=dev)
        if rank == 0:
            torch.set_num_threads(max(1, os.cpu_count() or 1))
            ra, rm = olayer.layer_ref(x, weights)
            refs[0].copy_(ra)
            refs[1].copy_(rm)
        dist.broadcast(refs, 0)
        ref_attn, ref_mlp = refs[0].cpu(), refs[1].cpu()
        local = {k: (c.to(dev), s.to(dev)) for k, (c, s) in sharded.shard_layer_weights(weights, rank, world).items()}
        del weights
        xd = x.to(dev)

        def check(label, layer, tol_attn, tol_mlp):
            attn, mlp = layer(xd)
            torch.cuda.synchronize()
            gave_up = 0.0
            try:
                w.check_status(dev)
            except RuntimeError as err:     # reported through the all-reduce below: no rank leaves the others in it
                gave_up = 1.0
                print(f"rank {rank} {label}: {err}", flush=True)
            errs = torch.tensor([og.rel_frobenius(attn.float().cpu(), ref_attn), og.rel_frobenius(mlp.float().cpu(), ref_mlp),
                                 gave_up], dtype=torch.float64, device=dev)
            dist.all_reduce(errs, op=dist.ReduceOp.MAX)       # every rank holds its own copy: the worst one counts
            e1, e2, bad = errs.tolist()
            if rank == 0:
                print(f"world={world} {label}: attn_err={e1:.2e} mlp_err={e2:.2e} (max over ranks)"
                      + (" A BOUNDED WAIT GAVE UP" if bad else ""), flush=True)
            return e1 < tol_attn and e2 < tol_mlp and not bad

        w.set_sm_margin(16)
        for rdt, chunks, tol in ((torch.float32, 1, GATE), (torch.float16, 1, FP16_PARTIALS), (torch.float16, 2, FP16_PARTIALS)):
            layer = sharded.ShardedDecoderLinears(local, world=world, reduce_dtype=rdt, chunks=chunks)
            ok = check(f"nccl reduce={rdt} chunks={chunks}", layer, tol, tol) and ok
            layer = None
        w.set_sm_margin(0)
        # the same layer with the partial outputs summed through the NVSwitch by the library's own
        # kernel (symmetric memory, barriers inside the kernel); skipped where the system offers no
        # NVLink multicast
        try:
            from wmma_ops_b200.collective import SwitchAllReduce
            sw16 = SwitchAllReduce(T, 4096, dev, partial_dtype=torch.float16)
            sw32 = SwitchAllReduce(T, 4096, dev, partial_dtype=torch.float32)
        except Exception as e:  # no symmetric memory / multicast
            sw16 = sw32 = None
            if rank == 0:
                print(f"switch all-reduce unavailable: {type(e).__name__}: {str(e)[:200]}", flush=True)
        if sw16 is not None:
            # margin: SMs the GEMMs leave to the sum kernel; 0 = its CTAs share SMs with the prefill kernel
            # margin: SMs the GEMMs leave to the sum kernel; 0 = its CTAs share SMs with the prefill kernel.
            # follow: the sum runs beside the GEMM that produces its input, token block by token block
            for label, sw, rdt, chunks, margin, follow, tol in (
                    ("switch fp32 partials", sw32, torch.float32, 1, 0, False, GATE),
                    ("switch fp16 partials", sw16, torch.float16, 1, 0, False, FP16_PARTIALS),
                    ("switch fp16 partials, 2 chunks, 32 SMs left", sw16, torch.float16, 2, 32, False, FP16_PARTIALS),
                    ("switch fp16 partials, 2 chunks, shared SMs", sw16, torch.float16, 2, 0, False, FP16_PARTIALS),
                    ("switch fp32 partials, 2 chunks, shared SMs", sw32, torch.float32, 2, 0, False, GATE),
                    ("switch fp16 partials, following, 32 SMs left", sw16, torch.float16, 1, 32, True, FP16_PARTIALS),
                    ("switch fp16 partials, following, shared SMs", sw16, torch.float16, 1, 0, True, FP16_PARTIALS),
                    ("switch fp32 partials, following, shared SMs", sw32, torch.float32, 1, 0, True, GATE),
                    ("switch fp16 partials, 2 chunks, following, shared SMs", sw16, torch.float16, 2, 0, True,
                     FP16_PARTIALS)):
                sw.max_ctas = 32 if (chunks > 1 or follow) else 0
                w.set_sm_margin(margin)
                layer = sharded.ShardedDecoderLinears(local, world=world, reduce_dtype=rdt, chunks=chunks, switch=sw,
                                                      follow=follow)
                for _ in range(2):      # twice: the barrier epochs advance, nothing is reset between calls
                    ok = check(label, layer, tol, tol) and ok
                layer = None
                sw.max_ctas = 0
                w.set_sm_margin(0)
            # Failure path, made without any fault: a following sum whose GEMM is never launched. Every CTA's
            # wait for its token block runs out (about a second), the kernel records {6, rank, CTA, block},
            # still meets the other ranks and returns; check_status raises and clears the counters, and the
            # next ordinary sum works.
            sw16.max_ctas = 8
            sw16.reduce_following(0, 512, 256, 32)
            torch.cuda.synchronize()
            try:
                w.check_status(dev)
                seen = ""
            except RuntimeError as err:
                seen = str(err)
            gave_up = "code=6" in seen and f"role={rank}" in seen
            if not gave_up:
                print(f"rank {rank}: expected the following sum to give up with code 6, saw '{seen}'", flush=True)
            ok = gave_up and ok
            ok = bool(sw16._blocks.abs().sum().item() == 0) and ok      # counters cleared by the reset hook
            sw16.max_ctas = 0
            layer = sharded.ShardedDecoderLinears(local, world=world, reduce_dtype=torch.float16, switch=sw16)
            ok = check("switch fp16 partials after a sum that gave up", layer, FP16_PARTIALS, FP16_PARTIALS) and ok
            layer = None
    except Exception:
        ok = False
        print(f"rank {rank} failed:\n{traceback.format_exc()}", flush=True)
    # every rank gets here, whatever happened above
    flag = torch.tensor([1 if ok else 0], device=dev)
    try:
        torch.cuda.synchronize()
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        layer = None
        sw16 = sw32 = None
        torch.cuda.synchronize()
        dist.barrier()
    finally:
        dist.destroy_process_group()
    passed = flag.item() == 1
    if rank == 0:
        print("SHARDED_PASS" if passed else "SHARDED_FAIL", flush=True)
    sys.exit(0 if passed else 1)


if __name__ == "__main__":
    main()
