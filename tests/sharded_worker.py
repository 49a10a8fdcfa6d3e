"""Worker for tests/test_sharded_multi_gpu.py: run under torch.distributed.run with one rank per
GPU (NCCL). Every rank computes the sharded layer on 256 tokens with full layer shapes and
compares the all-reduced outputs with the single-process CPU oracle."""
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

import wmma_ops_b200 as w  # noqa: E402
from oracle import gemm as og  # noqa: E402
from oracle import layer as olayer  # noqa: E402
from wmma_ops_b200 import sharded  # noqa: E402


def main():
    rank, local_rank, world = int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"]), int(os.environ["WORLD_SIZE"])
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    weights = olayer.make_layer_weights(seed=21)
    g = torch.Generator().manual_seed(5)
    x = torch.randn(1024, 4096, generator=g).to(torch.float16)
    local = {k: (c.to(dev), s.to(dev)) for k, (c, s) in sharded.shard_layer_weights(weights, rank, world).items()}
    ok = True
    w.set_sm_margin(16)
    for rdt, chunks, tol in ((torch.float32, 1, 1e-3), (torch.float16, 1, 3e-3), (torch.float16, 2, 3e-3)):
        layer = sharded.ShardedDecoderLinears(local, world=world, reduce_dtype=rdt, chunks=chunks)
        attn, mlp = layer(x.to(dev))
        torch.cuda.synchronize()
        w.check_status(dev)
        if rank == 0:
            ref_attn, ref_mlp = olayer.layer_ref(x, weights)
            e1 = og.rel_frobenius(attn.float(), ref_attn)
            e2 = og.rel_frobenius(mlp.float(), ref_mlp)
            print(f"world={world} reduce={rdt} attn_err={e1:.2e} mlp_err={e2:.2e}", flush=True)
            ok = ok and e1 < tol and e2 < 2 * tol
    # the same layer with the partial outputs summed through the NVSwitch by the library's own
    # multimem kernel (symmetric memory); skipped where the system offers no NVLink multicast
    try:
        from wmma_ops_b200.collective import SwitchAllReduce
        sw = SwitchAllReduce(1024, 4096, dev)
    except Exception as e:  # no symmetric memory / multicast
        sw = None
        if rank == 0:
            print(f"switch all-reduce unavailable: {type(e).__name__}: {str(e)[:200]}", flush=True)
    if sw is not None:
        for chunks in (1, 2):
            layer = sharded.ShardedDecoderLinears(local, world=world, reduce_dtype=torch.float16, chunks=chunks,
                                                  switch=sw)
            attn, mlp = layer(x.to(dev))
            torch.cuda.synchronize()
            w.check_status(dev)
            if rank == 0:
                ref_attn, ref_mlp = olayer.layer_ref(x, weights)
                e1 = og.rel_frobenius(attn.float(), ref_attn)
                e2 = og.rel_frobenius(mlp.float(), ref_mlp)
                print(f"world={world} switch chunks={chunks} attn_err={e1:.2e} mlp_err={e2:.2e}", flush=True)
                ok = ok and e1 < 3e-3 and e2 < 6e-3
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.broadcast(flag, 0)
    dist.barrier()
    dist.destroy_process_group()
    if rank == 0:
        print("SHARDED_PASS" if ok else "SHARDED_FAIL", flush=True)
    sys.exit(0 if flag.item() == 1 else 1)


if __name__ == "__main__":
    main()
