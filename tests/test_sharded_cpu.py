"""Shard plan and the multi-rank path of the sharded layer on CPU ranks (gloo, world size 2 and 3).
The GEMMs here are the oracle's (this is a test of the host logic: slicing, glue, all-reduce);
the GPU tests cover the kernels."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import int4, layer as olayer
from wmma_ops_b200 import sharded


def test_split_units_llama_ffn():
    # 11008 = 86 groups of 128
    assert [b - a for a, b in sharded.split_units(86, 2)] == [43, 43]
    assert [b - a for a, b in sharded.split_units(86, 4)] == [22, 22, 21, 21]
    assert [b - a for a, b in sharded.split_units(86, 8)] == [11] * 6 + [10] * 2
    for tp in (1, 2, 4, 8):
        r = sharded.split_units(86, tp)
        assert r[0][0] == 0 and r[-1][1] == 86
        assert all(r[i][1] == r[i + 1][0] for i in range(tp - 1))
    assert sharded.shard_range(11008, 7, 8) == (9728, 11008)
    assert sharded.shard_range(4096, 3, 8) == (1536, 2048)
    with pytest.raises(ValueError):
        sharded.shard_range(100, 0, 2)
    with pytest.raises(ValueError):
        sharded.split_units(3, 4)


def test_shards_tile_the_full_weights():
    shapes = sharded.LayerShapes(hidden=256, qkv_out=768, ffn=384, group=128)
    weights = olayer.make_layer_weights(seed=1, hidden=256, qkv_out=768, ffn=384, group=128)
    for world in (1, 2):
        shards = [sharded.shard_layer_weights(weights, r, world, shapes) for r in range(world)]
        # row-parallel shards stack back to the full matrix
        assert torch.equal(torch.cat([s["o"][0] for s in shards], 0), weights["o"][0])
        assert torch.equal(torch.cat([s["down"][0] for s in shards], 0), weights["down"][0])
        assert torch.equal(torch.cat([s["down"][1] for s in shards], 0), weights["down"][1])
        # column-parallel: gate and up halves use down's row partition
        for s in shards:
            assert s["gate_up"][0].shape[1] == 2 * s["down"][0].shape[0]
            assert s["qkv"][0].shape[1] == 3 * s["o"][0].shape[0]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, hidden, qkv_out, ffn, tokens, chunks, result, seq_len=None):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.set_num_threads(2)
        shapes = sharded.LayerShapes(hidden=hidden, qkv_out=qkv_out, ffn=ffn, group=128)
        weights = olayer.make_layer_weights(seed=1, hidden=hidden, qkv_out=qkv_out, ffn=ffn, group=128)
        local = sharded.shard_layer_weights(weights, rank, world, shapes)
        g = torch.Generator().manual_seed(5)
        x = torch.randn(tokens, hidden, generator=g).to(torch.float16)
        from oracle import attention as oattn
        layer = sharded.ShardedDecoderLinears(
            local, world=world, group=128, chunks=chunks,
            matmul=lambda a, name: int4.w4a16_ref(a, local[name][0], local[name][1], 128),
            attention=None if seq_len is None else (seq_len, True),
            attention_fn=lambda q, k, v, causal: oattn.attention_ref(q, k, v, causal))
        attn, mlp = layer(x)
        ref_attn, ref_mlp = olayer.layer_ref(x, weights, 128, seq_len=seq_len, causal=True)
        e1 = ((attn - ref_attn).norm() / ref_attn.norm()).item()
        e2 = ((mlp - ref_mlp).norm() / ref_mlp.norm()).item()
        result[rank] = (e1, e2)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,chunks", [(2, 1), (2, 2), (3, 1)])
def test_sharded_layer_gloo(world, chunks):
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        result = mgr.dict()
        port = _free_port()
        procs = [ctx.Process(target=_rank_main, args=(r, world, port, 384, 1152, 768, 512, chunks, result))
                 for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(180)
            assert p.exitcode == 0
        assert len(result) == world
        for r in range(world):
            e1, e2 = result[r]
            # sums of fp32 partials in a different order + one more fp16 rounding of activations
            assert e1 < 1e-3 and e2 < 2e-3, (r, e1, e2)


def test_sharded_layer_with_attention_gloo():
    # heads are cut by rank with the Q, K and V sections (3 heads of 128 on 3 ranks, one each): the
    # attention core between QKV and O needs no exchange and the result equals the unsharded oracle
    world = 3
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        result = mgr.dict()
        port = _free_port()
        procs = [ctx.Process(target=_rank_main, args=(r, world, port, 384, 1152, 768, 512, 1, result, 128))
                 for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(240)
            assert p.exitcode == 0
        for r in range(world):
            e1, e2 = result[r]
            assert e1 < 1e-3 and e2 < 2e-3, (r, e1, e2)
