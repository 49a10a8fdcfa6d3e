"""The sharded layer on one GPU: each rank's shard is computed in turn on the same device and the
partial outputs are summed on the host side of the test (ranks that wait on one another are never
run as separate launches on one GPU). Checks the kernels on shard shapes (1408/1280-column
tiles, K = 1408) and the plan, against the single-process oracle."""
import pytest
import torch

import wmma_ops_b200 as w
from oracle import gemm as og
from oracle import layer as olayer
from wmma_ops_b200 import sharded

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("world", [1, 8])
def test_layer_full_shapes_few_tokens(cuda, world):
    weights = olayer.make_layer_weights(seed=21)
    g = torch.Generator().manual_seed(5)
    x = torch.randn(192, 4096, generator=g).to(torch.float16)
    ref_attn, ref_mlp = olayer.layer_ref(x, weights)
    xd = x.to(cuda)
    layers = []
    for r in range(world):
        local = {k: (c.to(cuda), s.to(cuda)) for k, (c, s) in sharded.shard_layer_weights(weights, r, world).items()}
        layers.append(sharded.ShardedDecoderLinears(local, world=1))
    # emulate the two all-reduces by summing the ranks' partials (same fused calls the layer makes)
    G = sharded.GLUE_SCALE
    attn = None
    for layer in layers:
        qkv16 = layer._w4(xd, "qkv", out_dtype=torch.float16, alpha=G)
        part = layer._w4(qkv16[:, :layer.q_cols].contiguous(), "o")
        attn = part if attn is None else attn + part
    mlp = None
    h = (attn * G).half()
    for layer in layers:
        act = layer._w4(h, "gate_up", epilogue="silu_mul", alpha=G)
        assert act.shape == (192, layer.ffn_local) and act.dtype == torch.float16
        part = layer._w4(act, "down")
        mlp = part if mlp is None else mlp + part
    torch.cuda.synchronize()
    w.check_status()
    assert og.rel_frobenius(attn, ref_attn) < 1e-3
    assert og.rel_frobenius(mlp, ref_mlp) < 2e-3
    if world == 1:
        a2, m2 = layers[0](xd)
        torch.cuda.synchronize()
        assert torch.equal(a2, attn) and torch.equal(m2, mlp)


@pytest.mark.parametrize("shape", [("o", 512, 4096), ("down", 1408, 4096), ("down_short", 1280, 4096), ("qkv", 4096, 1536),
                                   ("gate_up", 4096, 2816)])
def test_shard_shaped_products_at_8192_tokens(cuda, shape):
    # one rank's products of the 8-way sharded layer at the workload's full token count, each against
    # the fp32 oracle: K = 512 (O), K = 1408 / 1280 (down: 11 or 10 groups of the 86), and the
    # column-parallel shards N = 3 x 512 and N = 2 x 1408
    from oracle import int4
    name, K, N = shape
    T = 8192
    codes, scales = int4.seeded_w4(K, N, 128, seed=61)
    g = torch.Generator().manual_seed(62)
    x = torch.randn(T, K, generator=g).to(torch.float16)
    ref = int4.w4a16_ref(x, codes, scales, 128)
    q, sc = w.int4_prepack(codes.to(cuda), scales.to(cuda), 128)
    xd = x.to(cuda)
    out = w.matmul_w4a16(xd, q, sc, 128)
    out16 = w.matmul_w4a16(xd, q, sc, 128, out_dtype=torch.float16, alpha=0.25)
    torch.cuda.synchronize()
    w.check_status()
    e32 = og.rel_frobenius(out, ref)
    e16 = og.rel_frobenius(out16.float(), 0.25 * ref)
    print(f"{name} [{T} x {K}] @ [{K} x {N}]: fp32 out {e32:.2e}, fp16 out {e16:.2e}")
    assert e32 < 1e-3 and e16 < 1e-3


@pytest.mark.parametrize("world", [1, 8])
def test_layer_with_attention_core(cuda, world):
    # the whole block: QKV, causal attention on each rank's own heads (4 of 32 at 8 ranks), O, gate/up,
    # down; ranks computed in turn on one device, sums emulated on the host side of the test
    seq, batch = 128, 2
    weights = olayer.make_layer_weights(seed=21)
    g = torch.Generator().manual_seed(6)
    x = torch.randn(batch * seq, 4096, generator=g).to(torch.float16)
    ref_attn, ref_mlp = olayer.layer_ref(x, weights, seq_len=seq, causal=True)
    xd = x.to(cuda)
    G = sharded.GLUE_SCALE
    layers = []
    for r in range(world):
        local = {k: (c.to(cuda), s.to(cuda)) for k, (c, s) in sharded.shard_layer_weights(weights, r, world).items()}
        layers.append(sharded.ShardedDecoderLinears(local, world=1, attention=(seq, True)))
    attn = None
    for layer in layers:
        qkv16 = layer._w4(xd, "qkv", out_dtype=torch.float16, alpha=G)
        part = layer._w4(layer._o_input(qkv16), "o")
        attn = part if attn is None else attn + part
    mlp = None
    h = (attn * G).half()
    for layer in layers:
        act = layer._w4(h, "gate_up", epilogue="silu_mul", alpha=G)
        part = layer._w4(act, "down")
        mlp = part if mlp is None else mlp + part
    torch.cuda.synchronize()
    w.check_status()
    e1, e2 = og.rel_frobenius(attn, ref_attn), og.rel_frobenius(mlp, ref_mlp)
    print(f"world={world}: attn_err {e1:.2e} mlp_err {e2:.2e}")
    assert e1 < 2e-3 and e2 < 3e-3        # the attention output is fp16: its rounding (2e-3 in the attention tests) rides along
    if world == 1:
        a2, m2 = layers[0](xd)
        torch.cuda.synchronize()
        assert torch.equal(a2, attn) and torch.equal(m2, mlp)
