"""flash_attention parity on the GPU against the fp32 softmax-attention oracle.

Tolerance: the output is fp16, so relative Frobenius error <= 2e-3 and max-abs <= 4e-3 against
the oracle's fp16-rounded fp32 result (the reference's README quotes < 1e-3 max error against
SDPA for unit-variance inputs; fp16 rounding of O alone is up to 1e-3 at |O| ~ 1..2)."""
import numpy as np
import pytest
import torch

import wmma_ops_b200 as w
from oracle import attention as oa
from oracle import gemm as og

pytestmark = pytest.mark.gpu
REL_TOL = 2e-3
ABS_TOL = 4e-3


def _check(cuda, Q, K, V, causal, scale=-1.0):
    O = w.flash_attention(Q.to(cuda), K.to(cuda), V.to(cuda), causal=causal, scale=scale)
    torch.cuda.synchronize()
    w.check_status()
    assert O.dtype == torch.float16 and O.shape == Q.shape
    ref = oa.attention_ref(Q, K, V, causal, scale)
    assert og.rel_frobenius(O.float(), ref.float()) < REL_TOL
    assert (O.cpu().float() - ref.float()).abs().max().item() < ABS_TOL
    return O


def test_golden_fixture(cuda, golden_dir):
    g = np.load(golden_dir / "attention_golden.npz")
    Q, K, V = (torch.from_numpy(g[k]) for k in ("Q", "K", "V"))
    O = w.flash_attention(Q.to(cuda), K.to(cuda), V.to(cuda))
    Oc = w.flash_attention(Q.to(cuda), K.to(cuda), V.to(cuda), causal=True)
    torch.cuda.synchronize()
    w.check_status()
    assert (O.cpu().float() - torch.from_numpy(g["O"]).float()).abs().max().item() < ABS_TOL
    assert (Oc.cpu().float() - torch.from_numpy(g["O_causal"]).float()).abs().max().item() < ABS_TOL


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("S", [1, 80, 128, 200, 256, 1000])
@pytest.mark.parametrize("causal", [False, True])
def test_small_and_ragged_sequences(cuda, D, S, causal):
    Q, K, V = oa.seeded_qkv(1, 2, S, D, seed=3)
    _check(cuda, Q, K, V, causal)


def test_custom_scale_and_batch_heads(cuda):
    Q, K, V = oa.seeded_qkv(2, 3, 384, 128, seed=4)
    _check(cuda, Q, K, V, True, 0.1)
    _check(cuda, Q, K, V, False, 0.02)


def test_causal_first_row_is_first_value(cuda):
    Q, K, V = oa.seeded_qkv(1, 2, 300, 128, seed=5)
    O = _check(cuda, Q, K, V, True)
    assert torch.equal(O[:, :, 0].cpu(), V[:, :, 0])


def test_large_logits_do_not_overflow(cuda):
    Q, K, V = oa.seeded_qkv(1, 1, 256, 128, seed=6)
    _check(cuda, Q * 6, K * 6, V, False)     # logits of several hundred before the max subtraction


@pytest.mark.parametrize("causal", [False, True])
def test_config4_shape_s1024_against_oracle(cuda, causal):
    # B=4, H=32, S=1024, D=128: the oracle runs on a sample of heads to stay within seconds
    Q, K, V = oa.seeded_qkv(4, 32, 1024, 128, seed=7)
    O = w.flash_attention(Q.to(cuda), K.to(cuda), V.to(cuda), causal=causal)
    torch.cuda.synchronize()
    w.check_status()
    for b, h in [(0, 0), (1, 7), (3, 31)]:
        ref = oa.attention_ref(Q[b:b + 1, h:h + 1], K[b:b + 1, h:h + 1], V[b:b + 1, h:h + 1], causal)
        assert og.rel_frobenius(O[b:b + 1, h:h + 1].float(), ref.float()) < REL_TOL


@pytest.mark.parametrize("S", [2048, 4096])
def test_config4_full_size_properties(cuda, S):
    # size-independent properties at the benchmark sizes: (1) V constant along the sequence
    # => O equals that constant row whatever the softmax weights are; (2) heads are independent:
    # a slice of the batched call equals the call on the slice
    g = torch.Generator(device="cuda").manual_seed(8)
    Q = torch.randn(4, 32, S, 128, generator=g, device=cuda).half()
    K = torch.randn(4, 32, S, 128, generator=g, device=cuda).half()
    row = torch.randn(4, 32, 1, 128, generator=g, device=cuda).half()
    O = w.flash_attention(Q, K, row.expand(4, 32, S, 128).contiguous(), causal=True)
    torch.cuda.synchronize()
    w.check_status()
    assert (O.float() - row.float()).abs().max().item() < 2e-3
    V = torch.randn(4, 32, S, 128, generator=g, device=cuda).half()
    full = w.flash_attention(Q, K, V)
    part = w.flash_attention(Q[2:3, 5:6].contiguous(), K[2:3, 5:6].contiguous(), V[2:3, 5:6].contiguous())
    torch.cuda.synchronize()
    w.check_status()
    assert torch.equal(full[2:3, 5:6], part)
    ref = oa.attention_ref(Q[2:3, 5:6], K[2:3, 5:6], V[2:3, 5:6], False)
    assert og.rel_frobenius(part.float(), ref.float()) < REL_TOL


@pytest.mark.parametrize("S", [2048, 4096])
def test_config4_causal_long_sequences_against_oracle(cuda, S):
    # B=4, H=32, D=128 at the two long sequence lengths, causal and not, against the fp32 oracle on two
    # (batch, head) pairs each (the oracle materialises S x S scores per head)
    Q, K, V = oa.seeded_qkv(4, 32, S, 128, seed=70 + S)
    Qd, Kd, Vd = Q.to(cuda), K.to(cuda), V.to(cuda)
    for causal in (True, False):
        O = w.flash_attention(Qd, Kd, Vd, causal=causal)
        torch.cuda.synchronize()
        w.check_status()
        for b, h in [(0, 3), (3, 30)]:
            ref = oa.attention_ref(Q[b:b + 1, h:h + 1], K[b:b + 1, h:h + 1], V[b:b + 1, h:h + 1], causal)
            got = O[b:b + 1, h:h + 1].float()
            err = og.rel_frobenius(got, ref.float())
            print(f"S={S} causal={causal} (b={b}, h={h}): rel {err:.2e} max-abs {(got.cpu() - ref.float()).abs().max().item():.2e}")
            assert err < REL_TOL
            assert (got.cpu() - ref.float()).abs().max().item() < ABS_TOL


# ---- decode shapes: a few query rows against a longer key/value sequence --------------------------

def _seeded_decode(B, H, Sq, Skv, D, seed):
    g = torch.Generator().manual_seed(seed)
    mk = lambda S: torch.randn(B, H, S, D, generator=g, dtype=torch.float32).to(torch.float16)  # noqa: E731
    return mk(Sq), mk(Skv), mk(Skv)


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("shape", [(1, 2, 1, 1, 128), (1, 2, 1, 300, 128), (2, 3, 4, 1000, 64), (1, 4, 16, 4096, 128),
                                   (1, 2, 16, 16, 128), (2, 2, 7, 37, 128), (1, 1, 3, 257, 64), (3, 5, 9, 2050, 128)])
def test_decode_shapes_against_oracle(cuda, shape, causal):
    B, H, Sq, Skv, D = shape
    Q, K, V = _seeded_decode(B, H, Sq, Skv, D, seed=90 + Sq)
    O = w.flash_attention(Q.to(cuda), K.to(cuda), V.to(cuda), causal=causal)
    torch.cuda.synchronize()
    w.check_status()
    assert O.dtype == torch.float16 and O.shape == Q.shape
    ref = oa.attention_ref(Q, K, V, causal)        # the causal mask lets row i see keys 0 .. Skv - Sq + i
    assert og.rel_frobenius(O.float(), ref.float()) < REL_TOL
    assert (O.cpu().float() - ref.float()).abs().max().item() < ABS_TOL


def test_decode_config_shape_sampled_heads(cuda):
    # B=4, H=32, one new token against 4096 cached keys: the oracle on a sample of (batch, head) pairs
    Q, K, V = _seeded_decode(4, 32, 1, 4096, 128, seed=97)
    O = w.flash_attention(Q.to(cuda), K.to(cuda), V.to(cuda), causal=True)
    O2 = w.flash_attention(Q.to(cuda), K.to(cuda), V.to(cuda), causal=True)
    torch.cuda.synchronize()
    w.check_status()
    assert torch.equal(O, O2)            # splits are merged in a fixed order
    for b, h in [(0, 0), (2, 17), (3, 31)]:
        ref = oa.attention_ref(Q[b:b + 1, h:h + 1], K[b:b + 1, h:h + 1], V[b:b + 1, h:h + 1], True)
        assert og.rel_frobenius(O[b:b + 1, h:h + 1].float(), ref.float()) < REL_TOL


def test_decode_rows_equal_the_last_rows_of_prefill(cuda):
    # the last four query rows of a causal prefill see exactly what a four-row decode call sees
    Q, K, V = oa.seeded_qkv(2, 3, 384, 128, seed=98)
    full = w.flash_attention(Q.to(cuda), K.to(cuda), V.to(cuda), causal=True)
    last = w.flash_attention(Q[:, :, -4:].contiguous().to(cuda), K.to(cuda), V.to(cuda), causal=True)
    torch.cuda.synchronize()
    w.check_status()
    assert (full[:, :, -4:].float() - last.float()).abs().max().item() < 2e-3


def test_errors(cuda):
    Q = torch.randn(1, 2, 64, 128, device=cuda).half()
    with pytest.raises(RuntimeError, match="Inputs must be float16"):
        w.flash_attention(Q.float(), Q, Q)
    with pytest.raises(RuntimeError, match="4D"):
        w.flash_attention(Q[0], Q[0], Q[0])
    with pytest.raises(RuntimeError, match="head dimension"):
        w.flash_attention(Q[..., :32].contiguous(), Q[..., :32].contiguous(), Q[..., :32].contiguous())
    with pytest.raises(RuntimeError, match="CUDA tensors"):
        w.flash_attention(Q.cpu(), Q, Q)
    with pytest.raises(RuntimeError, match="may be longer than Q"):
        w.flash_attention(Q, torch.cat([Q, Q], dim=2), torch.cat([Q, Q], dim=2))      # 64 query rows against 128 keys
    with pytest.raises(RuntimeError, match="may be longer than Q"):
        w.flash_attention(torch.cat([Q, Q], dim=2)[:, :, :8].contiguous(), Q[:, :, :4].contiguous(), Q[:, :, :4].contiguous())
    assert w.flash_attention(Q[:, :0], Q[:, :0], Q[:, :0]).shape == (1, 0, 64, 128)


@pytest.mark.gpu
@pytest.mark.parametrize("causal", [False, True])
def test_attention_reads_packed_projections_in_place(causal):
    """Q, K and V as sections of one packed [tokens, 3, heads, D] projection output and a token-major output
    buffer, all passed as views: the same bits as the contiguous call, and nothing outside the buffer written."""
    torch.manual_seed(11)
    dev = torch.device("cuda", 0)
    B, S, H, D = 2, 640, 3, 128
    qkv = (torch.randn(B * S, 3 * H * D, device=dev) * 0.5).half()
    v5 = qkv.view(B, S, 3, H, D)
    q, k, v = (v5[:, :, i].permute(0, 2, 1, 3) for i in range(3))
    assert not q.is_contiguous()
    ref = w.flash_attention(q.contiguous(), k.contiguous(), v.contiguous(), causal)
    buf = torch.zeros(B * S * H * D + 16, dtype=torch.float16, device=dev)
    o = buf[8:8 + B * S * H * D].view(B, S, H, D)
    got = w.flash_attention(q, k, v, causal, out=o.permute(0, 2, 1, 3))
    w.check_status()
    assert got.data_ptr() == o.data_ptr()
    assert torch.equal(o.permute(0, 2, 1, 3), ref)
    assert torch.all(buf[:8] == 0) and torch.all(buf[8 + B * S * H * D:] == 0)
