"""GEMM parity on the GPU: the CUDA path through the C ABI against the CPU oracle.

Tolerance: relative Frobenius error <= 1e-3 against the fp32 oracle (the accuracy gate of the
benchmark configuration); the closed-form case must be exact."""
import numpy as np
import pytest
import torch

import wmma_ops_b200 as w
from oracle import gemm as og

pytestmark = pytest.mark.gpu
TOL = 1e-3


def _sync_ok():
    torch.cuda.synchronize()
    w.check_status()


def test_known_answer_exact(cuda):
    A, B, C = og.known_answer_case()   # test_fragment_loading.py:225-274
    for fn in (w.matmul, w.matmul_adaptive, w.matmul_asmOpt, lambda a, b: w.matmul_tiled(a, b, 0),
               lambda a, b: w.matmul_tiled(a, b, 1), lambda a, b: w.matmul_tiled(a, b, 3)):
        out = fn(A.to(cuda), B.to(cuda))
        _sync_ok()
        assert out.dtype == torch.float32 and out.shape == (64, 64)
        assert (out.cpu() - C).abs().max().item() == 0.0


def test_golden_fixture_cases(cuda, golden_dir):
    g = np.load(golden_dir / "gemm_golden.npz")
    for i in range(3):
        A = torch.from_numpy(g[f"s{i}_A"]).to(cuda)
        B = torch.from_numpy(g[f"s{i}_B"]).to(cuda)
        Cin = torch.from_numpy(g[f"s{i}_Cin"]).to(cuda)
        for t in range(4):
            out = w.matmul_tiled(A, B, t)
            _sync_ok()
            assert og.rel_frobenius(out, torch.from_numpy(g[f"s{i}_C"])) < TOL
        out = w.gemm(A, B, 2.0, 0.5, Cin)
        _sync_ok()
        assert og.rel_frobenius(out, torch.from_numpy(g[f"s{i}_C_a2b05"])) < TOL


@pytest.mark.parametrize("shape", og.REFERENCE_SEEDED_SHAPES[:4] + og.REFERENCE_SEEDED_SHAPES[5:])
def test_reference_seeded_shapes(cuda, shape):
    # the procedure of test_fragment_loading.py:67-130 (seed 42, fp32 oracle), all names that
    # the reference sweeps (test_rocwmma_patch.py:278-291) on the first shape
    M, N, K = shape
    A, B = og.seeded_ab(M, N, K, seed=42)
    ref = og.gemm_ref(A, B)
    names = ["matmul_asmOpt", "matmul"]
    if shape == og.REFERENCE_SEEDED_SHAPES[0]:
        names = ["matmul", "matmul_adaptive", "matmul_hilbert", "matmul_kunroll", "matmul_native", "matmul_zerocopy",
                 "matmul_quad", "matmul_highOcc", "matmul_noPrefetch", "matmul_asmOpt", "matmul_swizzled",
                 "matmul_xor_optimized", "matmul_coop", "matmul_pingpong", "matmul_opt"]
    for name in names:
        out = getattr(w, name)(A.to(cuda), B.to(cuda))
        _sync_ok()
        assert og.rel_frobenius(out, ref) < TOL, name
        assert og.reference_pass(out, ref), name


@pytest.mark.parametrize("shape", [(512, 512, 64), (2048, 2048, 128), (4096, 4096, 2048)])
def test_reference_correctness_script_shapes(cuda, shape):
    # test_rocwmma_patch.py:50-128: compared with torch's own fp16 matmul on the GPU,
    # pass if max-rel < 1e-3 or max-abs < 0.1 (0.5 for the large case)
    M, N, K = shape
    g = torch.Generator(device="cuda").manual_seed(9)
    A = torch.randn(M, K, generator=g, device=cuda).half()
    B = torch.randn(K, N, generator=g, device=cuda).half()
    C = w.matmul(A, B)
    ref = torch.matmul(A, B).float()
    _sync_ok()
    err = (C - ref).abs().max().item()
    assert err / ref.abs().max().item() < 1e-3 or err < (0.5 if K >= 2048 else 0.1)


def test_cross_kernel_agreement(cuda):
    # test_fragment_loading.py:175-222: matmul and matmul_asmOpt on 2048x2048x512
    A, B = og.seeded_ab(2048, 2048, 512, seed=10)
    a = w.matmul(A.to(cuda), B.to(cuda))
    b = w.matmul_asmOpt(A.to(cuda), B.to(cuda))
    c = w.matmul_tiled(A.to(cuda), B.to(cuda), 0)
    _sync_ok()
    ref = og.gemm_ref(A, B)
    assert og.rel_frobenius(a, ref) < TOL and og.rel_frobenius(b, ref) < TOL and og.rel_frobenius(c, ref) < TOL
    assert (a - c).abs().max().item() < 1e-2


def test_config1_512_cubed_alpha_beta_inplace(cuda):
    M = N = K = 512
    A, B = og.seeded_ab(M, N, K, seed=1)
    Cin = og.seeded_c(M, N, seed=2)
    ref = og.gemm_ref(A, B)
    out = w.matmul(A.to(cuda), B.to(cuda)); _sync_ok()
    assert og.rel_frobenius(out, ref) < TOL
    ref2 = og.gemm_alphabeta_ref(A, B, 2.0, 0.5, Cin)
    out = w.gemm(A.to(cuda), B.to(cuda), alpha=2.0, beta=0.5, C=Cin.to(cuda)); _sync_ok()
    assert og.rel_frobenius(out, ref2) < 1e-5        # the reference reports < 0.001 % (README.md:108)
    out = w.gemm_adaptive(A.to(cuda), B.to(cuda), alpha=2.0, beta=0.5, C=Cin.to(cuda)); _sync_ok()
    assert og.rel_frobenius(out, ref2) < 1e-5
    Cd = Cin.to(cuda).clone()
    assert w.gemm_inplace(A.to(cuda), B.to(cuda), Cd, 2.0, 0.5) is None
    _sync_ok()
    assert og.rel_frobenius(Cd, ref2) < 1e-5         # README.md:109
    # beta != 0 without C degrades to alpha * A @ B; beta == 0 ignores C (wmma_gemm.hip:1913, :656)
    out = w.gemm(A.to(cuda), B.to(cuda), alpha=2.0, beta=0.5); _sync_ok()
    assert og.rel_frobenius(out, 2.0 * ref) < TOL
    out = w.gemm(A.to(cuda), B.to(cuda), alpha=1.0, beta=0.0, C=torch.full((M, N), float("nan"), device=cuda)); _sync_ok()
    assert og.rel_frobenius(out, ref) < TOL


@pytest.mark.parametrize("shape", [(1024, 1024, 1024), (2048, 2048, 2048), (4096, 4096, 2048)])
def test_config2_sweep_small(cuda, shape):
    M, N, K = shape
    A, B = og.seeded_ab(M, N, K, seed=3, scale_by_k=True)
    ref = og.gemm_ref(A, B)
    for fn in (w.matmul, w.matmul_adaptive):
        out = fn(A.to(cuda), B.to(cuda)); _sync_ok()
        assert og.rel_frobenius(out, ref) < TOL


def test_config2_split_k_shape(cuda):
    M, N, K = 256, 256, 16384
    A, B = og.seeded_ab(M, N, K, seed=4, scale_by_k=True)
    ref = og.gemm_ref(A, B)
    cfg, sk = w.select_tile(M, N, K, 148)
    assert sk > 1
    out = w.matmul_adaptive(A.to(cuda), B.to(cuda)); _sync_ok()
    assert og.rel_frobenius(out, ref) < TOL
    for split in (2, 5, 32):
        for tile in (0, 1, 2):
            out = w.matmul_splitk(A.to(cuda), B.to(cuda), split, tile); _sync_ok()
            assert og.rel_frobenius(out, ref) < TOL, (split, tile)
    # split-K is deterministic: partials are summed in ascending slice order
    o1 = w.matmul_splitk(A.to(cuda), B.to(cuda), 8, 0)
    o2 = w.matmul_splitk(A.to(cuda), B.to(cuda), 8, 0)
    _sync_ok()
    assert torch.equal(o1, o2)


@pytest.mark.parametrize("shape", [(1, 8, 8), (1, 11008, 4096), (127, 72, 136), (129, 264, 72), (300, 520, 1000),
                                   (128, 256, 64), (64, 8, 16384), (2, 8, 24)])
def test_ragged_shapes(cuda, shape):
    # M arbitrary, N % 8 == 0, K % 8 == 0; tails are zero-filled by TMA
    M, N, K = shape
    A, B = og.seeded_ab(M, N, K, seed=5)
    ref = og.gemm_ref(A, B)
    for t in range(4):
        out = w.matmul_tiled(A.to(cuda), B.to(cuda), t); _sync_ok()
        assert og.rel_frobenius(out, ref) < TOL, t
    out = w.matmul_adaptive(A.to(cuda), B.to(cuda)); _sync_ok()
    assert og.rel_frobenius(out, ref) < TOL


def test_empty_and_zero_k(cuda):
    A = torch.empty(0, 64, dtype=torch.float16, device=cuda)
    B = torch.empty(64, 8, dtype=torch.float16, device=cuda)
    assert w.matmul(A, B).shape == (0, 8)
    A = torch.empty(16, 0, dtype=torch.float16, device=cuda)
    B = torch.empty(0, 8, dtype=torch.float16, device=cuda)
    out = w.matmul(A, B); _sync_ok()
    assert torch.equal(out, torch.zeros(16, 8, device=cuda))
    C = torch.ones(16, 8, device=cuda)
    out = w.gemm(A, B, 3.0, 0.5, C); _sync_ok()
    assert torch.equal(out, torch.full((16, 8), 0.5, device=cuda))


def test_errors_match_reference_text(cuda):
    A = torch.randn(64, 64, device=cuda).half()
    B = torch.randn(64, 64, device=cuda).half()
    with pytest.raises(RuntimeError, match="Inputs must be float16"):
        w.matmul(A.float(), B)
    with pytest.raises(RuntimeError, match="Inputs must be 2D"):
        w.matmul(A[None], B)
    with pytest.raises(RuntimeError, match="Inner dimensions must match"):
        w.matmul(A, B[:32])
    with pytest.raises(RuntimeError, match="Invalid tile_config: 0=64x64, 1=128x64, 2=256x64, 3=128x128"):
        w.matmul_tiled(A, B, 7)
    with pytest.raises(RuntimeError, match="K dimension must be a multiple of 32"):
        w.matmul_kunroll(A[:, :48], B[:48])
    with pytest.raises(RuntimeError, match="M must be a multiple of 16"):
        w.matmul_pingpong(A[:8], B)
    with pytest.raises(RuntimeError, match="C must be float32"):
        w.gemm(A, B, 1.0, 1.0, torch.zeros(64, 64, device=cuda, dtype=torch.float16))
    with pytest.raises(RuntimeError, match="C dimensions must match"):
        w.gemm(A, B, 1.0, 1.0, torch.zeros(64, 32, device=cuda))
    with pytest.raises(RuntimeError, match="must be a multiple of 8"):
        w.matmul(A[:, :60].contiguous(), B[:60])
    with pytest.raises(RuntimeError, match="contiguous"):
        w.gemm_inplace(A, B, torch.zeros(64, 128, device=cuda)[:, ::2], 1.0, 1.0)
    # non-contiguous inputs are made contiguous, as in the reference (wmma_gemm.hip:1439-1440)
    out = w.matmul(A.t(), B); _sync_ok()
    assert og.rel_frobenius(out, og.gemm_ref(A.t(), B)) < TOL


def test_linearity_and_full_size_property(cuda):
    # size-independent checks at the benchmark's full size (8192^3): linearity in A and a
    # row-sum identity  C @ 1 == A @ (B @ 1), with fp64 reduction on the device
    n = 8192
    g = torch.Generator(device="cuda").manual_seed(6)
    A = (torch.randn(n, n, generator=g, device=cuda) * n ** -0.5).half()
    B = torch.randn(n, n, generator=g, device=cuda).half()
    C = w.matmul(A, B)
    C2 = w.matmul((A * 2).half(), B)      # exact scaling by 2 in fp16
    _sync_ok()
    assert torch.equal(C2, 2 * C)
    rows = C.double().sum(dim=1)
    expect = A.double() @ B.double().sum(dim=1)
    assert ((rows - expect).norm() / expect.norm()).item() < 1e-4
    Ca = w.matmul_adaptive(A, B); _sync_ok()
    assert ((Ca - C).double().norm() / C.double().norm()).item() < 1e-5


@pytest.mark.parametrize("n", [4096, 8192])
def test_config2_large_squares_against_the_oracle(cuda, n):
    # the two large squares of the sweep compared element for element with the fp32 oracle on the
    # host (seeded inputs scaled by K^-1/2, as the config states); every public route to the kernel
    A, B = og.seeded_ab(n, n, n, seed=2000 + n, scale_by_k=True)
    ref = og.gemm_ref(A, B)
    Ad, Bd = A.to(cuda), B.to(cuda)
    for name, fn in (("matmul", w.matmul), ("matmul_adaptive", w.matmul_adaptive), ("matmul_tiled(2)", lambda a, b: w.matmul_tiled(a, b, 2))):
        C = fn(Ad, Bd)
        _sync_ok()
        err = og.rel_frobenius(C, ref)
        print(f"{name} {n}^3: rel Frobenius {err:.2e}")
        assert err < TOL
        del C


def test_matmul_host_pipelined_matches_device_matmul(cuda):
    # pinned host operands, row blocks pipelined over three streams; same kernel, same K order
    g = torch.Generator().manual_seed(41)
    A = (torch.randn(1536, 512, generator=g) / 8).half().pin_memory()
    B = torch.randn(512, 768, generator=g).half().pin_memory()
    ref = w.matmul_adaptive(A.to(cuda), B.to(cuda)).cpu()
    out = torch.empty((1536, 768), dtype=torch.float32).pin_memory()
    for chunks in (1, 3, 6):
        out.zero_()
        got = w.matmul_host(A, B, out=out, chunks=chunks)
        assert got is out
        assert og.rel_frobenius(out, ref) < 1e-6
    # back-to-back asynchronous calls reuse the two buffer sets correctly
    outs = [torch.empty((1536, 768), dtype=torch.float32).pin_memory() for _ in range(4)]
    for o in outs:
        w.matmul_host(A, B, out=o, wait=False)
    torch.cuda.synchronize()
    w.check_status()
    for o in outs:
        assert torch.equal(o, outs[0]) and og.rel_frobenius(o, ref) < 1e-6
    with pytest.raises(RuntimeError, match="pinned"):
        w.matmul_host(A.clone(), B)


def test_adaptive_is_near_the_best_fixed_tile(cuda):
    # With the measured tile table installed (the one that ships with the package, or the one named by
    # WMMA_OPS_TILE_TABLE), matmul_adaptive is within 5 % (plus 2 us of timing noise for the
    # launch-bound small products) of the best fixed (tile, split_k) on every shape the reference tunes
    # and reports on (autotune.py:64-82, benchmark_summary.py:10-19) and on the config shapes.
    from wmma_ops_b200 import tune
    from wmma_ops_b200.ops import _launch_gemm, select_tile
    tune.install_from_env(force=True)
    sms = torch.cuda.get_device_properties(cuda).multi_processor_count
    worst = []
    for (M, N, K) in tune.TUNE_SHAPES:
        res = tune.measure_shape(M, N, K, cuda)
        best_key = min(res, key=res.get)
        tile, split = select_tile(M, N, K, sms)
        chosen = res.get(f"{tile}:{split}")
        if chosen is None:      # a split factor outside the candidate list: time it the same way
            A, B = tune._operands(M, N, K, cuda, 1)[0]
            C = torch.empty((M, N), dtype=torch.float32, device=cuda)
            chosen = tune._time_us(lambda: _launch_gemm(A, B, None, C, M, N, K, 1.0, 0.0, tile, split), 20)
        ratio = chosen / res[best_key]
        print(f"{M}x{N}x{K}: adaptive {tune.TILE_NAMES[tile]}/{split} {chosen:.1f} us, best {best_key} {res[best_key]:.1f} us, x{ratio:.3f}")
        if chosen > 1.05 * res[best_key] + 2.0:
            worst.append((M, N, K, tile, split, chosen, best_key, res[best_key]))
    torch.cuda.synchronize()
    w.check_status()
    assert not worst, worst
