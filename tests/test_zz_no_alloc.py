"""The split-K entry point for callers that cannot allocate device memory
(wmma_ops_gemm_f16f32_splitk_static): called through the C ABI, twice in a row, and compared
with the ordinary entry point, which gets its workspace from the caller.

Who needs it: code that runs inside another framework's memory pool, plugins that receive only
their input and output buffers, and loops where an allocation's possible device-wide
synchronisation is not acceptable. The scratch lives in a fixed array inside the library, so the
test also checks that a second call, which finds the first call's partial sums still in that
array, gives the same answer, and that a product too large for the array is refused.

Collected last on purpose: a run that stops at the first failure has then already run every
other test."""
import ctypes

import pytest
import torch

from wmma_ops_b200 import _lib

pytestmark = pytest.mark.gpu
TOL = 1e-3   # relative Frobenius error, the tolerance of the other GEMM tests


def _rel(a, b):
    return ((a.double() - b.double()).norm() / b.double().norm()).item()


def test_static_scratch_matches_workspace_entry_point(cuda):
    lib = _lib.load()
    M, N, K, split = 256, 256, 16384, 8
    g = torch.Generator().manual_seed(123)
    A = (torch.randn(M, K, generator=g) * K ** -0.5).half().to(cuda)
    B = torch.randn(K, N, generator=g).half().to(cuda)
    B2 = torch.randn(K, N, generator=g).half().to(cuda)
    Cin = torch.randn(M, N, generator=g).to(cuda)
    status = torch.zeros(4, dtype=torch.int32, device=cuda)
    stream = torch.cuda.current_stream(cuda).cuda_stream
    need = lib.wmma_ops_gemm_workspace_bytes(M, N, K, split)
    assert need <= lib.wmma_ops_gemm_static_scratch_bytes()
    ws = torch.empty(need, dtype=torch.uint8, device=cuda)

    def reference_call(Bm, alpha, beta):
        out = torch.empty(M, N, dtype=torch.float32, device=cuda)
        rc = lib.wmma_ops_gemm_f16f32(A.data_ptr(), Bm.data_ptr(), Cin.data_ptr(), out.data_ptr(), M, N, K, alpha, beta,
                                      _lib.TILE_128x64, split, ws.data_ptr(), ws.numel(), status.data_ptr(), stream)
        _lib.check(rc)
        return out

    def static_call(Bm, alpha, beta):
        out = torch.empty(M, N, dtype=torch.float32, device=cuda)
        rc = lib.wmma_ops_gemm_f16f32_splitk_static(A.data_ptr(), Bm.data_ptr(), Cin.data_ptr(), out.data_ptr(), M, N, K,
                                                    alpha, beta, _lib.TILE_128x64, split, status.data_ptr(), stream)
        _lib.check(rc)
        return out

    # the property the entry point exists for: with the output preallocated, a call takes no device
    # memory from anybody (torch's allocator included) and the driver reports the same free memory
    pre_out = torch.empty(M, N, dtype=torch.float32, device=cuda)
    rc = lib.wmma_ops_gemm_f16f32_splitk_static(A.data_ptr(), B.data_ptr(), None, pre_out.data_ptr(), M, N, K, 1.0, 0.0,
                                                _lib.TILE_128x64, split, status.data_ptr(), stream)   # first call: address look-up
    _lib.check(rc)
    torch.cuda.synchronize()
    before = (torch.cuda.memory_allocated(cuda), torch.cuda.memory_reserved(cuda), torch.cuda.mem_get_info(cuda)[0])
    for _ in range(3):
        rc = lib.wmma_ops_gemm_f16f32_splitk_static(A.data_ptr(), B.data_ptr(), None, pre_out.data_ptr(), M, N, K, 1.0, 0.0,
                                                    _lib.TILE_128x64, split, status.data_ptr(), stream)
        _lib.check(rc)
    torch.cuda.synchronize()
    after = (torch.cuda.memory_allocated(cuda), torch.cuda.memory_reserved(cuda), torch.cuda.mem_get_info(cuda)[0])
    assert after == before

    # two calls in a row with different operands: the second finds the first one's partials in the array
    for Bm, alpha, beta in ((B, 1.0, 0.0), (B2, 2.0, 0.5)):
        got = static_call(Bm, alpha, beta)
        want = reference_call(Bm, alpha, beta)
        torch.cuda.synchronize()
        assert status.cpu().tolist()[0] == 0
        assert _rel(got, want) < TOL
        fp32 = alpha * (A.float() @ Bm.float()) + beta * Cin
        assert _rel(got, fp32) < TOL


def test_static_scratch_auto_plan_and_limit(cuda):
    lib = _lib.load()
    M, N, K = 256, 256, 4096
    g = torch.Generator().manual_seed(7)
    A = (torch.randn(M, K, generator=g) * K ** -0.5).half().to(cuda)
    B = torch.randn(K, N, generator=g).half().to(cuda)
    out = torch.empty(M, N, dtype=torch.float32, device=cuda)
    stream = torch.cuda.current_stream(cuda).cuda_stream
    rc = lib.wmma_ops_gemm_f16f32_splitk_static(A.data_ptr(), B.data_ptr(), None, out.data_ptr(), M, N, K, 1.0, 0.0,
                                                _lib.TILE_AUTO, 0, None, stream)
    _lib.check(rc)
    torch.cuda.synchronize()
    assert _rel(out, A.float() @ B.float()) < TOL
    # more slices asked for than there are 64-deep k-blocks: the size check sees the plan that will run
    # (M = N = 512, K = 256 has 4 k-blocks: 4 slices = 4 MiB fit, the 32 asked for would not)
    M2, K2 = 512, 256
    A2 = (torch.randn(M2, K2, generator=g) * K2 ** -0.5).half().to(cuda)
    B3 = torch.randn(K2, M2, generator=g).half().to(cuda)
    out2 = torch.empty(M2, M2, dtype=torch.float32, device=cuda)
    rc = lib.wmma_ops_gemm_f16f32_splitk_static(A2.data_ptr(), B3.data_ptr(), None, out2.data_ptr(), M2, M2, K2, 1.0, 0.0,
                                                _lib.TILE_128x128, 32, None, stream)
    _lib.check(rc)
    torch.cuda.synchronize()
    assert _rel(out2, A2.float() @ B3.float()) < TOL
    # 4 slices of 2048 x 2048 fp32 = 64 MiB > 8 MiB: refused before anything is launched
    rc = lib.wmma_ops_gemm_f16f32_splitk_static(None, None, None, None, 2048, 2048, 4096, 1.0, 0.0, _lib.TILE_128x128, 4,
                                                None, None)
    assert rc == _lib.ERR_WORKSPACE
    msg = _lib.last_error()
    assert "built-in scratch" in msg and str(lib.wmma_ops_gemm_static_scratch_bytes()) in msg
