"""The Python host layer raises the reference's errors (wmma_gemm.hip TORCH_CHECK texts)
before anything touches a GPU, and has no CPU fallback."""
import pytest
import torch

import wmma_ops
import wmma_ops_b200 as w

REFERENCE_NAMES = [
    # wmma_gemm.hip:2122-2155
    "matmul", "matmul_adaptive", "matmul_hilbert", "matmul_kunroll", "matmul_native", "matmul_zerocopy",
    "matmul_tiled", "matmul_quad", "matmul_highOcc", "matmul_noPrefetch", "matmul_asmOpt", "matmul_swizzled",
    "matmul_xor_optimized", "matmul_coop", "matmul_pingpong", "matmul_opt", "gemm", "gemm_inplace", "gemm_adaptive",
]


def test_drop_in_module_exports_reference_names():
    for name in REFERENCE_NAMES:
        assert callable(getattr(wmma_ops, name)), name
        assert getattr(wmma_ops, name) is getattr(w, name)


def test_cpu_tensors_are_rejected_not_computed():
    A = torch.randn(16, 16).half()
    B = torch.randn(16, 16).half()
    for name in REFERENCE_NAMES:
        fn = getattr(w, name)
        with pytest.raises(RuntimeError, match="must be (CUDA|GPU) tensors"):
            if name == "matmul_tiled":
                fn(A, B, 1)
            elif name == "gemm_inplace":
                fn(A, B, torch.zeros(16, 16))
            else:
                fn(A, B)


def test_gemm_keyword_signature():
    import inspect
    sig = inspect.signature(w.gemm)
    assert list(sig.parameters) == ["A", "B", "alpha", "beta", "C"]
    assert sig.parameters["alpha"].default == 1.0 and sig.parameters["beta"].default == 0.0
    assert sig.parameters["C"].default is None
    sig = inspect.signature(w.gemm_inplace)
    assert list(sig.parameters) == ["A", "B", "C", "alpha", "beta"]
    assert list(inspect.signature(w.gemm_adaptive).parameters) == ["A", "B", "alpha", "beta", "C"]


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from wmma_ops_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setenv("WMMA_OPS_B200_LIB", str(tmp_path / "nope.so"))
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        _lib.load()
    monkeypatch.delenv("WMMA_OPS_B200_LIB")
    monkeypatch.setattr(_lib, "_lib", None)
    _lib.load()
