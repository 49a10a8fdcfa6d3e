"""Failure reporting on the GPU, without faulting or hanging it.

Every wait in the library's kernels is bounded and reports through a 4-int status word instead of
hanging. The production limit is about two seconds, so these tests use the library's self-test
kernel, whose single wait is on a barrier nobody arrives at and whose limit is a launch parameter:
the wait runs out after about a millisecond, the kernel returns normally, and the host reads
{code, role, block, detail}. check_status must raise on it, clear it, and re-zero the
zero-initialised workspaces (a kernel that gave up may have left arrival counters behind)."""
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

import wmma_ops_b200 as w
from wmma_ops_b200 import _lib, ops

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]


def test_bounded_wait_expires_and_reports(cuda):
    lib = _lib.load()
    status = torch.zeros(4, dtype=torch.int32, device=cuda)
    stream = torch.cuda.current_stream(cuda).cuda_stream
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    _lib.check(lib.wmma_ops_selftest_wait_expiry(2_000_000, 4242, status.data_ptr(), stream))   # ~1 ms of SM clocks
    t1.record()
    torch.cuda.synchronize()
    assert status.cpu().tolist() == [7, 77, 0, 4242]
    assert 0.2 < t0.elapsed_time(t1) < 200.0        # it waited, and it stopped waiting
    # the context is intact: an ordinary product still runs
    A = torch.randn(128, 64, device=cuda).half()
    B = torch.randn(64, 128, device=cuda).half()
    C = w.matmul(A, B)
    torch.cuda.synchronize()
    assert torch.allclose(C, A.float() @ B.float(), atol=1e-2)


def test_check_status_raises_clears_and_resets_workspaces(cuda):
    lib = _lib.load()
    w.check_status(cuda)                               # clean to begin with
    ws = ops._workspace(cuda, 4096, zero_init=True)    # a W4A16-style workspace with "counters"
    ws[:16] = 5                                        # as a kernel that gave up would leave them
    word = ops._status_word(cuda)
    _lib.check(lib.wmma_ops_selftest_wait_expiry(1_000_000, 17, word.data_ptr(), torch.cuda.current_stream(cuda).cuda_stream))
    with pytest.raises(RuntimeError, match=r"gave up waiting: code=7 role=77 block=0 detail=17"):
        w.check_status(cuda)
    assert word.cpu().tolist() == [0, 0, 0, 0]
    assert int(ws[:16].sum().item()) == 0
    w.check_status(cuda)                               # and stays clean


def test_limit_argument_is_validated(cuda):
    lib = _lib.load()
    status = torch.zeros(4, dtype=torch.int32, device=cuda)
    assert lib.wmma_ops_selftest_wait_expiry(10, 0, status.data_ptr(), None) == _lib.ERR_INVALID
    assert lib.wmma_ops_selftest_wait_expiry(1_000_000, 0, None, None) == _lib.ERR_INVALID


_DEBUG_SCRIPT = r"""
import sys, torch
sys.path.insert(0, {root!r})
import wmma_ops_b200 as w
from wmma_ops_b200 import _lib
lib = _lib.load()
assert lib.wmma_ops_debug_checks_enabled() == 1, "debug library not loaded"
dev = torch.device("cuda", 0)
# ordinary products under the index checks: nothing fires
A = torch.randn(300, 256, device=dev).half(); B = torch.randn(256, 264, device=dev).half()
C = w.matmul(A, B)
codes = torch.randint(0, 16, (512, 264), device=dev, dtype=torch.uint8)
scales = (torch.rand(4, 264, device=dev) * 0.019 + 0.001).half()
q, sc = w.int4_prepack(codes, scales, 128)
for M in (3, 16, 100):
    w.matmul_w4a16(A[:M, :].contiguous().repeat(1, 2)[:, :512].contiguous(), q, sc, 128)
Q = torch.randn(1, 2, 200, 128, device=dev).half()
w.flash_attention(Q, Q, Q, causal=True)
torch.cuda.synchronize(); w.check_status(dev)
assert torch.allclose(C, A.float() @ B.float(), atol=5e-2)
# the check itself: an index past the buffer is recorded and the store is skipped
out = torch.zeros(8, dtype=torch.int32, device=dev)
status = torch.zeros(4, dtype=torch.int32, device=dev)
_lib.check(lib.wmma_ops_selftest_debug_index(3, 8, out.data_ptr(), status.data_ptr(), None))
_lib.check(lib.wmma_ops_selftest_debug_index(11, 8, out.data_ptr(), status.data_ptr(), None))
torch.cuda.synchronize()
assert out.cpu().tolist() == [0, 0, 0, 1, 0, 0, 0, 0], out
assert status.cpu().tolist() == [9, 104, 0, 11], status
print("DEBUG_BUILD_OK")
"""


def test_debug_build_index_checks(cuda):
    # WMMA_OPS_DEBUG=1 loads the library built with device-side index checks (status-word writes,
    # skipped accesses, no traps) and synchronises after every call; run in a child process because
    # the choice of library is made at import
    res = subprocess.run([sys.executable, "-c", _DEBUG_SCRIPT.format(root=str(ROOT))], capture_output=True, text=True,
                         timeout=600, env={**os.environ, "WMMA_OPS_DEBUG": "1"})
    assert res.returncode == 0 and "DEBUG_BUILD_OK" in res.stdout, res.stdout[-2000:] + res.stderr[-2000:]


def test_release_build_has_no_index_checks(cuda):
    lib = _lib.load()
    if os.environ.get("WMMA_OPS_DEBUG", "0") not in ("", "0"):
        pytest.skip("debug library loaded")
    assert lib.wmma_ops_debug_checks_enabled() == 0
    out = torch.zeros(8, dtype=torch.int32, device=cuda)
    status = torch.zeros(4, dtype=torch.int32, device=cuda)
    _lib.check(lib.wmma_ops_selftest_debug_index(11, 8, out.data_ptr(), status.data_ptr(), None))
    torch.cuda.synchronize()
    assert int(out.sum().item()) == 0 and status.cpu().tolist() == [0, 0, 0, 0]   # store skipped, nothing recorded
