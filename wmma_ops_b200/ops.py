"""Host layer: the reference module's functions (wmma_gemm.hip:2120-2156, README.md:221-251)
with the same names, argument meaning and error messages, calling the sm_100a kernels
through the C ABI. torch supplies device memory and the current stream, nothing else.
"""
from __future__ import annotations

import ctypes
import os
import weakref
from typing import Optional, Tuple

import torch

from . import _lib

_DEBUG = os.environ.get("WMMA_OPS_DEBUG", "0") not in ("", "0")

_status_words: dict = {}
_workspaces: dict = {}


# --------------------------------------------------------------------------- plumbing
def _status_word(device: torch.device) -> torch.Tensor:
    key = (device.type, device.index)
    t = _status_words.get(key)
    if t is None:
        t = torch.zeros(4, dtype=torch.int32, device=device)
        _status_words[key] = t
    return t


def check_status(device=None) -> None:
    """Synchronises `device` and raises if a kernel's bounded wait gave up since the last check.

    A kernel that gives up may leave arrival counters of the zero-initialised W4A16 workspaces
    non-zero (only the last CTA to arrive resets them), so those workspaces of the device are
    cleared together with the status word before the error is raised."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    if device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    t = _status_word(device)
    vals = t.cpu().tolist()
    if vals[0] != 0:
        t.zero_()
        reset_workspaces(device)
        raise RuntimeError(
            f"wmma_ops_b200 kernel gave up waiting: code={vals[0]} role={vals[1]} block={vals[2]} detail={vals[3]}"
        )


_reset_hooks: "weakref.WeakSet" = weakref.WeakSet()


def _register_reset(obj) -> None:
    """obj.reset() is called (while obj lives) whenever reset_workspaces runs for obj.device."""
    _reset_hooks.add(obj)


def reset_workspaces(device) -> None:
    """Zero-fills every zero-initialised scratch buffer this module holds for `device` (W4A16
    partial sums and their arrival counters). Called after a non-zero status word."""
    device = torch.device(device)
    for (dtype, index, _stream_id, zero_init), bufs in _workspaces.items():
        if zero_init and dtype == device.type and index == device.index:
            for b in bufs:
                b.zero_()
    for obj in list(_reset_hooks):
        if torch.device(obj.device) == device:
            obj.reset()


def _workspace(device: torch.device, nbytes: int, zero_init: bool = False) -> torch.Tensor:
    """Scratch buffer (split-K partials; W4A16 partials and arrival counters) for the current
    stream of `device`.

    One buffer per (device, stream): kernels on different streams may overlap on the GPU and must
    not share partial sums or arrival counters; calls on one stream are ordered and may. A buffer
    that has been handed out is never freed (a kernel still running, or a captured CUDA graph, may
    hold its address): when a larger one is needed the old one is kept in the list. A buffer that is
    first needed while its stream is being captured is allocated there and then (torch serves it
    from the graph's memory pool; the reference kept here keeps it alive as long as the graph needs it)."""
    stream_id = torch.cuda.current_stream(device).cuda_stream
    key = (device.type, device.index, stream_id, zero_init)
    bufs = _workspaces.setdefault(key, [])
    if bufs and bufs[-1].numel() >= nbytes:
        return bufs[-1]
    size = max(nbytes, 1 << 20)
    t = torch.zeros(size, dtype=torch.uint8, device=device) if zero_init else torch.empty(
        size, dtype=torch.uint8, device=device)
    bufs.append(t)
    return t


class _NullGuard:
    def __enter__(self):
        return None

    def __exit__(self, *exc):
        return False


_NULL_GUARD = _NullGuard()


def _device_guard(device: torch.device):
    """torch.cuda.device(device), or nothing when it is the current device already (the context
    manager costs a few microseconds per call, as much as a small kernel)."""
    idx = device.index
    if idx is None or idx == torch.cuda.current_device():
        return _NULL_GUARD
    return torch.cuda.device(device)


def _stream(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _post(device: torch.device) -> None:
    if _DEBUG:
        check_status(device)


def _require(cond: bool, msg: str) -> None:
    if not cond:
        raise RuntimeError(msg)


# --------------------------------------------------------------------------- validation
def _check_ab(A, B, where: str = "CUDA") -> Tuple[torch.Tensor, torch.Tensor, int, int, int]:
    """The reference's TORCH_CHECK sequence (wmma_gemm.hip:1433-1446), same order and text.

    The device check is made for every entry point. The reference omits it in matmul_tiled and some
    variants (wmma_gemm.hip:1473-1480), where operands on two GPUs reach the kernel; here that would
    put another GPU's memory behind a TMA tensor map, so it is an error everywhere."""
    _require(isinstance(A, torch.Tensor) and isinstance(B, torch.Tensor), "Inputs must be tensors")
    _require(A.is_cuda and B.is_cuda, f"Inputs must be {where} tensors")
    _require(A.device == B.device, "Inputs must be on same device")
    _require(A.dtype == torch.float16 and B.dtype == torch.float16, "Inputs must be float16")
    _require(A.dim() == 2 and B.dim() == 2, "Inputs must be 2D")
    _require(A.size(1) == B.size(0), "Inner dimensions must match")
    return A, B, A.size(0), B.size(1), A.size(1)


def _finish_ab(A: torch.Tensor, B: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    A = A.contiguous()
    B = B.contiguous()
    _require(A.data_ptr() % 16 == 0, "A must be 16-byte aligned")
    _require(B.data_ptr() % 16 == 0, "B must be 16-byte aligned")
    return A, B


def _check_c(C: torch.Tensor, A: torch.Tensor, M: int, N: int) -> None:
    """wmma_gemm.hip:1916-1921."""
    _require(C.is_cuda, "C must be a CUDA tensor")
    _require(C.device == A.device, "C must be on same device as A and B")
    _require(C.dtype == torch.float32, "C must be float32")
    _require(C.dim() == 2, "C must be 2D")
    _require(C.size(0) == M and C.size(1) == N, "C dimensions must match output (M×N)")


# --------------------------------------------------------------------------- launch
def _launch_gemm(A, B, C_in, C_out, M, N, K, alpha, beta, tile_cfg, split_k) -> None:
    lib = _lib.load()
    dev = A.device
    with _device_guard(dev):
        ws_ptr, ws_bytes = None, 0
        if tile_cfg == _lib.TILE_AUTO and split_k == 0 and M > 0 and N > 0 and K > 0:
            cfg, sk = select_tile(M, N, K, _sm_count(dev))   # measured table first, then the cost model
            tile_cfg, split_k = cfg, sk
        if split_k > 1:
            need = lib.wmma_ops_gemm_workspace_bytes(M, N, K, split_k)
            ws = _workspace(dev, need)
            ws_ptr, ws_bytes = ws.data_ptr(), ws.numel()
        rc = lib.wmma_ops_gemm_f16f32(
            _ptr(A), _ptr(B), _ptr(C_in), _ptr(C_out), M, N, K, float(alpha), float(beta),
            int(tile_cfg), int(split_k), ws_ptr, ws_bytes, _status_word(dev).data_ptr(), _stream(dev))
        _lib.check(rc)
        _post(dev)


_sm_counts: dict = {}
_table_checked = False


def _sm_count(device: torch.device) -> int:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    n = _sm_counts.get(idx)
    if n is None:
        n = torch.cuda.get_device_properties(idx).multi_processor_count
        _sm_counts[idx] = n
    return n


def set_sm_margin(sms: int) -> None:
    """Leaves `sms` SMs free of this library's persistent kernels (process-wide), so that a
    collective running on another stream can overlap a GEMM."""
    _lib.check(_lib.load().wmma_ops_set_sm_margin(int(sms)))


def select_tile(M: int, N: int, K: int, num_sms: int = 148) -> Tuple[int, int]:
    """(tile_cfg, split_k) for an MxNxK product: the Blackwell counterpart of the reference's
    select_optimal_tile (wmma_tile_selection.hpp:30-66) and split_k::compute_config
    (wmma_xor_swizzle.hpp:293-332). Pure host arithmetic; works without a GPU."""
    global _table_checked
    if not _table_checked:
        # a measured tile table (WMMA_OPS_TILE_TABLE, or the one shipped with the package) takes
        # precedence over the built-in cost model for the shape buckets it holds
        _table_checked = True
        from . import tune
        tune.install_from_env()
    cfg = ctypes.c_int(0)
    sk = ctypes.c_int(0)
    _lib.check(_lib.load().wmma_ops_select_tile(M, N, K, num_sms, ctypes.byref(cfg), ctypes.byref(sk)))
    return cfg.value, sk.value


def _matmul_impl(A, B, tile_cfg: int, split_k: int, where: str = "CUDA", extra=None) -> torch.Tensor:
    A, B, M, N, K = _check_ab(A, B, where)
    if extra is not None:
        extra(M, N, K)
    A, B = _finish_ab(A, B)
    C = torch.empty((M, N), dtype=torch.float32, device=A.device)
    _launch_gemm(A, B, None, C, M, N, K, 1.0, 0.0, tile_cfg, split_k)
    return C


# --------------------------------------------------------------------------- matmul family
_DEFAULT_TILE = _lib.TILE_128x256


def _main_tile(A, B) -> int:
    """The tile of the main kernel: the 256x256 CTA pair when the product has at least one full
    pair tile, else the 1-CTA 128x256 tile."""
    try:
        return _lib.TILE_256x256_PAIR if A.size(0) >= 256 and B.size(1) >= 256 else _DEFAULT_TILE
    except Exception:
        return _DEFAULT_TILE


def matmul(A: torch.Tensor, B: torch.Tensor) -> torch.Tensor:
    """C = A @ B, fp16 inputs, fp32 output (wmma_matmul, wmma_gemm.hip:1432-1470).
    Fixed large tile, as the reference's matmul uses one fixed tile."""
    return _matmul_impl(A, B, _main_tile(A, B), 1)


def matmul_adaptive(A: torch.Tensor, B: torch.Tensor) -> torch.Tensor:
    """C = A @ B with the tile shape and split-K factor chosen from (M,N,K) for 148 SMs
    (wmma_matmul_adaptive, wmma_gemm.hip:1197-1263)."""
    return _matmul_impl(A, B, _lib.TILE_AUTO, 0)


_TILED_MAP = {0: _lib.TILE_128x64, 1: _lib.TILE_128x128, 2: _lib.TILE_128x256, 3: _lib.TILE_256x256_PAIR}


def matmul_tiled(A: torch.Tensor, B: torch.Tensor, tile_config: int) -> torch.Tensor:
    """C = A @ B with an explicit tile shape (wmma_matmul_tiled, wmma_gemm.hip:1473-1528).
    The reference's 0..3 (64x64, 128x64, 256x64, 128x128) select the four Blackwell tiles
    128x64, 128x128, 128x256 and the 256x256 CTA pair; other values raise the reference's error."""
    A, B, M, N, K = _check_ab(A, B, "CUDA")
    A, B = _finish_ab(A, B)
    if tile_config not in _TILED_MAP:
        raise RuntimeError("Invalid tile_config: 0=64x64, 1=128x64, 2=256x64, 3=128x128")
    C = torch.empty((M, N), dtype=torch.float32, device=A.device)
    _launch_gemm(A, B, None, C, M, N, K, 1.0, 0.0, _TILED_MAP[tile_config], 1)
    return C


def matmul_splitk(A: torch.Tensor, B: torch.Tensor, split_k: int = 0, tile_config: int = -1) -> torch.Tensor:
    """C = A @ B through the split-K path (K cut into slices, fp32 partials in a cached
    workspace, summed in ascending slice order). The reference implements this in
    wmma_xor_swizzle.hpp:1196-1219 but binds no Python name to it. split_k=0 lets the table choose."""
    A, B, M, N, K = _check_ab(A, B)
    A, B = _finish_ab(A, B)
    cfg = _TILED_MAP[tile_config] if tile_config in _TILED_MAP else _lib.TILE_AUTO
    _require(tile_config == -1 or tile_config in _TILED_MAP,
             "Invalid tile_config: 0=64x64, 1=128x64, 2=256x64, 3=128x128")
    C = torch.empty((M, N), dtype=torch.float32, device=A.device)
    if cfg == _lib.TILE_AUTO and split_k > 0:
        cfg, _ = select_tile(M, N, max(K, 1), _sm_count(A.device))
    _launch_gemm(A, B, None, C, M, N, K, 1.0, 0.0, cfg, split_k)
    return C


def _k16_n8_m16(M, N, K):
    _require(K % 16 == 0, f"K must be a multiple of 16 for WMMA (got K={K})")
    _require(N % 8 == 0, f"N must be a multiple of 8 for half8 vector loads (got N={N})")
    _require(M % 16 == 0, f"M must be a multiple of 16 for clean tiles (got M={M})")


def _k16(M, N, K):
    _require(K % 16 == 0, f"K must be a multiple of 16 for WMMA (got K={K})")


def matmul_pingpong(A, B):
    """Alias of the warp-specialised kernel with wmma_matmul_pingpong's checks (wmma_gemm.hip:1272-1292)."""
    return _matmul_impl(A, B, _DEFAULT_TILE, 1, where="GPU", extra=_k16_n8_m16)


def matmul_hilbert(A, B):
    """Alias with wmma_matmul_hilbert's checks (wmma_gemm.hip:1378-1398)."""
    return _matmul_impl(A, B, _DEFAULT_TILE, 1, where="GPU", extra=_k16_n8_m16)


def matmul_opt(A, B):
    """Alias with wmma_matmul_opt's checks (wmma_gemm.hip:1329-1347); large tile."""
    return _matmul_impl(A, B, _lib.TILE_128x256, 1, where="GPU", extra=_k16)


def matmul_kunroll(A, B):
    """Alias with wmma_matmul_kunroll's K % 32 check (wmma_gemm.hip:1606-1622)."""
    def extra(M, N, K):
        _require(K % 32 == 0, "K dimension must be a multiple of 32 for K-unrolled kernel")
    return _matmul_impl(A, B, _DEFAULT_TILE, 1, extra=extra)


def matmul_quad(A, B):
    """Alias with wmma_matmul_quad's K % 16 check (wmma_gemm.hip:1648-1664)."""
    def extra(M, N, K):
        _require(K % 16 == 0, "K dimension must be a multiple of 16 for quad-buffered kernel")
    return _matmul_impl(A, B, _DEFAULT_TILE, 1, extra=extra)


def matmul_native(A, B):
    """Alias (wmma_matmul_native, wmma_gemm.hip:1533-1566)."""
    return _matmul_impl(A, B, _DEFAULT_TILE, 1)


def matmul_zerocopy(A, B):
    """Alias (wmma_matmul_zerocopy, wmma_gemm.hip:1570-1603)."""
    return _matmul_impl(A, B, _DEFAULT_TILE, 1)


def matmul_highOcc(A, B):
    """Alias on the narrowest tile (wmma_matmul_highOcc, wmma_gemm.hip:1688-1724, is the reference's small-tile variant)."""
    return _matmul_impl(A, B, _lib.TILE_128x64, 1)


def matmul_noPrefetch(A, B):
    """Alias (wmma_matmul_noPrefetch, wmma_gemm.hip:1727-1765)."""
    return _matmul_impl(A, B, _DEFAULT_TILE, 1)


def matmul_asmOpt(A, B):
    """Alias (wmma_matmul_asmOpt, wmma_gemm.hip:1768-1804)."""
    return _matmul_impl(A, B, _DEFAULT_TILE, 1)


def matmul_swizzled(A, B):
    """Alias (wmma_matmul_swizzled, wmma_gemm.hip:1807-1842); the 128-byte hardware swizzle is always on."""
    return _matmul_impl(A, B, _DEFAULT_TILE, 1)


def matmul_xor_optimized(A, B):
    """Alias (wmma_matmul_xor_optimized, wmma_gemm.hip:1845-1888)."""
    return _matmul_impl(A, B, _DEFAULT_TILE, 1)


def matmul_coop(A, B):
    """Alias (wmma_matmul_coop, wmma_gemm.hip:2081-2117)."""
    return _matmul_impl(A, B, _DEFAULT_TILE, 1)


# --------------------------------------------------------------------------- gemm family
def _gemm_impl(A, B, alpha, beta, C, tile_cfg, split_k) -> torch.Tensor:
    A, B, M, N, K = _check_ab(A, B)
    A, B = _finish_ab(A, B)
    C_in = None
    if float(beta) != 0.0 and C is not None:
        _check_c(C, A, M, N)
        C_in = C.contiguous()
    C_out = torch.empty((M, N), dtype=torch.float32, device=A.device)
    _launch_gemm(A, B, C_in, C_out, M, N, K, alpha, beta, tile_cfg, split_k)
    return C_out


def gemm(A, B, alpha: float = 1.0, beta: float = 0.0, C: Optional[torch.Tensor] = None) -> torch.Tensor:
    """alpha * A @ B + beta * C into a new fp32 tensor (wmma_gemm, wmma_gemm.hip:1891-1945).
    C is read only when beta != 0 and C is given; beta != 0 with C=None yields alpha * A @ B."""
    return _gemm_impl(A, B, alpha, beta, C, _DEFAULT_TILE, 1)


def gemm_adaptive(A, B, alpha: float = 1.0, beta: float = 0.0, C: Optional[torch.Tensor] = None) -> torch.Tensor:
    """gemm with the tile chosen from the shape (wmma_gemm_adaptive, wmma_gemm.hip:1997-2078)."""
    return _gemm_impl(A, B, alpha, beta, C, _lib.TILE_AUTO, 0)


def gemm_inplace(A, B, C, alpha: float = 1.0, beta: float = 0.0) -> None:
    """C = alpha * A @ B + beta * C, written into C (wmma_gemm_inplace, wmma_gemm.hip:1949-1994).

    Deviation: the reference calls C.contiguous() and so writes into a temporary when C is
    not contiguous, leaving the caller's tensor unchanged (wmma_gemm.hip:1970); here that
    case raises instead of silently doing nothing."""
    _require(isinstance(C, torch.Tensor), "C must be a tensor")
    _require(A.is_cuda and B.is_cuda and C.is_cuda, "Inputs must be CUDA tensors")
    _require(A.device == B.device and A.device == C.device, "All tensors must be on same device")
    _require(A.dtype == torch.float16 and B.dtype == torch.float16, "A and B must be float16")
    _require(C.dtype == torch.float32, "C must be float32")
    _require(A.dim() == 2 and B.dim() == 2 and C.dim() == 2, "Inputs must be 2D")
    _require(A.size(1) == B.size(0), "Inner dimensions must match")
    M, K, N = A.size(0), A.size(1), B.size(1)
    _require(C.size(0) == M and C.size(1) == N, "C dimensions must match output (M×N)")
    _require(C.is_contiguous(), "C must be contiguous for in-place GEMM")
    A, B = _finish_ab(A, B)
    _launch_gemm(A, B, C, C, M, N, K, alpha, beta, _DEFAULT_TILE, 1)
    return None


# --------------------------------------------------------------------------- host-buffer GEMM
class _HostGemmState:
    """Device buffers, streams and events of matmul_host for one (device, M, N, K)."""

    def __init__(self, dev: torch.device, M: int, N: int, K: int, chunks: int):
        self.s_in = torch.cuda.Stream(device=dev)
        self.s_mm = torch.cuda.Stream(device=dev)
        self.s_out = torch.cuda.Stream(device=dev)
        self.bufs = [(torch.empty((M, K), dtype=torch.float16, device=dev),
                      torch.empty((K, N), dtype=torch.float16, device=dev),
                      torch.empty((M, N), dtype=torch.float32, device=dev)) for _ in range(2)]
        self.mm_done = [torch.cuda.Event() for _ in range(2)]    # the slot's A and B have been consumed
        self.out_done = [torch.cuda.Event() for _ in range(2)]   # the slot's C has been copied out
        self.ev_b = torch.cuda.Event()
        self.ev_a = [torch.cuda.Event() for _ in range(chunks)]
        self.ev_c = [torch.cuda.Event() for _ in range(chunks)]
        self.calls = 0


_host_gemm_states: dict = {}


def matmul_host(A: torch.Tensor, B: torch.Tensor, out: Optional[torch.Tensor] = None, chunks: int = 8,
                device: Optional[torch.device] = None, wait: bool = True) -> torch.Tensor:
    """C = A @ B for operands that live in (pinned) host memory: fp16 A [M,K] and B [K,N] in,
    fp32 C [M,N] out, also in pinned host memory. No counterpart in the reference (its callers
    move tensors themselves); this is the end-to-end form of matmul_adaptive.

    The copies and the GEMM are pipelined on three streams: B goes up first, then A in `chunks`
    row blocks; the product of a row block starts as soon as the block has arrived, and its rows
    of C go back down while the next block is still coming up, so the PCIe link is busy in both
    directions at once. Two sets of device buffers let consecutive calls overlap as well.
    A and B must be ready in host memory when the call is made. wait=False returns without
    synchronising the host: the caller's current stream is made to wait for the result, so `out` is
    complete for anything queued on that stream afterwards, or once that stream is synchronised."""
    _require(not A.is_cuda and not B.is_cuda, "matmul_host takes host tensors")
    _require(A.dtype == torch.float16 and B.dtype == torch.float16, "Inputs must be float16")
    _require(A.dim() == 2 and B.dim() == 2, "Inputs must be 2D")
    _require(A.size(1) == B.size(0), "Inner dimensions must match")
    _require(A.is_contiguous() and B.is_contiguous(), "matmul_host: inputs must be contiguous")
    _require(A.is_pinned() and B.is_pinned(), "matmul_host: inputs must be in pinned host memory")
    M, K = A.shape
    N = B.size(1)
    if out is None:
        out = torch.empty((M, N), dtype=torch.float32).pin_memory()
    _require(not out.is_cuda and out.dtype == torch.float32 and tuple(out.shape) == (M, N) and out.is_contiguous()
             and out.is_pinned(), "matmul_host: out must be a pinned, contiguous float32 host tensor [M, N]")
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    _lib.load()
    if M == 0 or N == 0:
        return out
    chunks = max(1, min(int(chunks), M // 256 if M >= 256 else 1))
    key = (dev.index, M, N, K, chunks)
    st = _host_gemm_states.get(key)
    if st is None:
        with torch.cuda.device(dev):
            st = _HostGemmState(dev, M, N, K, chunks)
        _host_gemm_states[key] = st
    slot = st.calls & 1
    st.calls += 1
    dA, dB, dC = st.bufs[slot]
    bounds = [(j * M // chunks, (j + 1) * M // chunks) for j in range(chunks)]
    with torch.cuda.device(dev):
        with torch.cuda.stream(st.s_in):
            st.s_in.wait_event(st.mm_done[slot])       # the GEMMs that read this slot two calls ago
            dB.copy_(B, non_blocking=True)
            st.ev_b.record(st.s_in)
            for j, (a, b) in enumerate(bounds):
                dA[a:b].copy_(A[a:b], non_blocking=True)
                st.ev_a[j].record(st.s_in)
        with torch.cuda.stream(st.s_mm):
            st.s_mm.wait_event(st.ev_b)
            st.s_mm.wait_event(st.out_done[slot])      # this slot's C of two calls ago has left
            for j, (a, b) in enumerate(bounds):
                st.s_mm.wait_event(st.ev_a[j])
                _launch_gemm(dA[a:b], dB, None, dC[a:b], b - a, N, K, 1.0, 0.0, _lib.TILE_AUTO, 0)
                st.ev_c[j].record(st.s_mm)
            st.mm_done[slot].record(st.s_mm)
        with torch.cuda.stream(st.s_out):
            for j, (a, b) in enumerate(bounds):
                st.s_out.wait_event(st.ev_c[j])
                out[a:b].copy_(dC[a:b], non_blocking=True)
            st.out_done[slot].record(st.s_out)
        # stream-ordered result: work queued on the caller's stream after this call sees `out` complete
        torch.cuda.current_stream(dev).wait_event(st.out_done[slot])
    if wait:
        st.out_done[slot].synchronize()
    return out
