"""Restatement of the reference's host-side dispatch heuristics. TEST INFRASTRUCTURE.

These document what the reference picks on its AMD part; the B200 table is allowed to differ
(it is sized for 148 SMs), so tests use these to pin the oracle against the reference header
and to check invariants both plans share (every K-slice non-empty, >= 256 of K per slice,
at most 32 slices).
"""
from __future__ import annotations

from dataclasses import dataclass

# enum TileConfig (wmma_tile_selection.hpp:17-23)
SMALL_64x64, MEDIUM_128x64, LARGE_256x64, WIDE_128x128, K_UNROLL = 0, 1, 2, 3, 4


def select_optimal_tile_ref(M: int, N: int, K: int) -> int:
    """wmma_tile_selection.hpp:30-66, rule by rule and in the same order."""
    max_dim = max(M, N)
    aspect = float(M) / float(N)  # float32 in the reference; these comparisons are far from ties
    if max_dim < 512:
        return SMALL_64x64
    if aspect > 4.0 and M >= 4096:
        return SMALL_64x64
    if N >= 8192 and M >= 2048:
        return LARGE_256x64
    if 768 <= max_dim <= 1536 and K >= 512:
        return K_UNROLL
    return MEDIUM_128x64


@dataclass
class SplitKPlanRef:
    split_factor: int
    k_per_split: int
    workspace_size: int


def split_k_config_ref(M: int, N: int, K: int, block_m: int = 128, block_n: int = 64, block_k: int = 16,
                       num_cus: int = 40) -> SplitKPlanRef:
    """split_k::compute_config (wmma_xor_swizzle.hpp:293-332): target 4 tiles per CU, at most 32
    slices, at least 256 of K per slice, factor rounded up to a power of two."""
    base_tiles = -(-M // block_m) * -(-N // block_n)
    target = num_cus * 4
    if base_tiles >= target:
        return SplitKPlanRef(1, K, 0)
    sf = -(-target // base_tiles)
    sf = min(sf, 32)
    sf = min(sf, max(1, K // 256))
    p = 1
    while p < sf:
        p *= 2
    sf = p
    return SplitKPlanRef(sf, -(-K // sf), sf * M * N * 4)
