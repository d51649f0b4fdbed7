"""Split-K launch planning (pure Python, no CUDA needed).

``plan_kivi_decode`` keeps the contract of the reference's
``src/phasekv/kernels/launch_config.py:23-64``: same arguments, same validation errors, same
returned ``DecodeLaunchConfig`` for every input (pinned by tests/golden/planner.json), so code
that inspects the plan keeps working.  ``block_n`` and ``num_warps`` are notions of the
reference's Triton kernels; the CUDA kernels accept them and treat them as advisory, while an
explicit ``num_splits`` is honoured exactly (``split_len = ceil(S / min(S, num_splits))``).
"""
from __future__ import annotations

from dataclasses import dataclass
from functools import lru_cache
from typing import Optional


@dataclass(frozen=True)
class DecodeLaunchConfig:
    num_splits: int
    split_len: int
    block_n: int
    num_warps: int


def _cdiv(a: int, b: int) -> int:
    return -(-a // b)


def _pow2_ceil(n: int) -> int:
    return 1 if n <= 1 else 1 << (n - 1).bit_length()


def _pow2_floor(n: int) -> int:
    return 1 << (n.bit_length() - 1)


@lru_cache(maxsize=2048)
def plan_kivi_decode(seq_len: int, num_heads: int, head_dim: int, sm_count: int,
                     num_splits: Optional[int] = None, block_n: Optional[int] = None,
                     num_warps: Optional[int] = None) -> DecodeLaunchConfig:
    """Plan one packed segment from its length, the head shape and the GPU size."""
    if seq_len <= 0 or num_heads <= 0 or head_dim <= 0 or sm_count <= 0:
        raise ValueError("sequence, heads, head_dim and SM count must be positive")
    if head_dim & (head_dim - 1):
        raise ValueError("head_dim must be a power of two")
    if num_splits is not None and num_splits <= 0:
        raise ValueError("num_splits must be positive")
    if block_n is not None and (block_n <= 0 or block_n & (block_n - 1)):
        raise ValueError("block_n must be a positive power of two")
    if num_warps is not None and num_warps not in (1, 2, 4, 8, 16, 32):
        raise ValueError("num_warps must be one of 1, 2, 4, 8, 16, 32")

    if block_n is None:
        # tiles of about 1024 elements, at most 32 tokens
        block_n = _pow2_floor(max(1, min(32, 1024 // head_dim, seq_len)))
    if num_warps is None:
        num_warps = min(32, max(4, _pow2_ceil(_cdiv(block_n * head_dim, 256))))

    if num_splits is None:
        tiles = _cdiv(seq_len, block_n)
        floor_blocks = _cdiv(4 * sm_count, num_heads)            # four blocks per SM to start
        cap = min(128, _pow2_ceil(_cdiv(32 * sm_count, num_heads)))  # at most 32 per SM / 128 splits
        wanted = min(tiles, cap, _pow2_ceil(max(floor_blocks, _cdiv(tiles, 16))))
        split_len = _cdiv(tiles, wanted) * block_n               # tile-aligned boundaries
    else:
        split_len = _cdiv(seq_len, min(seq_len, num_splits))
    return DecodeLaunchConfig(_cdiv(seq_len, split_len), split_len, block_n, num_warps)
