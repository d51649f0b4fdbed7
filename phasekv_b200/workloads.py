"""Seeded synthetic inputs for the decode-attention path.

The reference's own micro-benchmarks draw K, V and q from ``torch.randn``
(scripts/bench_decode_kernel.py:72-74, scripts/bench_phasekv_launch.py:55-57); the
tensors made here stand in for them.  Everything is generated on the CPU from an
explicit ``torch.Generator`` so that a CPU checker and the GPU see identical bits.

K carries four fixed outlier channels scaled by 8 (the channel-wise outliers that
motivate per-channel key quantisation in KIVI-style caches).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Tuple

import torch

#: frozen outlier channels per head_dim
OUTLIER_CHANNELS: Dict[int, Tuple[int, ...]] = {
    8: (1, 6),
    64: (3, 17, 29, 50),
    128: (5, 40, 77, 100),
    256: (5, 40, 177, 200),
}
OUTLIER_GAIN = 8.0


@dataclass(frozen=True)
class Shape:
    """Attention shape of one transformer layer."""

    name: str
    num_q_heads: int
    num_kv_heads: int
    head_dim: int
    num_layers: int


QWEN2_0_5B = Shape("qwen2-0.5b", 14, 2, 64, 24)
QWEN2_5_7B = Shape("qwen2.5-7b", 28, 4, 128, 28)


def make_kv(gen: torch.Generator, num_kv_heads: int, length: int, head_dim: int,
            batch: int = 1) -> Tuple[torch.Tensor, torch.Tensor]:
    """K, V ~ N(0, 1) as float16 ``[batch, Hkv, length, hd]``; K gets the outlier channels."""
    k = torch.randn(batch, num_kv_heads, length, head_dim, generator=gen).half()
    v = torch.randn(batch, num_kv_heads, length, head_dim, generator=gen).half()
    for c in OUTLIER_CHANNELS.get(head_dim, ()):
        k[..., c] = (k[..., c].float() * OUTLIER_GAIN).half()
    return k, v


def make_query(gen: torch.Generator, num_q_heads: int, head_dim: int, batch: int = 1) -> torch.Tensor:
    """q ~ N(0, 1) as float16 ``[batch, Hq, 1, hd]``."""
    return torch.randn(batch, num_q_heads, 1, head_dim, generator=gen).half()


def three_tier_dense(seed: int, shape: Shape, prompt_len: int, cold_len: int, hot_len: int):
    """Dense float16 tiers in the fixed draw order prompt, cold, hot, then q.

    Returns ``((pk, pv), (ck, cv), (hk, hv), q)``; an empty tier is ``(None, None)``.
    """
    gen = torch.Generator().manual_seed(seed)
    tiers = []
    for length in (prompt_len, cold_len, hot_len):
        tiers.append(make_kv(gen, shape.num_kv_heads, length, shape.head_dim) if length > 0
                     else (None, None))
    q = make_query(gen, shape.num_q_heads, shape.head_dim)
    return tiers[0], tiers[1], tiers[2], q


def layer_seed(seed: int, layer: int, seq: int = 0) -> int:
    """Distinct, reproducible seed per (layer, sequence); plain arithmetic, no ``hash``."""
    return seed * 1_000_003 + layer * 1009 + seq


def jittered_lengths(seed: int, num_seqs: int, prompt: int, cold: int, hot: int,
                     jitter: float = 0.25, hot_capacity: int | None = None):
    """Per-sequence (prompt, cold, hot) lengths scaled by ``1 + u``, ``u ~ U(-jitter, jitter)``."""
    gen = torch.Generator().manual_seed(seed)
    u = (torch.rand(num_seqs, generator=gen) * 2.0 - 1.0) * jitter
    out = []
    for i in range(num_seqs):
        f = 1.0 + float(u[i])
        h = max(1, round(hot * f))
        if hot_capacity is not None:
            h = min(h, hot_capacity)
        out.append((max(1, round(prompt * f)), max(1, round(cold * f)), h))
    return out


def decode_algorithmic_bytes(shape: Shape, prompt_len: int, prompt_bits: int, cold_len: int,
                             cold_bits: int, hot_len: int, k_group: int = 32, v_group: int = 32) -> int:
    """Bytes one decode-attention call must move for one layer of one sequence.

    Per token and KV head a packed tier holds ``2*hd*bits/8`` code bytes plus
    ``4*hd/k_group + 4*hd/v_group`` bytes of float16 scale and zero; the hot tier holds
    ``4*hd``.  q is read and o written once (float16).  Split-K partials are excluded.
    """
    hd, hkv, hq = shape.head_dim, shape.num_kv_heads, shape.num_q_heads

    def bpt(bits: int) -> float:
        return 2 * hd * bits / 8 + 4 * hd / k_group + 4 * hd / v_group

    total = hkv * (prompt_len * bpt(prompt_bits) + cold_len * bpt(cold_bits) + hot_len * 4 * hd)
    total += 2 * hq * hd * 2
    return int(total)


def gpu_three_tier(shape: Shape, prompt_len: int, prompt_bits: int, cold_len: int, cold_bits: int,
                   hot_len: int, seed: int, device, group: int = 32, hot_capacity: int | None = None):
    """One sequence's packed three-tier KV of one layer, drawn and packed on ``device`` (same
    distribution as the CPU generators, different bits: for timing and for rows that need no CPU
    checker).  Returns ``(LayerTiers, q float16 [Hq, hd])``."""
    from .kernels import packing
    from .kernels.tiers import LayerTiers, PackedKVSegment
    gen = torch.Generator(device=device).manual_seed(seed)

    def kv(length):
        k = torch.randn(1, shape.num_kv_heads, length, shape.head_dim, generator=gen, device=device).half()
        v = torch.randn(1, shape.num_kv_heads, length, shape.head_dim, generator=gen, device=device).half()
        for c in OUTLIER_CHANNELS.get(shape.head_dim, ()):
            k[..., c] *= OUTLIER_GAIN
        return k, v

    def pack(length, bits):
        k, v = kv(length)
        return PackedKVSegment(packing.quantize_pack(k, bits, -2, group), packing.quantize_pack(v, bits, -1, group))

    prompt = pack(prompt_len, prompt_bits)
    cold = [pack(cold_len, cold_bits)] if cold_len > 0 else []
    hk = hv = None
    if hot_len > 0:
        hk, hv = kv(hot_capacity or hot_len)
    q = torch.randn(shape.num_q_heads, shape.head_dim, generator=gen, device=device).half()
    return LayerTiers(prompt=prompt, cold=cold, hot_k=hk, hot_v=hv, hot_len=hot_len), q
