"""Dequantise-then-attend semantics of the three-tier decode, on the GPU.

Same surface as the reference's ``src/phasekv/kernels/reference.py`` (``ThreeTierKV`` :28,
``fused_decode_attention_reference`` :72, ``dense_fp16_attention`` :99).  It expands every tier
to float16 with the CUDA ``unpack_dequantize`` kernel and runs a plain float32 softmax attention
in torch on the same device, so it saves no bandwidth; it exists for error measurements next to
the fused kernels (scripts/bench_decode_kernel.py:59-63 uses it that way) and is not on the
decode path.
"""
from __future__ import annotations

import math
from typing import List

import torch

from .packing import unpack_dequantize
from .tiers import ThreeTierKV  # noqa: F401


def _dequant_concat(kv: ThreeTierKV):
    ks: List[torch.Tensor] = []
    vs: List[torch.Tensor] = []
    if kv.prompt_k is not None:
        ks.append(unpack_dequantize(kv.prompt_k)), vs.append(unpack_dequantize(kv.prompt_v))
    if kv.cold_k is not None:
        ks.append(unpack_dequantize(kv.cold_k)), vs.append(unpack_dequantize(kv.cold_v))
    if kv.hot_k is not None:
        ks.append(kv.hot_k.to(torch.float16)), vs.append(kv.hot_v.to(torch.float16))
    if not ks:
        raise ValueError("all three tiers are empty, nothing to attend to")
    return torch.cat(ks, dim=-2), torch.cat(vs, dim=-2)


def _expand_gqa(x: torch.Tensor, num_attention_heads: int) -> torch.Tensor:
    hkv = x.shape[1]
    if hkv == num_attention_heads:
        return x
    if num_attention_heads % hkv != 0:
        raise ValueError(f"{num_attention_heads} query heads are not a multiple of {hkv} KV heads")
    return x.repeat_interleave(num_attention_heads // hkv, dim=1)


def dense_fp16_attention(q, k, v, num_attention_heads: int) -> torch.Tensor:
    """Uncompressed float16 attention, no causal mask: q ``[b, Hq, q_len, hd]``, k/v ``[b, Hkv, S, hd]``."""
    k = _expand_gqa(k, num_attention_heads)
    v = _expand_gqa(v, num_attention_heads)
    scores = torch.matmul(q.float(), k.float().transpose(-1, -2)) * (1.0 / math.sqrt(q.shape[-1]))
    return torch.matmul(torch.softmax(scores, dim=-1), v.float()).to(torch.float16)


def fused_decode_attention_reference(q: torch.Tensor, kv: ThreeTierKV, num_attention_heads: int) -> torch.Tensor:
    """q ``[b, Hq, q_len, hd]`` float16 -> ``[b, Hq, q_len, hd]`` float16."""
    if q.dim() != 4:
        raise ValueError(f"q must be [b, Hq, q_len, hd], got {tuple(q.shape)}")
    k_all, v_all = _dequant_concat(kv)
    return dense_fp16_attention(q, k_all, v_all, num_attention_heads)
