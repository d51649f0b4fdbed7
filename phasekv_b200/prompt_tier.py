"""Stage-A prompt tier on a dense cache: keep the selected prompt tokens per head and fake-quantise them once.

``pack_selected`` does what the reference's ``src/phasekv/prompt_tier.py:78-104`` ``select_and_pack`` does once
the per-head positions are known (``select_prompt_indices`` :24-75 derives them from the eager attention
matrices of the evaluation pipeline, which is outside this package): per-head eviction, then ``_pack_prompt``
(:107-118), the in-place ``prompt_bits`` quantisation of ``[0, K0)``.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from . import hetero_cache as hc
from .decode_tier import _quantize_slice


def pack_selected(cache, keep_per_layer: Optional[Sequence[torch.Tensor]], state: hc.HeteroTierState) -> None:
    """``keep_per_layer[l]``: int64 ``[B, Hkv, K0]`` original positions to keep in layer ``l`` (``None``: keep the
    whole prompt).  Updates ``state.prompt_len_phys``."""
    if keep_per_layer is not None:
        if len(keep_per_layer) != hc.cache_num_layers(cache):
            raise ValueError("one index tensor per cache layer is needed")
        if keep_per_layer[0].shape[-1] < hc.cache_seq_len(cache):
            hc.evict_per_head(cache, keep_per_layer)
    state.prompt_len_phys = hc.cache_seq_len(cache)
    _pack_prompt(cache, state.prompt_len_phys, state)


def _pack_prompt(cache, prompt_phys_len: int, state: hc.HeteroTierState) -> None:
    if prompt_phys_len <= 0 or state.prompt_bits >= 16:
        return
    for layer in range(hc.cache_num_layers(cache)):
        _quantize_slice(cache, layer, slice(0, prompt_phys_len), state.prompt_bits, state.group_size)
