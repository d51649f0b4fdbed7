"""Stage-A prompt tier on a dense cache: keep the selected prompt tokens per head and fake-quantise them once.

Same calls as the reference's ``src/phasekv/prompt_tier.py``: ``select_prompt_indices`` (:24-75) derives the
per-head positions to keep from the eager attention matrices of the prefill (sink tokens, the most recent
tokens, and the best-voted tokens in between, pooled so that they form clusters), ``select_and_pack`` (:78-104)
evicts everything else per head and ``_pack_prompt`` (:107-118) fake-quantises ``[0, K0)`` to ``prompt_bits`` in
place.  ``pack_selected`` is the second half for callers that already hold the positions.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from . import hetero_cache as hc
from .decode_tier import _quantize_slice


def select_prompt_indices(attentions, *, prompt_len: int, model_config, prefill_keep_ratio: float, sink_tokens: int,
                          obs_window: int, pool_kernel: int, pooling: str):
    """Per layer an int64 ``[B, Hkv, K0]`` tensor of original positions, strictly ascending, without touching the
    cache.  The budget ``K0 = round(prompt_len * prefill_keep_ratio)`` (at least the sinks, at least 1) is filled
    with the sink tokens first, then the most recent ``obs_window`` tokens, then the best-voted of the rest."""
    if attentions is None or not attentions:
        raise ValueError("prompt selection needs the prefill attention matrices of every layer")
    if prompt_len <= 0 or not 0.0 < prefill_keep_ratio <= 1.0:
        raise ValueError("prompt_len and prefill_keep_ratio are invalid")
    if sink_tokens < 0 or obs_window <= 0:
        raise ValueError("sink_tokens must not be negative and obs_window must be positive")
    hkv = hc.num_kv_heads_of(model_config)
    sink = min(sink_tokens, prompt_len)
    budget = min(prompt_len, max(1, sink, round(prompt_len * prefill_keep_ratio)))
    sink_keep = min(sink, budget)
    recent_keep = min(obs_window, budget - sink_keep, prompt_len - sink_keep)
    recent_start = prompt_len - recent_keep
    select_k = budget - sink_keep - recent_keep
    result = []
    for attention in attentions:
        if attention is None or attention.shape[-1] != prompt_len:
            raise ValueError("a prefill attention matrix is missing or its key length differs from prompt_len")
        b, device = attention.shape[0], attention.device
        fixed = torch.cat((torch.arange(sink_keep, device=device), torch.arange(recent_start, prompt_len, device=device)))
        fixed = fixed.view(1, 1, -1).expand(b, hkv, -1)
        if select_k:
            votes = hc.observation_votes(attention, hkv, min(obs_window, prompt_len))
            candidates = hc.pool_scores(votes[..., sink_keep:recent_start], pool_kernel, pooling)
            fixed = torch.cat((fixed, hc.topk_per_head(candidates.contiguous(), select_k) + sink_keep), dim=-1)
        if fixed.shape[-1] != budget:
            raise RuntimeError("the number of kept prompt tokens differs from the budget")
        result.append(fixed.sort(dim=-1).values)
    return result


def select_and_pack(cache, *, attentions, prompt_len: int, model_config, state: hc.HeteroTierState,
                    prefill_keep_ratio: float, sink_tokens: int, obs_window: int, pool_kernel: int, pooling: str) -> None:
    """Per-head attention selection followed by the in-place low-bit packing of the kept prompt; updates
    ``state.prompt_len_phys``."""
    keep_per_layer = select_prompt_indices(
        attentions, prompt_len=prompt_len, model_config=model_config, prefill_keep_ratio=prefill_keep_ratio,
        sink_tokens=sink_tokens, obs_window=obs_window, pool_kernel=pool_kernel, pooling=pooling)
    if len(keep_per_layer) != hc.cache_num_layers(cache):
        raise ValueError("the number of attention layers differs from the number of cache layers")
    pack_selected(cache, keep_per_layer, state)


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
