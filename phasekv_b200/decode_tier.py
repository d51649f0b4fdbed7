"""Stage-A decode tier on a dense cache: float16 hot window + lazily batched cold compression, on CUDA.

Same call as the reference's ``src/phasekv/decode_tier.py:25-75`` ``maintain`` (and ``_quantize_cold`` :78-88):
after each decode step, once at least ``lazy_g`` generated tokens have slid out of the ``recent_window``, that
batch is reduced per head to the ``decode_keep_ratio`` share with the largest value norms and fake-quantised to
``cold_bits`` in place.  The prompt tier ``[0, K0)`` is never touched.  Per layer: one norm launch, one top-k
launch, two gathers, two in-place quantisations.
"""
from __future__ import annotations

import torch

from . import hetero_cache as hc
from . import quant


def maintain(cache, *, step: int, model_config, state: hc.HeteroTierState, decode_keep_ratio: float,
             lazy_g: int) -> None:
    k0, recent = state.prompt_len_phys, state.recent_window
    seq = hc.cache_seq_len(cache)
    aged = seq - k0 - state.cold_len - recent
    if aged < max(1, lazy_g):
        return
    base, batch = k0 + state.cold_len, aged
    keep_b = batch if decode_keep_ratio >= 1.0 else max(1, int(round(decode_keep_ratio * batch)))
    if keep_b < batch:
        keep_per_layer = []
        for layer in range(hc.cache_num_layers(cache)):
            v = hc.layer_kv(cache, layer)[1]
            b, hkv = v.shape[0], v.shape[1]
            signal = hc.value_norm_signal(v, slice(base, base + batch))
            sel = hc.topk_per_head(signal, keep_b) + base
            head = torch.arange(0, base, device=v.device).view(1, 1, -1).expand(b, hkv, -1)
            tail = torch.arange(base + batch, seq, device=v.device).view(1, 1, -1).expand(b, hkv, -1)
            keep_per_layer.append(torch.cat([head, sel, tail], dim=-1))
        hc.evict_per_head(cache, keep_per_layer)
    _quantize_cold(cache, slice(base, base + keep_b), state)
    state.cold_len += keep_b


def _quantize_cold(cache, token_slice: slice, state: hc.HeteroTierState) -> None:
    """Fake-quantise tokens ``token_slice`` of every layer to ``cold_bits`` (K per channel, V per token), in place."""
    if state.cold_bits >= 16 or token_slice.stop <= token_slice.start:
        return
    for layer in range(hc.cache_num_layers(cache)):
        _quantize_slice(cache, layer, token_slice, state.cold_bits, state.group_size)


def _quantize_slice(cache, layer: int, token_slice: slice, bits: int, group_size: int) -> None:
    key, value = hc.layer_kv(cache, layer)
    if not (key.is_contiguous() and value.is_contiguous()):
        key, value = key.contiguous(), value.contiguous()
        hc.set_layer_kv(cache, layer, key, value)
    quant.fake_quant_(key, token_slice.start, token_slice.stop, bits, -2, group_size)
    quant.fake_quant_(value, token_slice.start, token_slice.stop, bits, -1, group_size)
