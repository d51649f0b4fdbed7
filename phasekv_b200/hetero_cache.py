"""Stage-A three-tier bookkeeping on a dense KV cache, on CUDA.  The cache is any object with ``key_cache`` /
``value_cache`` lists of ``[B, Hkv, S, hd]`` tensors (transformers 4.x ``DynamicCache``, or a stand-in) or with
``layers[i].keys`` / ``.values`` (transformers 5.x); ``layer_kv`` / ``set_layer_kv`` hide the difference.

Same surface as the part of the reference's ``src/phasekv/hetero_cache.py`` that the decode tier needs:
``cache_num_layers`` (:36), ``cache_seq_len`` (:40), ``value_norm_signal`` (:98), ``topk_per_head`` (:157),
``evict_per_head`` (:120), ``HeteroTierState`` (:175), and the attention-vote helpers of the prompt selection
(``aggregate_to_kv_heads`` :56, ``observation_votes`` :67, ``pool_scores`` :80).  The selection signal, the top-k
of a lazy batch and the per-head compaction are one launch each instead of torch pipelines; the vote helpers
operate on the eager attention matrices of the evaluation pipeline with tensor operations.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence

import torch

from . import _native as nv
from . import quant


#: rows longer than this exceed the shared memory of the rank-counting top-k kernel


def _per_layer_lists(cache) -> bool:
    return hasattr(cache, "key_cache") and hasattr(cache, "value_cache")


def cache_num_layers(cache) -> int:
    return len(cache.key_cache) if _per_layer_lists(cache) else len(cache.layers)


def layer_kv(cache, layer_idx: int):
    """``(K, V)`` of one layer, ``(None, None)`` if the layer holds nothing yet."""
    if _per_layer_lists(cache):
        if len(cache.key_cache) <= layer_idx:
            return None, None
        return cache.key_cache[layer_idx], cache.value_cache[layer_idx]
    if len(cache.layers) <= layer_idx:
        return None, None
    layer = cache.layers[layer_idx]
    return getattr(layer, "keys", None), getattr(layer, "values", None)


def set_layer_kv(cache, layer_idx: int, key: torch.Tensor, value: torch.Tensor) -> None:
    if _per_layer_lists(cache):
        cache.key_cache[layer_idx], cache.value_cache[layer_idx] = key, value
    else:
        cache.layers[layer_idx].keys, cache.layers[layer_idx].values = key, value


def cache_seq_len(cache, layer_idx: int = 0) -> int:
    key, _ = layer_kv(cache, layer_idx)
    return 0 if key is None else key.shape[-2]


def num_kv_heads_of(model_config) -> int:
    return getattr(model_config, "num_key_value_heads", getattr(model_config, "num_attention_heads"))


# The three functions below turn the attention matrices of an eager prefill into per-head importance scores.
# They are host-side glue of the evaluation pipeline (the matrices are [B, Hq, q, kv] float tensors a model
# returned) and are written with tensor operations that run wherever those matrices live.
def aggregate_to_kv_heads(scores: torch.Tensor, num_kv_heads: int) -> torch.Tensor:
    """Sum scores given per query head ``[B, Hq, ...]`` over each GQA group -> ``[B, Hkv, ...]``."""
    b, hq = scores.shape[0], scores.shape[1]
    if hq == num_kv_heads:
        return scores
    if hq % num_kv_heads != 0:
        raise ValueError(f"{hq} query heads are not a multiple of {num_kv_heads} KV heads")
    return scores.view(b, num_kv_heads, hq // num_kv_heads, *scores.shape[2:]).sum(dim=2)


def observation_votes(attn_layer: torch.Tensor, num_kv_heads: int, obs_window: int) -> torch.Tensor:
    """Votes of the last ``obs_window`` query rows of a prefill attention matrix for every key position, summed
    over each GQA group: ``[B, Hkv, kv_len]`` float32."""
    w = max(1, min(obs_window, attn_layer.shape[-2]))
    return aggregate_to_kv_heads(attn_layer[:, :, -w:, :].float().sum(dim=2), num_kv_heads)


def pool_scores(scores: torch.Tensor, kernel: Optional[int], mode: str = "maxpool") -> torch.Tensor:
    """1-D pooling along the sequence (stride 1, zero padding of ``kernel // 2``) so that selected tokens form
    contiguous clusters; ``kernel`` of ``None`` or <= 1 returns the scores unchanged."""
    if kernel is None or kernel <= 1:
        return scores
    b, h, length = scores.shape
    x = scores.reshape(b * h, 1, length)
    if mode == "maxpool":
        pooled = torch.nn.functional.max_pool1d(x, kernel_size=kernel, stride=1, padding=kernel // 2)
    elif mode == "avgpool":
        pooled = torch.nn.functional.avg_pool1d(x, kernel_size=kernel, stride=1, padding=kernel // 2)
    else:
        raise ValueError(f"unknown pooling {mode!r}: maxpool or avgpool")
    return pooled[..., :length].reshape(b, h, length)


def value_norm_signal(value_layer: torch.Tensor, token_slice: slice) -> torch.Tensor:
    """Cheap importance of the tokens in ``token_slice`` of a ``[B, Hkv, S, hd]`` value tensor: the L2 norm of
    each value vector, float32 ``[B, Hkv, len(slice)]``."""
    nv.require_cuda(value_layer, "value_layer")
    b, h, seq, hd = value_layer.shape
    start, stop, step = token_slice.indices(seq)
    if step != 1:
        raise ValueError("token_slice must be contiguous")
    n = max(0, stop - start)
    out = torch.empty((b, h, n), dtype=torch.float32, device=value_layer.device)
    if n == 0:
        return out
    v = value_layer if value_layer.is_contiguous() else value_layer.contiguous()
    view = v[:, :, start:stop, :]
    with torch.cuda.device(v.device):
        nv.check(nv.lib().pkv_value_norm(view.data_ptr(), quant._dtype_code(v), b * h, seq * hd, n, hd, out.data_ptr(),
                                         nv.stream_of(v.device)))
    return out


def topk_per_head(signal: torch.Tensor, select_k: int) -> torch.Tensor:
    """Positions (relative to the slice) of the ``select_k`` largest entries of ``signal [B, Hkv, n]`` per head,
    int64 ``[B, Hkv, min(select_k, n)]``.  They come back in ascending position order (the reference returns
    them in score order and every consumer sorts them); NaN counts as the largest value, as ``torch.topk`` has
    it, and ties go to the lower position.  Rows of any length: short rows are ranked by counting, a whole
    prompt's candidates per head by a radix select, both on the GPU."""
    nv.require_cuda(signal, "signal")
    b, h, n = signal.shape
    k = max(0, min(int(select_k), n))
    out = torch.empty((b, h, k), dtype=torch.long, device=signal.device)
    if k == 0:
        return out
    sig = signal.float().contiguous()
    with torch.cuda.device(sig.device):
        nv.check(nv.lib().pkv_topk_rows(sig.data_ptr(), b * h, n, k, out.data_ptr(), nv.stream_of(sig.device)))
    return out


def gather_tokens(tensor: torch.Tensor, indices: torch.Tensor) -> torch.Tensor:
    """``tensor [B, Hkv, S, hd]`` gathered along tokens at ``indices [B, Hkv, K]`` (int64) -> ``[B, Hkv, K, hd]``.
    The kernel never dereferences an index outside ``[0, S)`` (such a row comes out as zeros); callers that take
    indices from outside validate them first (``evict_per_head``, ``PhaseKVCache.from_dense_prefill``)."""
    nv.require_cuda(tensor, "tensor")
    b, h, seq, hd = tensor.shape
    idx = indices.to(device=tensor.device, dtype=torch.long).contiguous()
    if idx.shape[:2] != (b, h):
        raise ValueError(f"indices must be [{b}, {h}, K], got {tuple(idx.shape)}")
    keep = idx.shape[2]
    src = tensor.contiguous()
    out = torch.empty((b, h, keep, hd), dtype=tensor.dtype, device=tensor.device)
    if keep:
        with torch.cuda.device(src.device):
            nv.check(nv.lib().pkv_gather_tokens(src.data_ptr(), out.data_ptr(), idx.data_ptr(), b * h, seq, keep,
                                                hd * tensor.element_size(), nv.stream_of(src.device)))
    return out


def evict_per_head(cache, keep_indices: Sequence[Optional[torch.Tensor]]):
    """Keep, per layer and per head, the tokens named by ``keep_indices[layer]`` (``[B, Hkv, budget]``; ``None``
    leaves a layer alone); positions are put in ascending order first so time order is preserved."""
    for layer in range(cache_num_layers(cache)):
        idx = keep_indices[layer]
        if idx is None:
            continue
        k, v = layer_kv(cache, layer)
        idx = torch.sort(idx.to(device=k.device, dtype=torch.long), dim=-1).values
        if idx.numel() and (int(idx.min()) < 0 or int(idx.max()) >= k.shape[2]):
            raise ValueError(f"layer {layer}: keep_indices must lie in [0, {k.shape[2]})")
        set_layer_kv(cache, layer, gather_tokens(k, idx), gather_tokens(v, idx))
    return cache


@dataclass
class HeteroTierState:
    """Where the three tiers sit in the physical cache (prompt ``[0, K0)``, cold ``[K0, K0 + cold_len)``, hot the
    rest) and how many bits each gets."""

    prompt_len_phys: int = 0
    cold_len: int = 0
    prompt_bits: int = 2
    cold_bits: int = 4
    group_size: int = 32
    recent_window: int = 32

    def reset(self) -> None:
        self.prompt_len_phys = 0
        self.cold_len = 0

    def hot_len(self, cache) -> int:
        return max(0, cache_seq_len(cache) - self.prompt_len_phys - self.cold_len)

    def logical_bytes(self, cache) -> int:
        """Bytes the three tiers would take at their bit widths (the physical tensors stay 16-bit)."""
        first_key = layer_kv(cache, 0)[0] if cache_num_layers(cache) else None
        if first_key is None:
            return 0
        b, hkv, seq, head_dim = first_key.shape
        layers = cache_num_layers(cache)
        k0 = max(0, min(self.prompt_len_phys, seq))
        cold = max(0, min(self.cold_len, seq - k0))
        hot = max(0, seq - k0 - cold)
        return (quant.quantized_tier_bytes(k0, layers, hkv, head_dim, self.prompt_bits, self.prompt_bits, self.group_size, b)
                + quant.quantized_tier_bytes(cold, layers, hkv, head_dim, self.cold_bits, self.cold_bits, self.group_size, b)
                + quant.fp16_tier_bytes(hot, layers, hkv, head_dim, b))
