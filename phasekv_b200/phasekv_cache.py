"""The packed three-tier KV cache of a whole model, on CUDA.

Public surface of the reference's ``src/phasekv/phasekv_cache.py:136-485`` ``PhaseKVCache``: built from a dense
prefill cache (``from_dense_prefill``), then driven by a custom attention layer, per decode step
``append_hot`` for every layer followed by ``finish_decode_step`` (which cools aged hot tokens into a new frozen
cold segment), or per new prompt chunk ``begin_prompt_chunk`` / ``append_prompt_token`` / ``finish_prompt_chunk``.
``layer_tiers(l)`` is what ``kernels.attention_triton.fused_phasekv_decode`` reads.

What is different here: packing, cooling and gathering are single kernel launches (``pkv_quantize_pack``,
``pkv_cold_select_pack``, ``pkv_gather_tokens``) and every tensor lives on a CUDA device; the class derives from
``transformers.Cache`` when that can be imported and constructed, whatever its version, and from ``object``
otherwise.  Error messages carry the reference's wording for the state a caller got wrong, so code (and tests)
that match on them keep working.
"""
from __future__ import annotations

from dataclasses import replace
from numbers import Integral, Real
from typing import List, Optional, Sequence

import torch

from .cold_tier import cool_aged_tokens
from .hetero_cache import gather_tokens
from .kernels.packing import PackedTensor, quantize_pack
from .kernels.tiers import LayerTiers, PackedKVSegment

try:  # any transformers version, or none
    from transformers.cache_utils import Cache as _CacheBase
except Exception:  # pragma: no cover - transformers is optional
    _CacheBase = object

_PACKED_BITS = (2, 4, 8)
_INDEX_DTYPES = (torch.int8, torch.int16, torch.int32, torch.int64, torch.uint8)


def _require_positive_int(name: str, value) -> None:
    if isinstance(value, bool) or not isinstance(value, Integral) or value <= 0:
        raise ValueError(f"{name} 必须为正整数 (must be a positive integer), got {value!r}")


def _validate_config(prompt_bits, cold_bits, group_size, recent_window, lazy_g, decode_keep_ratio) -> None:
    for name, bits in (("prompt_bits", prompt_bits), ("cold_bits", cold_bits)):
        if isinstance(bits, bool) or not isinstance(bits, Integral) or bits not in _PACKED_BITS:
            raise ValueError(f"{name}: packed widths are 2, 4 or 8 bits, got {bits!r}")
    for name, value in (("group_size", group_size), ("recent_window", recent_window), ("lazy_g", lazy_g)):
        _require_positive_int(name, value)
    if (isinstance(decode_keep_ratio, bool) or not isinstance(decode_keep_ratio, Real)
            or not 0.0 < decode_keep_ratio <= 1.0):
        raise ValueError(f"decode_keep_ratio must lie in (0, 1], got {decode_keep_ratio!r}")


def _pack_kv(key: torch.Tensor, value: torch.Tensor, bits: int, group_size: int) -> PackedKVSegment:
    """K per channel (groups of tokens), V per token (groups along head_dim); ``[B, Hkv, S, hd]`` float16."""
    return PackedKVSegment(quantize_pack(key, bits, axis=-2, group_size=group_size),
                           quantize_pack(value, bits, axis=-1, group_size=group_size))


def _gather_kv(key: torch.Tensor, value: torch.Tensor, indices: torch.Tensor):
    """Keep, per batch entry and KV head, the tokens at ``indices [B, Hkv, K]``."""
    return gather_tokens(key, indices), gather_tokens(value, indices)


def _dense_layers(dense_cache):
    """Per-layer K and V lists of a prefill cache: ``key_cache`` / ``value_cache`` attributes (transformers 4.x
    ``DynamicCache``, or any stand-in), else the ``layers[i].keys`` / ``.values`` of a 5.x cache."""
    if hasattr(dense_cache, "key_cache") and hasattr(dense_cache, "value_cache"):
        return list(dense_cache.key_cache), list(dense_cache.value_cache)
    layers = getattr(dense_cache, "layers", None)
    if layers is not None and all(hasattr(l, "keys") and hasattr(l, "values") for l in layers):
        return [l.keys for l in layers], [l.values for l in layers]
    raise TypeError("dense_cache 必须提供逐层 key_cache/value_cache (per-layer key_cache/value_cache lists, "
                    "e.g. a DynamicCache)")


class PhaseKVCache(_CacheBase):
    """Low-bit cache for a custom attention layer; normally made by :meth:`from_dense_prefill`.

    ``get_seq_length()`` is the number of tokens a layer physically holds, ``true_seq_length`` the number of
    tokens whose forward pass has been committed (the next RoPE position).  ``update()`` of the standard cache
    protocol returns dense K/V and is therefore refused.
    """

    def __init__(self, layers: List[LayerTiers], *, seen_tokens: int, prompt_bits: int, cold_bits: int,
                 group_size: int, recent_window: int, lazy_g: int, decode_keep_ratio: float) -> None:
        if _CacheBase is not object:
            for kwargs in ({}, {"layers": []}):
                try:
                    super().__init__(**kwargs)
                    break
                except (TypeError, ValueError):
                    continue
        _validate_config(prompt_bits, cold_bits, group_size, recent_window, lazy_g, decode_keep_ratio)
        _require_positive_int("seen_tokens", seen_tokens)
        if not layers:
            raise ValueError("layers must hold at least one layer of KV")
        for layer_idx, layer in enumerate(layers):
            if layer.hot_k is None or layer.hot_v is None:
                raise ValueError(f"layer {layer_idx} has no hot_k/hot_v; build the cache with from_dense_prefill()")
        self.layers = layers
        self._seen_tokens = int(seen_tokens)
        self.prompt_bits, self.cold_bits, self.group_size = prompt_bits, cold_bits, group_size
        self.recent_window, self.lazy_g, self.decode_keep_ratio = recent_window, lazy_g, decode_keep_ratio
        self._pending_layers: set = set()        # layers that already got this decode step's token
        self._prompt_chunk_len = 0                # > 0 while a prompt chunk is being written
        self._prompt_chunk_start: List[int] = []  # hot_len of every layer when the chunk began

    # ------------------------------------------------------------------ construction
    @classmethod
    @torch.no_grad()
    def from_dense_prefill(cls, dense_cache, *, prompt_len: int, keep_indices: Optional[Sequence[torch.Tensor]] = None,
                           prompt_bits: int = 2, cold_bits: int = 4, group_size: int = 32, recent_window: int = 32,
                           lazy_g: int = 16, decode_keep_ratio: float = 1.0) -> "PhaseKVCache":
        """Select (optionally) and pack the prefill K/V of every layer; ``dense_cache`` is left untouched.

        ``keep_indices[layer]`` is an integer tensor ``[B, Hkv, K0]`` of original positions (they may differ per
        head; ``K0`` must be the same in every layer); ``None`` keeps everything.  K must already carry RoPE.
        """
        _require_positive_int("prompt_len", prompt_len)
        _validate_config(prompt_bits, cold_bits, group_size, recent_window, lazy_g, decode_keep_ratio)
        keys, values = _dense_layers(dense_cache)
        if len(keys) == 0 or len(keys) != len(values):
            raise ValueError(f"the prefill cache needs the same non-zero number of K and V layers, got {len(keys)}/{len(values)}")
        if keep_indices is not None and len(keep_indices) != len(keys):
            raise ValueError(f"keep_indices needs {len(keys)} layers, got {len(keep_indices)}")
        capacity = recent_window + lazy_g  # the protected window plus one batch waiting to be cooled
        layers: List[LayerTiers] = []
        retained: Optional[int] = None
        for layer_idx, (key, value) in enumerate(zip(keys, values)):
            where = f"第 {layer_idx} 层 prefill (layer {layer_idx})"
            if not isinstance(key, torch.Tensor) or not isinstance(value, torch.Tensor):
                raise TypeError(f"{where}: K/V must be tensors")
            if key.ndim != 4 or key.shape != value.shape or any(s == 0 for s in key.shape):
                raise ValueError(f"{where}: K/V must be non-empty [B,Hkv,S,hd] of one shape, got {tuple(key.shape)}/{tuple(value.shape)}")
            if key.dtype not in (torch.float16, torch.bfloat16) or value.dtype != key.dtype:
                raise ValueError(f"{where}: K/V must both be float16 or bfloat16, got {key.dtype}/{value.dtype}")
            if key.device != value.device:
                raise ValueError(f"{where}: K/V must be on 同一设备 (one device), got {key.device}/{value.device}")
            if key.shape[2] != prompt_len:
                raise ValueError(f"{where}: KV length should be prompt_len={prompt_len}, got {key.shape[2]}")
            if keep_indices is not None:
                indices = keep_indices[layer_idx]
                if not isinstance(indices, torch.Tensor) or indices.dtype not in _INDEX_DTYPES:
                    raise ValueError(f"layer {layer_idx}: keep_indices 必须是整数张量 (must be an integer tensor); "
                                     "fractional positions are not truncated")
                if indices.ndim != 3 or indices.shape[:2] != key.shape[:2] or indices.shape[2] == 0:
                    raise ValueError(f"layer {layer_idx}: keep_indices must be [{key.shape[0]},{key.shape[1]},K0] with K0>0, "
                                     f"got {tuple(indices.shape)}")
                indices = indices.to(device=key.device, dtype=torch.long).sort(dim=-1).values
                if bool((indices < 0).any()) or bool((indices >= prompt_len).any()):
                    raise ValueError(f"layer {layer_idx}: keep_indices must lie in [0, {prompt_len})")
                if bool((indices[..., 1:] == indices[..., :-1]).any()):
                    raise ValueError(f"layer {layer_idx}: keep_indices repeats a position within one batch entry / head")
                key, value = _gather_kv(key.contiguous(), value.contiguous(), indices)
            if retained is not None and key.shape[2] != retained:
                raise ValueError(f"every layer must keep the same number of prompt tokens: layer 0 keeps {retained}, "
                                 f"layer {layer_idx} keeps {key.shape[2]}")
            retained = key.shape[2]
            key, value = key.to(torch.float16), value.to(torch.float16)  # packed attention and the hot tier are float16
            shape = (key.shape[0], key.shape[1], capacity, key.shape[3])
            layers.append(LayerTiers(prompt=_pack_kv(key, value, prompt_bits, group_size),
                                     hot_k=torch.empty(shape, dtype=torch.float16, device=key.device),
                                     hot_v=torch.empty(shape, dtype=torch.float16, device=key.device)))
        return cls(layers, seen_tokens=prompt_len, prompt_bits=prompt_bits, cold_bits=cold_bits, group_size=group_size,
                   recent_window=recent_window, lazy_g=lazy_g, decode_keep_ratio=decode_keep_ratio)

    # ------------------------------------------------------------------ reading
    def __len__(self) -> int:
        return len(self.layers)

    def layer_tiers(self, layer_idx: int) -> LayerTiers:
        if isinstance(layer_idx, bool) or not isinstance(layer_idx, Integral) or not 0 <= layer_idx < len(self.layers):
            raise IndexError(f"layer_idx must be an integer in [0, {len(self.layers)}), got {layer_idx!r}")
        return self.layers[layer_idx]

    def get_seq_length(self, layer_idx: Optional[int] = 0) -> int:
        return self.layer_tiers(0 if layer_idx is None else layer_idx).physical_len

    def get_max_cache_shape(self) -> None:
        """The cache grows with every frozen segment; the hot capacity is not a bound on it."""
        return None

    @property
    def true_seq_length(self) -> int:
        return self._seen_tokens

    @property
    def prompt_chunk_len(self) -> int:
        return self._prompt_chunk_len

    # ------------------------------------------------------------------ one decode step
    @torch.no_grad()
    def append_hot(self, layer_idx: int, key: torch.Tensor, value: torch.Tensor) -> None:
        """One token (K with RoPE applied, and V) per layer per step; nothing is cooled or committed here."""
        if self._prompt_chunk_len:
            raise RuntimeError("a prompt chunk is open: use append_prompt_token() inside it and finish_prompt_chunk() after it")
        layer = self.layer_tiers(layer_idx)
        if layer_idx in self._pending_layers:
            raise RuntimeError(f"第 {layer_idx} 层在当前 decode 步已追加 (layer {layer_idx} already got this step's token); "
                               "call finish_decode_step() after the forward pass")
        self._append_token(layer_idx, layer, key, value)
        self._pending_layers.add(layer_idx)

    @torch.no_grad()
    def finish_decode_step(self) -> None:
        """Once per single-token forward pass: cool what has aged out, then advance the true length by one."""
        if self._prompt_chunk_len:
            raise RuntimeError("a prompt chunk is open: call finish_prompt_chunk(), not finish_decode_step()")
        missing = sorted(set(range(len(self.layers))) - self._pending_layers)
        if missing:
            raise RuntimeError(f"finish_decode_step() needs one token in 每一层 (every layer); 尚未追加的层为 {missing}")
        lengths = [(layer.physical_len, layer.hot_len) for layer in self.layers]
        if len(set(lengths)) != 1:
            raise RuntimeError(f"(physical, hot) lengths differ between layers before cooling: {lengths}")
        for layer in self.layers:
            self._cool_aged_tokens(layer)
        self._seen_tokens += 1
        self._pending_layers.clear()

    def _cool_aged_tokens(self, layer: LayerTiers) -> None:
        """Only the oldest batch of the hot buffer is touched; frozen prompt and cold segments never are."""
        cool_aged_tokens(layer, self.recent_window, self.lazy_g, self.decode_keep_ratio, self.cold_bits, self.group_size)

    # ------------------------------------------------------------------ a new prompt chunk (multi-turn input)
    @torch.no_grad()
    def begin_prompt_chunk(self, length: int) -> None:
        """Make room for ``length`` new input tokens behind the hot tokens (growing the hot buffers if needed)."""
        _require_positive_int("length", length)
        self._require_idle("begin_prompt_chunk()")
        for layer in self.layers:
            needed = layer.hot_len + length
            if needed <= layer.hot_k.shape[2]:
                continue
            new_k, new_v = self._empty_hot(layer, needed)
            hot_k, hot_v = layer.hot_views()
            new_k[:, :, :layer.hot_len, :].copy_(hot_k)
            new_v[:, :, :layer.hot_len, :].copy_(hot_v)
            layer.hot_k, layer.hot_v = new_k, new_v
        self._prompt_chunk_start = [layer.hot_len for layer in self.layers]
        self._prompt_chunk_len = length

    @torch.no_grad()
    def append_prompt_token(self, layer_idx: int, key: torch.Tensor, value: torch.Tensor) -> None:
        """Inside a chunk tokens are written one by one, each attended to right after, so no query sees its future."""
        if not self._prompt_chunk_len:
            raise RuntimeError("no prompt chunk is open; call begin_prompt_chunk(length) first")
        layer = self.layer_tiers(layer_idx)
        written = layer.hot_len - self._prompt_chunk_start[layer_idx]
        if written >= self._prompt_chunk_len:
            raise RuntimeError(f"第 {layer_idx} 层已写满 (layer {layer_idx} is full): all {self._prompt_chunk_len} tokens of "
                               "this prompt chunk are written")
        self._append_token(layer_idx, layer, key, value)

    @torch.no_grad()
    def finish_prompt_chunk(self) -> None:
        """Freeze the whole chunk at ``prompt_bits`` as a new prompt extension.  The hot tokens generated before the
        chunk stay as they are (float16, still subject to the usual cooling schedule); older segments are untouched."""
        if not self._prompt_chunk_len:
            raise RuntimeError("no prompt chunk is open; call begin_prompt_chunk(length) first")
        for layer_idx, (layer, start) in enumerate(zip(self.layers, self._prompt_chunk_start)):
            written = layer.hot_len - start
            if written != self._prompt_chunk_len:
                raise RuntimeError(f"第 {layer_idx} 层 (layer {layer_idx}) prompt chunk is incomplete: "
                                   f"期望 {self._prompt_chunk_len} 个，实际 {written} 个")
        for layer, start in zip(self.layers, self._prompt_chunk_start):
            segment = _pack_kv(layer.hot_k[:, :, start:layer.hot_len, :].contiguous(),
                               layer.hot_v[:, :, start:layer.hot_len, :].contiguous(), self.prompt_bits, self.group_size)
            hot_k, hot_v = self._empty_hot(layer, self.recent_window + self.lazy_g)
            hot_k[:, :, :start, :].copy_(layer.hot_k[:, :, :start, :])
            hot_v[:, :, :start, :].copy_(layer.hot_v[:, :, :start, :])
            layer.prompt_extensions.append(segment)
            layer.hot_k, layer.hot_v = hot_k, hot_v
            layer.hot_len = start
        self._seen_tokens += self._prompt_chunk_len
        self._prompt_chunk_len = 0
        self._prompt_chunk_start = []

    # ------------------------------------------------------------------ shared write path
    def _append_token(self, layer_idx: int, layer: LayerTiers, key: torch.Tensor, value: torch.Tensor) -> None:
        """A failed check leaves hot_len and the pending set unchanged."""
        where = f"layer {layer_idx} new K/V"
        if not isinstance(key, torch.Tensor) or not isinstance(value, torch.Tensor):
            raise TypeError(f"{where} must be tensors")
        expected = (*layer.hot_k.shape[:2], 1, layer.hot_k.shape[-1])
        if key.shape != expected or value.shape != expected:
            raise ValueError(f"{where} must be one token of shape {expected}, got {tuple(key.shape)}/{tuple(value.shape)}")
        if key.dtype != torch.float16 or value.dtype != torch.float16:
            raise ValueError(f"{where} must be float16, got {key.dtype}/{value.dtype}; a bfloat16 model converts before writing")
        if key.device != layer.hot_k.device or value.device != layer.hot_v.device:
            raise ValueError(f"{where} must be on 同一设备 (the device of the hot tier, {layer.hot_k.device}), "
                             f"got {key.device}/{value.device}")
        if layer.hot_len >= layer.hot_k.shape[2]:
            raise RuntimeError(f"layer {layer_idx}: hot tier is full (hot_len={layer.hot_len}, capacity={layer.hot_k.shape[2]})")
        position = layer.hot_len
        layer.hot_k[:, :, position:position + 1, :].copy_(key)
        layer.hot_v[:, :, position:position + 1, :].copy_(value)
        layer.hot_len += 1

    @staticmethod
    def _empty_hot(layer: LayerTiers, capacity: int):
        shape = (*layer.hot_k.shape[:2], capacity, layer.hot_k.shape[-1])
        return layer.hot_k.new_empty(shape), layer.hot_v.new_empty(shape)

    def _require_idle(self, operation: str) -> None:
        if self._prompt_chunk_len:
            raise RuntimeError(f"{operation} 不能在新增 prompt 块内调用 (not inside a prompt chunk); finish the chunk's forward "
                               "pass and call finish_prompt_chunk() first")
        if self._pending_layers:
            raise RuntimeError(f"{operation} 不能在 decode 步内调用 (not inside a decode step); layers {sorted(self._pending_layers)} "
                               "are written, finish the others and call finish_decode_step() first")

    # ------------------------------------------------------------------ accounting and the Cache protocol
    def physical_nbytes(self) -> int:
        """Bytes of KV held, including the reserved hot capacity; scratch of packing and attention is not counted."""
        total = 0
        for layer in self.layers:
            total += layer.prompt.nbytes
            total += sum(s.nbytes for s in layer.prompt_extensions) + sum(s.nbytes for s in layer.cold)
            total += layer.hot_k.numel() * layer.hot_k.element_size() + layer.hot_v.numel() * layer.hot_v.element_size()
        return total

    def update(self, key_states, value_states, layer_idx, cache_kwargs=None):
        raise RuntimeError("PhaseKVCache 不返回稠密 K/V (does not return dense K/V) and cannot serve Cache.update(); install the "
                           "PhaseKV attention adapter, which calls append_hot() / append_prompt_token() and reads layer_tiers()")

    @torch.no_grad()
    def reorder_cache(self, beam_idx: torch.LongTensor) -> None:
        """Reorder the batch dimension of every tier between steps."""
        self._require_idle("reorder_cache()")
        if not isinstance(beam_idx, torch.Tensor) or beam_idx.ndim != 1 or beam_idx.dtype != torch.long or beam_idx.numel() == 0:
            raise ValueError("beam_idx must be a non-empty one-dimensional torch.long tensor")
        for layer_idx, layer in enumerate(self.layers):
            if bool((beam_idx < 0).any()) or bool((beam_idx >= layer.hot_k.shape[0]).any()):
                raise ValueError(f"beam_idx is outside the batch range [0, {layer.hot_k.shape[0]}) of layer {layer_idx}")

        def reorder(pt: PackedTensor) -> PackedTensor:
            index = beam_idx.to(pt.packed.device)
            return replace(pt, packed=pt.packed.index_select(0, index), scale=pt.scale.index_select(0, index),
                           mins=pt.mins.index_select(0, index), orig_shape=(index.numel(), *pt.orig_shape[1:]))

        def reorder_segment(seg: PackedKVSegment) -> PackedKVSegment:
            return PackedKVSegment(reorder(seg.key), reorder(seg.value))

        for layer in self.layers:
            layer.prompt = reorder_segment(layer.prompt)
            layer.prompt_extensions = [reorder_segment(s) for s in layer.prompt_extensions]
            layer.cold = [reorder_segment(s) for s in layer.cold]
            layer.hot_k = layer.hot_k.index_select(0, beam_idx.to(layer.hot_k.device))
            layer.hot_v = layer.hot_v.index_select(0, beam_idx.to(layer.hot_v.device))
