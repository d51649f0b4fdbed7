"""The packed three-tier KV cache of a whole model, on CUDA.

Public surface of the reference's ``src/phasekv/phasekv_cache.py:136-485`` ``PhaseKVCache``: built from a dense
prefill cache (``from_dense_prefill``), then driven by a custom attention layer, per decode step
``append_hot`` for every layer followed by ``finish_decode_step`` (which cools aged hot tokens into a new frozen
cold segment), or per new prompt chunk ``begin_prompt_chunk`` / ``append_prompt_token`` / ``finish_prompt_chunk``.
``layer_tiers(l)`` is what ``kernels.attention_triton.fused_phasekv_decode`` reads.

How it is organised here:

* the cache is a small state machine (``_Phase``: idle, inside a decode step, inside a prompt chunk); every public
  call first asks the machine whether it is allowed, so a refused call leaves nothing half done;
* the cold tier of a layer lives in pre-allocated arenas (``cold_arena.ColdArena``) that the cooling kernel fills
  in place, for ALL layers in one launch; ``LayerTiers.cold`` still lists one ``PackedKVSegment`` per cooling step,
  as the reference has it, but those are views into the arena, and the decode kernels read a whole run of steps as
  one segment;
* packing, cooling and gathering are kernel launches (``pkv_quantize_pack``, ``pkv_cold_select_pack_layers``,
  ``pkv_gather_tokens``) on CUDA tensors; the decode path never synchronises with the host;
* the class derives from ``transformers.Cache`` when that can be imported and constructed, whatever its version,
  and from ``object`` otherwise.  Error messages carry the reference's wording for the state a caller got wrong, so
  code (and tests) that match on them keep working.
"""
from __future__ import annotations

import enum
from dataclasses import replace
from numbers import Integral, Real
from typing import List, Optional, Sequence

import torch

from . import _native as nv
from .cold_arena import ColdArena, CoolingTable, cool_layers_into_arenas
from .cold_tier import select_and_pack_cold
from .hetero_cache import gather_tokens
from .kernels.packing import PackedTensor, quantize_pack
from .kernels.tiers import LayerTiers, PackedKVSegment

try:  # any transformers version, or none
    from transformers.cache_utils import Cache as _CacheBase
except Exception:  # pragma: no cover - transformers is optional
    _CacheBase = object

_PACKED_BITS = (2, 4, 8)
_INDEX_DTYPES = (torch.int8, torch.int16, torch.int32, torch.int64, torch.uint8)
_ROPE_DTYPES = {torch.float16: nv.PKV_DTYPE_F16, torch.bfloat16: nv.PKV_DTYPE_BF16, torch.float32: nv.PKV_DTYPE_F32}


class _Phase(enum.Enum):
    IDLE = "idle"
    DECODE_STEP = "decode step"      # some layers already hold this step's token
    PROMPT_CHUNK = "prompt chunk"    # a chunk of new input tokens is being written


# --------------------------------------------------------------------------- argument checks
def _is_int(value) -> bool:
    return isinstance(value, Integral) and not isinstance(value, bool)


def _require_positive_int(name: str, value) -> None:
    if not _is_int(value) or value <= 0:
        raise ValueError(f"{name} 必须为正整数 (must be a positive integer), got {value!r}")


def _validate_config(prompt_bits, cold_bits, group_size, recent_window, lazy_g, decode_keep_ratio) -> None:
    for name, bits in (("prompt_bits", prompt_bits), ("cold_bits", cold_bits)):
        if not _is_int(bits) or bits not in _PACKED_BITS:
            raise ValueError(f"{name}: packed widths are 2, 4 or 8 bits, got {bits!r}")
    for name, value in (("group_size", group_size), ("recent_window", recent_window), ("lazy_g", lazy_g)):
        _require_positive_int(name, value)
    ratio_ok = isinstance(decode_keep_ratio, Real) and not isinstance(decode_keep_ratio, bool)
    if not ratio_ok or not 0.0 < decode_keep_ratio <= 1.0:
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


def _check_prefill_layer(layer_idx: int, key, value, prompt_len: int) -> None:
    where = f"第 {layer_idx} 层 prefill (layer {layer_idx})"
    if not isinstance(key, torch.Tensor) or not isinstance(value, torch.Tensor):
        raise TypeError(f"{where}: K/V must be tensors")
    if key.ndim != 4 or key.shape != value.shape or 0 in key.shape:
        raise ValueError(f"{where}: K/V must be non-empty [B,Hkv,S,hd] of one shape, got "
                         f"{tuple(key.shape)}/{tuple(value.shape)}")
    if key.dtype not in (torch.float16, torch.bfloat16) or value.dtype != key.dtype:
        raise ValueError(f"{where}: K/V must both be float16 or bfloat16, got {key.dtype}/{value.dtype}")
    if key.device != value.device:
        raise ValueError(f"{where}: K/V must be on 同一设备 (one device), got {key.device}/{value.device}")
    if key.shape[2] != prompt_len:
        raise ValueError(f"{where}: KV length should be prompt_len={prompt_len}, got {key.shape[2]}")


def _sorted_keep_indices(layer_idx: int, indices, key: torch.Tensor, prompt_len: int) -> torch.Tensor:
    if not isinstance(indices, torch.Tensor) or indices.dtype not in _INDEX_DTYPES:
        raise ValueError(f"layer {layer_idx}: keep_indices 必须是整数张量 (must be an integer tensor); "
                         "fractional positions are not truncated")
    if indices.ndim != 3 or indices.shape[:2] != key.shape[:2] or indices.shape[2] == 0:
        raise ValueError(f"layer {layer_idx}: keep_indices must be [{key.shape[0]},{key.shape[1]},K0] with K0>0, "
                         f"got {tuple(indices.shape)}")
    indices = indices.to(device=key.device, dtype=torch.long).sort(dim=-1).values
    # one read-back for all three conditions (prefill time, not the decode path)
    lowest, highest, repeats = (int(v) for v in torch.stack([
        indices.min(), indices.max(), (indices[..., 1:] == indices[..., :-1]).sum()]).tolist())
    if lowest < 0 or highest >= prompt_len:
        raise ValueError(f"layer {layer_idx}: keep_indices must lie in [0, {prompt_len})")
    if repeats:
        raise ValueError(f"layer {layer_idx}: keep_indices repeats a position within one batch entry / head")
    return indices


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
        self._phase = _Phase.IDLE
        self._written: set = set()                # decode step: layers that already hold this step's token
        self._chunk_len = 0                       # prompt chunk: tokens it will hold
        self._chunk_start: List[int] = []         # prompt chunk: hot_len of every layer when it began
        self._cooling_table = CoolingTable()
        for layer in layers:
            if not hasattr(layer, "_cold_runs"):
                layer._cold_runs = []             # arenas, each a run of cooling steps of one size

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
            raise ValueError(f"the prefill cache needs the same non-zero number of K and V layers, got "
                             f"{len(keys)}/{len(values)}")
        if keep_indices is not None and len(keep_indices) != len(keys):
            raise ValueError(f"keep_indices needs {len(keys)} layers, got {len(keep_indices)}")
        capacity = recent_window + lazy_g  # the protected window plus one batch waiting to be cooled
        layers: List[LayerTiers] = []
        for layer_idx, (key, value) in enumerate(zip(keys, values)):
            _check_prefill_layer(layer_idx, key, value, prompt_len)
            if keep_indices is not None:
                chosen = _sorted_keep_indices(layer_idx, keep_indices[layer_idx], key, prompt_len)
                key, value = _gather_kv(key.contiguous(), value.contiguous(), chosen)
            if layers and key.shape[2] != layers[0].prompt.length:
                raise ValueError(f"every layer must keep the same number of prompt tokens: layer 0 keeps "
                                 f"{layers[0].prompt.length}, layer {layer_idx} keeps {key.shape[2]}")
            key, value = key.to(torch.float16), value.to(torch.float16)  # packed attention and the hot tier are float16
            hot_shape = (key.shape[0], key.shape[1], capacity, key.shape[3])
            layers.append(LayerTiers(prompt=_pack_kv(key, value, prompt_bits, group_size),
                                     hot_k=torch.empty(hot_shape, dtype=torch.float16, device=key.device),
                                     hot_v=torch.empty(hot_shape, dtype=torch.float16, device=key.device)))
        return cls(layers, seen_tokens=prompt_len, prompt_bits=prompt_bits, cold_bits=cold_bits, group_size=group_size,
                   recent_window=recent_window, lazy_g=lazy_g, decode_keep_ratio=decode_keep_ratio)

    # ------------------------------------------------------------------ reading
    def __len__(self) -> int:
        return len(self.layers)

    def layer_tiers(self, layer_idx: int) -> LayerTiers:
        if not _is_int(layer_idx) or not 0 <= layer_idx < len(self.layers):
            raise IndexError(f"layer_idx must be an integer in [0, {len(self.layers)}), got {layer_idx!r}")
        return self.layers[layer_idx]

    def get_seq_length(self, layer_idx: Optional[int] = 0) -> int:
        return self.layer_tiers(0 if layer_idx is None else layer_idx).physical_len

    def get_max_cache_shape(self) -> None:
        """The cache grows with every frozen segment; the hot capacity is not a bound on it."""
        return None

    def get_mask_sizes(self, query_length, layer_idx: int = 0):
        """``(kv_length, kv_offset)`` for the mask a model prepares before calling its layers (the base class
        would look for its own layer objects in ``self.layers``).  Older transformers pass the cache positions
        instead of the query length.  The PhaseKV attention layer ignores the mask: visibility follows from what
        has been written."""
        if isinstance(query_length, torch.Tensor):
            query_length = query_length.shape[0]
        return self.get_seq_length(layer_idx) + int(query_length), 0

    @property
    def is_compileable(self) -> bool:
        return False

    @property
    def is_initialized(self) -> bool:
        return True

    @property
    def is_sliding(self) -> List[bool]:
        return [False] * len(self.layers)

    @property
    def true_seq_length(self) -> int:
        return self._seen_tokens

    @property
    def prompt_chunk_len(self) -> int:
        return self._chunk_len if self._phase is _Phase.PROMPT_CHUNK else 0

    # ------------------------------------------------------------------ the state machine
    def _refuse_inside_chunk(self, hint: str) -> None:
        if self._phase is _Phase.PROMPT_CHUNK:
            raise RuntimeError(f"a prompt chunk is open: {hint}")

    def _require_chunk(self) -> None:
        if self._phase is not _Phase.PROMPT_CHUNK:
            raise RuntimeError("no prompt chunk is open; call begin_prompt_chunk(length) first")

    def _require_idle(self, operation: str) -> None:
        if self._phase is _Phase.PROMPT_CHUNK:
            raise RuntimeError(f"{operation} 不能在新增 prompt 块内调用 (not inside a prompt chunk); finish the chunk's "
                               "forward pass and call finish_prompt_chunk() first")
        if self._phase is _Phase.DECODE_STEP:
            raise RuntimeError(f"{operation} 不能在 decode 步内调用 (not inside a decode step); layers "
                               f"{sorted(self._written)} are written, finish the others and call "
                               "finish_decode_step() first")

    # ------------------------------------------------------------------ one decode step
    @torch.no_grad()
    def append_hot(self, layer_idx: int, key: torch.Tensor, value: torch.Tensor) -> None:
        """One token (K with RoPE applied, and V) per layer per step; nothing is cooled or committed here."""
        self._refuse_inside_chunk("use append_prompt_token() inside it and finish_prompt_chunk() after it")
        layer = self.layer_tiers(layer_idx)
        if layer_idx in self._written:
            raise RuntimeError(f"第 {layer_idx} 层在当前 decode 步已追加 (layer {layer_idx} already got this step's "
                               "token); call finish_decode_step() after the forward pass")
        self._write_token(layer_idx, layer, key, value)
        self._written.add(layer_idx)
        self._phase = _Phase.DECODE_STEP

    @torch.no_grad()
    def finish_decode_step(self) -> None:
        """Once per single-token forward pass: cool what has aged out, then advance the true length by one."""
        self._refuse_inside_chunk("call finish_prompt_chunk(), not finish_decode_step()")
        if len(self._written) != len(self.layers):
            missing = sorted(set(range(len(self.layers))) - self._written)
            raise RuntimeError(f"finish_decode_step() needs one token in 每一层 (every layer); 尚未追加的层为 {missing}")
        # all layers move in lockstep; the cheap signature first (physical_len walks every cold segment)
        if len({(layer.hot_len, len(layer.cold), len(layer.prompt_extensions)) for layer in self.layers}) != 1:
            lengths = sorted({(layer.physical_len, layer.hot_len) for layer in self.layers})
            raise RuntimeError(f"(physical, hot) lengths differ between layers before cooling: {lengths}")
        self._cool_aged_tokens()
        self._seen_tokens += 1
        self._written.clear()
        self._phase = _Phase.IDLE

    def _cool_aged_tokens(self) -> None:
        """Only the oldest batch of the hot buffers is touched; frozen prompt and cold segments never are.  All
        layers hold the same number of hot tokens, so they cool together: one launch fills the next slot of every
        layer's arena (value-norm top-k, quantise+pack, compaction of the hot buffers)."""
        hot_len = self.layers[0].hot_len
        aged = hot_len - self.recent_window
        if aged < self.lazy_g:
            return
        keep = max(1, round(self.decode_keep_ratio * aged))  # Python's round: half to even
        slot_tokens = -(-keep // self.group_size) * self.group_size
        same_place = len({(l.hot_k.device, tuple(l.hot_k.shape)) for l in self.layers}) == 1
        if (slot_tokens * self.cold_bits) % 8 or not same_place:
            # a slot that is not a whole number of bytes, or layers on several devices: a tensor set per step
            for layer in self.layers:
                layer.cold.append(select_and_pack_cold(layer.hot_k, layer.hot_v, hot_len, aged, keep, self.cold_bits,
                                                       self.group_size))
                layer.hot_len -= aged
            return
        arenas = []
        for layer in self.layers:
            runs = layer._cold_runs
            if not runs or runs[-1].keep != keep:
                runs.append(ColdArena(layer.hot_k, self.cold_bits, self.group_size, keep))
            arenas.append(runs[-1])
        if arenas[0].full:
            for layer, arena in zip(self.layers, arenas):
                before = len(layer.cold) - arena.events
                arena.grow()
                layer.cold[before:] = arena.views  # the same steps, now views of the larger arena
        cool_layers_into_arenas([(l.hot_k, l.hot_v) for l in self.layers], arenas, self._cooling_table, hot_len, aged,
                                keep, self.cold_bits, self.group_size)
        for layer, arena in zip(self.layers, arenas):
            layer.cold.append(arena.commit_event())
            layer.hot_len -= aged

    # ------------------------------------------------------------------ a new prompt chunk (multi-turn input)
    @torch.no_grad()
    def begin_prompt_chunk(self, length: int) -> None:
        """Make room for ``length`` new input tokens behind the hot tokens (growing the hot buffers if needed)."""
        _require_positive_int("length", length)
        self._require_idle("begin_prompt_chunk()")
        for layer in self.layers:
            if layer.hot_len + length > layer.hot_k.shape[2]:
                self._resize_hot(layer, layer.hot_len + length, keep_tokens=layer.hot_len)
        self._chunk_start = [layer.hot_len for layer in self.layers]
        self._chunk_len = length
        self._phase = _Phase.PROMPT_CHUNK

    @torch.no_grad()
    def append_prompt_token(self, layer_idx: int, key: torch.Tensor, value: torch.Tensor) -> None:
        """Inside a chunk tokens are written one by one, each attended to right after, so no query sees its future."""
        self._require_chunk()
        layer = self.layer_tiers(layer_idx)
        if layer.hot_len - self._chunk_start[layer_idx] >= self._chunk_len:
            raise RuntimeError(f"第 {layer_idx} 层已写满 (layer {layer_idx} is full): all {self._chunk_len} tokens of "
                               "this prompt chunk are written")
        self._write_token(layer_idx, layer, key, value)

    @torch.no_grad()
    def finish_prompt_chunk(self) -> None:
        """Freeze the whole chunk at ``prompt_bits`` as a new prompt extension.  The hot tokens generated before the
        chunk stay as they are (float16, still subject to the usual cooling schedule); older segments are untouched."""
        self._require_chunk()
        for layer_idx, (layer, start) in enumerate(zip(self.layers, self._chunk_start)):
            written = layer.hot_len - start
            if written != self._chunk_len:
                raise RuntimeError(f"第 {layer_idx} 层 (layer {layer_idx}) prompt chunk is incomplete: "
                                   f"期望 {self._chunk_len} 个，实际 {written} 个")
        for layer, start in zip(self.layers, self._chunk_start):
            chunk_k = layer.hot_k[:, :, start:layer.hot_len, :].contiguous()
            chunk_v = layer.hot_v[:, :, start:layer.hot_len, :].contiguous()
            layer.prompt_extensions.append(_pack_kv(chunk_k, chunk_v, self.prompt_bits, self.group_size))
            self._resize_hot(layer, self.recent_window + self.lazy_g, keep_tokens=start)
            layer.hot_len = start
        self._seen_tokens += self._chunk_len
        self._chunk_len, self._chunk_start = 0, []
        self._phase = _Phase.IDLE

    # ------------------------------------------------------------------ the adapter's fused write
    @torch.no_grad()
    def append_rotated(self, layer_idx: int, query: torch.Tensor, key: torch.Tensor, value: torch.Tensor,
                       cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
        """What an attention layer does between its projections and decode attention, in one launch: rotary
        position embedding of ``query [n, Hq, hd]`` and ``key [n, Hkv, hd]`` with ``cos / sin [n, hd]``, conversion
        of all three to float16 and the write of the ``n`` new keys and ``value [n, Hkv, hd]`` into the float16
        tier.  Returns the rotated queries, float16 ``[n, Hq, hd]``.

        ``n`` is 1 in a decode step (this is ``append_hot`` then) and the whole chunk inside a prompt chunk (this
        is ``append_prompt_token`` for each of its tokens then; the caller attends with
        ``fused_phasekv_chunk_decode``, which applies the causal rule inside the chunk).  The tensors may be views
        of the projections' outputs (any token stride); batch 1."""
        layer = self.layer_tiers(layer_idx)
        in_chunk = self._phase is _Phase.PROMPT_CHUNK
        where = f"layer {layer_idx} new Q/K/V"
        for t in (query, key, value, cos, sin):
            if not isinstance(t, torch.Tensor):
                raise TypeError(f"{where} and cos/sin must be tensors")
        hkv, hd = layer.hot_k.shape[1], layer.hot_k.shape[3]
        n = query.shape[0] if query.ndim == 3 else -1
        if layer.hot_k.shape[0] != 1:
            raise ValueError("append_rotated() serves batch 1")
        if n <= 0 or query.shape[2] != hd or query.shape[1] % hkv or key.shape != (n, hkv, hd) or value.shape != key.shape:
            raise ValueError(f"{where} must be [n, Hq, {hd}] / [n, {hkv}, {hd}] / [n, {hkv}, {hd}], got "
                             f"{tuple(query.shape)}/{tuple(key.shape)}/{tuple(value.shape)}")
        if query.dtype not in (torch.float16, torch.bfloat16) or key.dtype != query.dtype or value.dtype != query.dtype:
            raise ValueError(f"{where} must all be float16 or all bfloat16")
        if cos.shape != (n, hd) or sin.shape != (n, hd) or cos.dtype != sin.dtype or cos.dtype not in _ROPE_DTYPES:
            raise ValueError(f"cos/sin must be [{n}, {hd}] of one floating dtype, got {tuple(cos.shape)}/{tuple(sin.shape)}")
        for t in (query, key, value, cos, sin):
            if t.device != layer.hot_k.device:
                raise ValueError(f"{where} must be on 同一设备 (the device of the hot tier, {layer.hot_k.device})")
            if t.stride(-1) != 1 or (t.ndim == 3 and t.stride(1) != hd):
                raise ValueError(f"{where}: heads and head_dim must be dense (only the token stride is free)")
        if in_chunk:
            if layer.hot_len - self._chunk_start[layer_idx] + n > self._chunk_len:
                raise RuntimeError(f"第 {layer_idx} 层已写满 (layer {layer_idx} is full): the prompt chunk holds "
                                   f"{self._chunk_len} tokens")
        else:
            if n != 1:
                raise ValueError(f"a decode step appends one token, got {n}; call begin_prompt_chunk(length) for new input")
            if layer_idx in self._written:
                raise RuntimeError(f"第 {layer_idx} 层在当前 decode 步已追加 (layer {layer_idx} already got this step's "
                                   "token); call finish_decode_step() after the forward pass")
        slot = layer.hot_len
        if slot + n > layer.hot_k.shape[2]:
            raise RuntimeError(f"layer {layer_idx}: hot tier is full (hot_len={slot}, capacity={layer.hot_k.shape[2]})")
        out = torch.empty((n, query.shape[1], hd), dtype=torch.float16, device=query.device)
        with torch.cuda.device(query.device):
            nv.check(nv.lib().pkv_rope_append(
                query.data_ptr(), key.data_ptr(), value.data_ptr(), _ROPE_DTYPES[query.dtype], query.stride(0),
                key.stride(0), value.stride(0), cos.data_ptr(), sin.data_ptr(), _ROPE_DTYPES[cos.dtype], cos.stride(0),
                n, query.shape[1], hkv, hd, out.data_ptr(), layer.hot_k.data_ptr(), layer.hot_v.data_ptr(),
                layer.hot_k.shape[2], slot, None, nv.stream_of(query.device)))
        layer.hot_len = slot + n
        if not in_chunk:
            self._written.add(layer_idx)
            self._phase = _Phase.DECODE_STEP
        return out

    # ------------------------------------------------------------------ shared write path
    def _write_token(self, layer_idx: int, layer: LayerTiers, key: torch.Tensor, value: torch.Tensor) -> None:
        """A failed check leaves hot_len and the step's bookkeeping unchanged."""
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
        slot = layer.hot_len
        if slot >= layer.hot_k.shape[2]:
            raise RuntimeError(f"layer {layer_idx}: hot tier is full (hot_len={slot}, capacity={layer.hot_k.shape[2]})")
        layer.hot_k[:, :, slot:slot + 1, :].copy_(key)
        layer.hot_v[:, :, slot:slot + 1, :].copy_(value)
        layer.hot_len = slot + 1

    @staticmethod
    def _resize_hot(layer: LayerTiers, capacity: int, keep_tokens: int) -> None:
        """New hot buffers of ``capacity`` token slots holding the first ``keep_tokens`` tokens of the old ones."""
        shape = (*layer.hot_k.shape[:2], capacity, layer.hot_k.shape[-1])
        new_k, new_v = layer.hot_k.new_empty(shape), layer.hot_v.new_empty(shape)
        new_k[:, :, :keep_tokens, :].copy_(layer.hot_k[:, :, :keep_tokens, :])
        new_v[:, :, :keep_tokens, :].copy_(layer.hot_v[:, :, :keep_tokens, :])
        layer.hot_k, layer.hot_v = new_k, new_v

    # ------------------------------------------------------------------ accounting and the Cache protocol
    def physical_nbytes(self) -> int:
        """Bytes of KV held, including the reserved hot capacity; scratch of packing and attention, and the unused
        part of the cold arenas, are not counted."""
        total = 0
        for layer in self.layers:
            total += sum(s.nbytes for s in (layer.prompt, *layer.prompt_extensions, *layer.cold))
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
        batch = self.layers[0].hot_k.shape[0]
        if int(beam_idx.min()) < 0 or int(beam_idx.max()) >= batch:
            raise ValueError(f"beam_idx is outside the batch range [0, {batch}) of layer 0")

        def pick(t: torch.Tensor) -> torch.Tensor:
            return t.index_select(0, beam_idx.to(t.device))

        def reorder(pt: PackedTensor) -> PackedTensor:
            return replace(pt, packed=pick(pt.packed), scale=pick(pt.scale), mins=pick(pt.mins),
                           orig_shape=(beam_idx.numel(), *pt.orig_shape[1:]))

        def reorder_segment(seg: PackedKVSegment) -> PackedKVSegment:
            return PackedKVSegment(reorder(seg.key), reorder(seg.value))

        for layer in self.layers:
            layer.prompt = reorder_segment(layer.prompt)
            layer.prompt_extensions = [reorder_segment(s) for s in layer.prompt_extensions]
            layer.cold = [reorder_segment(s) for s in layer.cold]  # now tensors of their own, no longer arena views
            layer._cold_runs = []
            layer.hot_k, layer.hot_v = pick(layer.hot_k), pick(layer.hot_v)
