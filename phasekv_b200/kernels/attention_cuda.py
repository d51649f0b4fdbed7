"""Single-pass mixed-precision split-K decode attention over the three-tier KV cache (CUDA).

Entry points keep the names, argument order, defaults, return types and ``ValueError`` behaviour
of the reference's ``src/phasekv/kernels/attention_triton.py``:

  decode_attention_packed (:95), decode_attention_packed_splitk (:269),
  fused_three_tier_decode (:487), fused_three_tier_decode_single (:414),
  _kivi_layer_partial (:604), _fp16_layer_partial (:285), _reduce_splits (:257),
  _merge_partials (:300), fused_phasekv_decode (:643)

Differences by design: every call is ONE split-K launch over all segments of the layer (prompt,
prompt extensions, each frozen cold segment and the float16 hot buffer) plus one merge launch,
and each KV byte is read once for the whole GQA group instead of once per query head.
``block_n``/``num_warps`` are accepted, validated and otherwise advisory.
"""
from __future__ import annotations

import ctypes
from dataclasses import replace
from functools import lru_cache
from typing import List, Optional, Sequence, Tuple

import torch

from .. import _native as nv
from .launch_config import plan_kivi_decode
from .packing import PackedTensor, _vals_per_byte


@lru_cache(maxsize=32)
def _device_sm_count(device: torch.device) -> int:
    return nv.sm_count(device)


# --------------------------------------------------------------------------- segments
def _packed_segment(key: PackedTensor, value: PackedTensor, num_splits: Optional[int]) -> Tuple[nv.Segment, list]:
    """Describe one packed K/V pair with ``orig_shape == (Hkv, S, hd)`` to the kernels."""
    if len(key.orig_shape) != 3 or tuple(value.orig_shape) != tuple(key.orig_shape):
        raise ValueError("packed K/V must share an original shape [Hkv, S, hd]")
    if key.axis == 1 and value.axis == 2:
        kind = nv.PKV_SEG_KIVI
    elif key.axis == 2 and value.axis == 2:
        kind = nv.PKV_SEG_PER_TOKEN
    else:
        raise ValueError("K must be packed along tokens or head_dim, V along head_dim")
    _vals_per_byte(key.bits), _vals_per_byte(value.bits)
    k_rows = [key.packed, key.scale, key.mins]
    pitches = [0, 0]
    if kind == nv.PKV_SEG_KIVI and all(_padded_rows(t) for t in k_rows) and key.scale.stride(1) == key.mins.stride(1):
        pitches = [key.packed.stride(1), key.scale.stride(1)]  # uint8 rows: bytes; float16 rows: elements
    else:
        k_rows = [t.contiguous() for t in k_rows]
    keep = k_rows + [value.packed.contiguous(), value.scale.contiguous(), value.mins.contiguous()]
    seg = nv.Segment(*(t.data_ptr() for t in keep), int(key.orig_shape[1]), 0, kind,
                     int(key.bits), int(value.bits), int(key.group_size), int(value.group_size),
                     int(num_splits or 0), *pitches)
    return seg, keep


def _padded_rows(t: torch.Tensor) -> bool:
    """``t`` is ``[Hkv, hd, n]`` with dense elements, rows a fixed pitch apart and heads ``hd`` rows apart
    (what ``quantize_pack`` hands out for keys, or a slice of it along the last dimension)."""
    return (t.dim() == 3 and t.stride(2) == 1 and t.stride(1) >= t.shape[2]
            and (t.shape[0] == 1 or t.stride(0) == t.shape[1] * t.stride(1)))


def _fp16_segment(hot_k: torch.Tensor, hot_v: torch.Tensor) -> Tuple[nv.Segment, list]:
    """``hot_k``/``hot_v`` are ``[Hkv, hot, hd]`` views; only the token and dim strides must be dense."""
    if hot_k.dtype != torch.float16 or hot_v.dtype != torch.float16:
        hot_k, hot_v = hot_k.to(torch.float16), hot_v.to(torch.float16)
    hd = hot_k.shape[-1]

    def dense_rows(t):
        return t.stride(-1) == 1 and t.stride(-2) == hd
    if not (dense_rows(hot_k) and dense_rows(hot_v) and hot_k.stride(0) == hot_v.stride(0)):
        hot_k, hot_v = hot_k.contiguous(), hot_v.contiguous()
    head_stride = hot_k.stride(0) if hot_k.shape[0] > 1 else hot_k.shape[1] * hd
    seg = nv.Segment(hot_k.data_ptr(), None, None, hot_v.data_ptr(), None, None,
                     int(hot_k.shape[1]), int(head_stride), nv.PKV_SEG_FP16, 8, 8, 1, 1, 0, 0, 0)
    return seg, [hot_k, hot_v]


_WORKSPACES: dict = {}


def _workspace(device: torch.device, stream: int, nbytes: int) -> torch.Tensor:
    """Scratch for split-K partials, cached per (device, stream) and grown on demand."""
    key = (device.index, stream)
    ws = _WORKSPACES.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _WORKSPACES[key] = ws
    return ws


def _prepare_call(segments: Sequence[nv.Segment], hq: int, num_kv_heads: int, hd: int, dev: torch.device):
    """ctypes segment array and scratch size of one decode call (the plan is a function of lengths only)."""
    n = len(segments)
    arr = (nv.Segment * n)(*segments)
    need = ctypes.c_size_t(0)
    nv.check(nv.lib().pkv_decode_workspace_bytes(arr, n, hq, num_kv_heads, hd, _device_sm_count(dev), ctypes.byref(need)))
    return arr, n, int(need.value)


def _launch_decode(q: torch.Tensor, arr, n: int, need: int, num_kv_heads: int, want_out: bool, want_partial: bool):
    hq, hd = q.shape
    dev = q.device
    out = torch.empty((hq, hd), dtype=torch.float16, device=dev) if want_out else None
    m = l = acc = None
    if want_partial:
        m = torch.empty((hq,), dtype=torch.float32, device=dev)
        l = torch.empty((hq,), dtype=torch.float32, device=dev)
        acc = torch.empty((hq, hd), dtype=torch.float32, device=dev)
    switch = dev.index is not None and torch.cuda.current_device() != dev.index
    if switch:
        prev = torch.cuda.current_device()
        torch.cuda.set_device(dev)
    try:
        stream = nv.stream_of(dev)
        ws = _workspace(dev, stream, need)
        nv.check(nv.lib().pkv_decode_attention(q.data_ptr(), arr, n, hq, num_kv_heads, hd, 1.0 / (hd ** 0.5),
                                               _device_sm_count(dev), ws.data_ptr(), ws.numel(), nv.ptr(out), nv.ptr(m),
                                               nv.ptr(l), nv.ptr(acc), stream))
    finally:
        if switch:
            torch.cuda.set_device(prev)
    return out, (m, l, acc)


def _run_decode(q: torch.Tensor, segments: Sequence[nv.Segment], keep: list, num_attention_heads: int,
                num_kv_heads: int, want_out: bool, want_partial: bool):
    hq, hd = q.shape
    # one-off calls on tensors of unknown age: the kernel that packed them may be the one launched just before
    for seg in segments:
        seg.flags |= nv.PKV_SEG_FLAG_FRESH
    arr, n, need = _prepare_call(segments, hq, num_kv_heads, hd, q.device)
    res = _launch_decode(q, arr, n, need, num_kv_heads, want_out, want_partial)
    del keep
    return res


def _check_query(q: torch.Tensor, num_attention_heads: int, hd: int, hkv: int) -> torch.Tensor:
    nv.require_cuda(q, "q")
    if tuple(q.shape) != (num_attention_heads, hd):
        raise ValueError(f"q must be [Hq={num_attention_heads}, hd={hd}], got {tuple(q.shape)}")
    if q.dtype != torch.float16:
        raise ValueError("query must be [Hq, head_dim] float16")
    if num_attention_heads % hkv != 0:
        raise ValueError(f"Hq {num_attention_heads} is not a multiple of Hkv {hkv}")
    return q.contiguous()


# --------------------------------------------------------------------------- per-token layout
def decode_attention_packed(q: torch.Tensor, packed_k: PackedTensor, packed_v: PackedTensor,
                            num_attention_heads: int, block_n: int = 64) -> torch.Tensor:
    """Packed-KV decode attention, per-token layout (both K and V from
    ``quantize_pack(x, bits, -1, gs)`` of ``[Hkv, S, hd]``), without splitting the sequence."""
    return decode_attention_packed_splitk(q, packed_k, packed_v, num_attention_heads, 1, block_n)


def _split_request(num_splits: Optional[int], length: int) -> Optional[int]:
    return None if num_splits is None else max(1, min(int(num_splits), length))


def decode_attention_packed_splitk(q: torch.Tensor, packed_k: PackedTensor, packed_v: PackedTensor,
                                   num_attention_heads: int, num_splits: Optional[int] = 8,
                                   block_n: int = 64) -> torch.Tensor:
    """Split-K flash-decoding over one per-token-layout segment.  ``num_splits`` is honoured as given (the
    reference's default of 8 leaves most of a large GPU idle); ``None`` lets the library size the grid."""
    hkv, S, hd = packed_k.orig_shape
    q = _check_query(q, num_attention_heads, hd, hkv)
    vpb, gs = _vals_per_byte(packed_k.bits), packed_k.group_size
    if hd % vpb != 0 or hd % gs != 0:
        raise ValueError(f"head_dim({hd}) must be divisible by vpb({vpb}) and group_size({gs})")
    seg, keep = _packed_segment(packed_k, packed_v, _split_request(num_splits, S))
    out, _ = _run_decode(q, [seg], keep, num_attention_heads, hkv, True, False)
    return out


def _three_tier_segments(kv, num_splits: Optional[int]):
    segs, keep, hkv, hd = [], [], None, None
    for k, v in ((kv.prompt_k, kv.prompt_v), (kv.cold_k, kv.cold_v)):
        if k is not None:
            s, kp = _packed_segment(k, v, _split_request(num_splits, k.orig_shape[1]))
            segs.append(s), keep.extend(kp)
            hkv, _, hd = k.orig_shape
    if kv.hot_k is not None and kv.hot_k.shape[-2] > 0:
        s, kp = _fp16_segment(kv.hot_k, kv.hot_v)
        segs.append(s), keep.extend(kp)
        hkv, hd = kv.hot_k.shape[0], kv.hot_k.shape[-1]
    if not segs:
        raise ValueError("all three tiers are empty, nothing to attend to")
    return segs, keep, hkv, hd


def fused_three_tier_decode(q, kv, num_attention_heads, num_splits: Optional[int] = 8, block_n: int = 64):
    """One attention over [packed prompt] + [packed cold] + [float16 hot] (per-token layout,
    ``kv`` a ``ThreeTierKV`` with ``[Hkv, len, hd]`` tiers).  Returns ``[Hq, hd]`` float16.  ``num_splits=None``
    lets the library size the grid."""
    segs, keep, hkv, hd = _three_tier_segments(kv, num_splits)
    q = _check_query(q, num_attention_heads, hd, hkv)
    out, _ = _run_decode(q, segs, keep, num_attention_heads, hkv, True, False)
    return out


def fused_three_tier_decode_single(q, kv, num_attention_heads, num_splits: int = 32, block_n: int = 64):
    """Same result as :func:`fused_three_tier_decode`.  In the reference this is the (slower)
    one-launch variant; here every entry point already is a single split-K launch, with the
    tier chosen per work item rather than per lane."""
    return fused_three_tier_decode(q, kv, num_attention_heads, num_splits, block_n)


# --------------------------------------------------------------------------- partial algebra
def _reduce_splits(pm: torch.Tensor, pl: torch.Tensor, pacc: torch.Tensor):
    """Merge split partials laid out as the reference does, ``pm, pl [Hq, splits]`` and
    ``pacc [Hq, splits, hd]``, into one un-normalised partial ``(m [Hq], l [Hq], acc [Hq, hd])``."""
    return _merge_stacked(pm.t().contiguous().float(), pl.t().contiguous().float(),
                          pacc.transpose(0, 1).contiguous().float(), want_out=False)[1]


def _merge_stacked(m: torch.Tensor, l: torch.Tensor, acc: torch.Tensor, want_out: bool):
    """m, l ``[parts, Hq]``, acc ``[parts, Hq, hd]`` float32 contiguous."""
    nv.require_cuda(acc, "partials")
    parts, hq, hd = acc.shape
    dev = acc.device
    out = torch.empty((hq, hd), dtype=torch.float16, device=dev) if want_out else None
    mo = torch.empty((hq,), dtype=torch.float32, device=dev)
    lo = torch.empty((hq,), dtype=torch.float32, device=dev)
    ao = torch.empty((hq, hd), dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        nv.check(nv.lib().pkv_merge_partials(m.data_ptr(), l.data_ptr(), acc.data_ptr(), parts, hq, hd,
                                             nv.ptr(out), mo.data_ptr(), lo.data_ptr(), ao.data_ptr(),
                                             nv.stream_of(dev)))
    return out, (mo, lo, ao)


def _merge_partials(partials) -> torch.Tensor:
    """Log-sum-exp merge of a list of ``(m, l, acc)`` partials into the final ``[Hq, hd]`` float16."""
    m = torch.stack([p[0] for p in partials]).contiguous().float()
    l = torch.stack([p[1] for p in partials]).contiguous().float()
    acc = torch.stack([p[2] for p in partials]).contiguous().float()
    return _merge_stacked(m, l, acc, want_out=True)[0]


def _fp16_layer_partial(q, hot_k, hot_v, num_attention_heads):
    """Un-normalised partial of the float16 hot tier, ``hot_k``/``hot_v`` ``[Hkv, hot, hd]``."""
    hkv, hot, hd = hot_k.shape
    q = _check_query(q, num_attention_heads, hd, hkv)
    seg, keep = _fp16_segment(hot_k, hot_v)
    return _run_decode(q, [seg], keep, num_attention_heads, hkv, False, True)[1]


def _kivi_layer_partial(q, key: PackedTensor, value: PackedTensor, num_attention_heads: int,
                        num_splits: Optional[int] = None, block_n: Optional[int] = None,
                        num_warps: Optional[int] = None):
    """Read one real PhaseKV packed segment (K along tokens, V along head_dim, batch removed) and
    return the softmax partial ``(m, l, acc)`` that can be merged across segments."""
    if key.axis != 1 or value.axis != 2 or len(key.orig_shape) != 3:
        raise ValueError("K must be packed along the token axis and V along head_dim, with batch removed")
    hkv, seq_len, head_dim = key.orig_shape
    if tuple(value.orig_shape) != tuple(key.orig_shape) or seq_len <= 0:
        raise ValueError("packed K/V shapes differ or are empty")
    if tuple(q.shape) != (num_attention_heads, head_dim) or q.dtype != torch.float16:
        raise ValueError("query must be [Hq, head_dim] float16")
    if num_attention_heads % hkv or head_dim & (head_dim - 1):
        raise ValueError("Hq must be a multiple of Hkv and head_dim a power of two")
    if q.device != key.packed.device or q.device != value.packed.device:
        raise ValueError("query and packed K/V must be on the same device")
    nv.require_cuda(q, "q")
    # validates num_splits / block_n / num_warps exactly as the reference planner does
    plan_kivi_decode(seq_len, num_attention_heads, head_dim, _device_sm_count(q.device),
                     num_splits, block_n, num_warps)
    seg, keep = _packed_segment(key, value, num_splits)
    return _run_decode(q.contiguous(), [seg], keep, num_attention_heads, hkv, False, True)[1]


# --------------------------------------------------------------------------- the decode entry point
def _remove_batch(pt: PackedTensor) -> PackedTensor:
    if pt.orig_shape[0] != 1:
        raise ValueError("the PhaseKV decode path supports batch=1 only")
    return replace(pt, packed=pt.packed[0], scale=pt.scale[0], mins=pt.mins[0],
                   orig_shape=tuple(pt.orig_shape[1:]), axis=pt.axis - 1)


def _cached_packed_segment(segment, num_splits: Optional[int]):
    """Descriptor of a frozen packed segment of a ``LayerTiers``.  Segments are immutable once built
    (the prompt is read-only, cold segments are never re-quantised), so the descriptor is built once
    and kept on the segment object; it is rebuilt if the tensors behind it were replaced."""
    key, value = segment.key, segment.value
    tag = (key.packed.data_ptr(), value.packed.data_ptr(), key.scale.data_ptr(), value.scale.data_ptr(),
           int(num_splits or 0))
    cached = getattr(segment, "_pkv_descriptor", None)
    if cached is not None and cached[0] == tag:
        return cached[1], cached[2], cached[3]
    k, v = _remove_batch(key), _remove_batch(value)
    if k.axis != 1 or v.axis != 2:
        raise ValueError("K must be packed along the token axis and V along head_dim")
    seg, keep = _packed_segment(k, v, num_splits)
    shape = (k.orig_shape[0], k.orig_shape[2])
    try:
        segment._pkv_descriptor = (tag, seg, keep, shape)
    except AttributeError:  # objects without a __dict__ are simply not cached
        pass
    return seg, keep, shape


def _cold_descriptors(cold: Sequence, num_splits: Optional[int]):
    """Descriptors of the cold tier.  Consecutive cooling steps that are the slots 0..k-1 of one arena the
    tensor-core kernel can read (``ColdArena.decode_ready``) become ONE descriptor over the arena; every other
    step gets its own.  Yields ``(descriptor, tensors to keep alive, origin, (Hkv, hd))`` where ``origin`` is the
    arena or the segment object."""
    i = 0
    while i < len(cold):
        arena = getattr(cold[i], "_arena", None)
        if arena is not None and arena.decode_ready and getattr(cold[i], "_arena_event", -1) == 0:
            k = 1
            while (i + k < len(cold) and getattr(cold[i + k], "_arena", None) is arena
                   and cold[i + k]._arena_event == k):
                k += 1
            if k == arena.events:
                yield arena.descriptor(), list(arena.tensors()), arena, (arena.shape[1], arena.shape[2])
                i += k
                continue
        s, kp, shape = _cached_packed_segment(cold[i], num_splits)
        yield s, kp, cold[i], shape
        i += 1


def _layer_descriptors(tiers, num_splits: Optional[int] = None):
    segs: List[nv.Segment] = []
    keep: list = []
    origins: list = []
    hkv = hd = None
    for segment in [tiers.prompt, *tiers.prompt_extensions]:
        s, kp, (hkv, hd) = _cached_packed_segment(segment, num_splits)
        segs.append(s), keep.append(kp), origins.append(segment)
    for s, kp, origin, (hkv, hd) in _cold_descriptors(tiers.cold, num_splits):
        segs.append(s), keep.append(kp), origins.append(origin)
    if tiers.hot_len:
        hot_k, hot_v = tiers.hot_views()
        if hot_k.shape[0] != 1:
            raise ValueError("the PhaseKV decode path supports batch=1 only")
        s, kp = _fp16_segment(hot_k[0], hot_v[0])
        segs.append(s), keep.extend(kp)
        hkv, hd = hot_k.shape[1], hot_k.shape[3]
    return segs, keep, hkv, hd, origins


def layer_segments(tiers, num_splits: Optional[int] = None):
    """Segment descriptors for every tier of a ``LayerTiers`` (batch 1), in prompt, extensions,
    cold, hot order, plus the tensors that must stay alive while they are in use."""
    return _layer_descriptors(tiers, num_splits)[:4]


def _unread(origin) -> bool:
    """Whether a packed segment may still be being written by the kernel enqueued just before a decode launch:
    a segment object no decode launch has read yet, or an arena with a slot filled since its last launch."""
    if hasattr(origin, "launched_events"):
        return origin.events > origin.launched_events
    return not getattr(origin, "_pkv_seen", False)


def _mark_read(origin) -> None:
    if hasattr(origin, "launched_events"):
        origin.launched_events = origin.events
        return
    try:
        origin._pkv_seen = True
    except AttributeError:
        pass


def fused_phasekv_decode(q: torch.Tensor, tiers, num_attention_heads: int,
                         num_splits: Optional[int] = None, block_n: Optional[int] = None,
                         num_warps: Optional[int] = None) -> torch.Tensor:
    """Batch-1 PhaseKV decode attention for one query token: ``q`` ``[Hq, hd]`` float16 against
    ``tiers`` (what ``PhaseKVCache.layer_tiers`` returns).  The packed tiers are never expanded in
    memory; all segments, however many cold segments have been frozen, go through one launch."""
    # A decode loop calls this once per layer and token with tiers that rarely change shape: the segment array
    # and the scratch size are kept on the tiers object and reused while every segment object, the hot buffers
    # and the hot length are the same.
    hot = tiers.hot_k if tiers.hot_len else None
    cold = tiers.cold
    # frozen segments are only ever appended to their lists, so the lists' lengths and last members identify them
    # (a caller that swaps a segment in the middle of a list gets a new LayerTiers, as the cache's reorder does)
    last = cold[-1] if cold else (tiers.prompt_extensions[-1] if tiers.prompt_extensions else tiers.prompt)
    tag = (id(tiers.prompt), tiers.prompt.key.packed.data_ptr(), len(tiers.prompt_extensions), len(cold), id(last),
           last.key.packed.data_ptr(),
           None if hot is None else (hot.data_ptr(), tiers.hot_v.data_ptr(), hot.shape[2], hot.stride(1)),
           num_splits, num_attention_heads)
    cached = getattr(tiers, "_pkv_call", None)
    fresh = ()
    if cached is None or cached[0] != tag:
        segs, keep, hkv, hd, origins = _layer_descriptors(tiers, num_splits)
        arr, n, need = _prepare_call(segs, num_attention_heads, hkv, hd, q.device)
        # A packed segment this entry point has not launched over yet may have been written by the kernel that
        # was enqueued just before this call (prefill packing, a cooling step): its first launch must not read
        # it ahead of the stream dependency.  From the second launch on it is settled.
        fresh = [(i, o) for i, o in enumerate(origins) if _unread(o)]
        for i, _ in fresh:
            arr[i].flags |= nv.PKV_SEG_FLAG_FRESH
        cached = [tag, arr, n, need, keep, hkv, hd, tiers.hot_len]
        # reusable only if the hot descriptor points into the caller's own buffers (a strided hot buffer is
        # described through a dense copy, which the next call must refresh)
        in_place = hot is None or (keep[-2].data_ptr() == hot.data_ptr() and keep[-1].data_ptr() == tiers.hot_v.data_ptr())
        try:
            tiers._pkv_call = cached if in_place else None
        except AttributeError:
            pass
    elif cached[7] != tiers.hot_len:
        # one more token in the same hot buffers: only the last descriptor's length and the scratch size change
        arr, n, hkv, hd = cached[1], cached[2], cached[5], cached[6]
        arr[n - 1].seq_len = tiers.hot_len
        need = ctypes.c_size_t(0)
        nv.check(nv.lib().pkv_decode_workspace_bytes(arr, n, num_attention_heads, hkv, hd, _device_sm_count(q.device),
                                                     ctypes.byref(need)))
        cached[3], cached[7] = int(need.value), tiers.hot_len
    arr, n, need, hkv, hd = cached[1], cached[2], cached[3], cached[5], cached[6]
    q = _check_query(q, num_attention_heads, hd, hkv)
    if hd & (hd - 1):
        raise ValueError("head_dim must be a power of two")
    plan_kivi_decode(max(1, tiers.prompt.length), num_attention_heads, hd, _device_sm_count(q.device),
                     num_splits, block_n, num_warps)
    out, _ = _launch_decode(q, arr, n, need, hkv, True, False)
    for i, origin in fresh:
        arr[i].flags &= ~nv.PKV_SEG_FLAG_FRESH
        _mark_read(origin)
    return out

# --------------------------------------------------------------------------- batched serving
class BatchDecodePlan:
    """Work list for one layer of a batch of sequences, resident on the device.

    The reference serves a batch by looping ``fused_phasekv_decode`` over sequences (it raises for
    ``orig_shape[0] != 1``, attention_triton.py:655-657).  Here all sequences of a layer go through one
    split-K launch and one merge launch; the plan (segment descriptors, work items of balanced cost,
    per-sequence ranges of partials) is built on the host from lengths and pointers and stays valid
    until one of them changes, e.g. for the frozen tiers between two cooling steps.
    """

    def __init__(self, tiers_list: Sequence, num_attention_heads: int):
        if not tiers_list:
            raise ValueError("empty batch")
        segs: List[nv.Segment] = []
        offsets = [0]
        self._keep: list = []
        hkv = hd = None
        for tiers in tiers_list:
            s, keep, hkv_i, hd_i = layer_segments(tiers)
            if hkv is not None and (hkv_i, hd_i) != (hkv, hd):
                raise ValueError("all sequences of a batch must share the KV head count and head_dim")
            hkv, hd = hkv_i, hd_i
            segs.extend(s)
            self._keep.append(keep)
            offsets.append(len(segs))
        if num_attention_heads % hkv != 0:
            raise ValueError(f"Hq {num_attention_heads} is not a multiple of Hkv {hkv}")
        self.batch, self.num_q_heads, self.num_kv_heads, self.head_dim = len(tiers_list), num_attention_heads, hkv, hd
        first = tiers_list[0]
        self.device = (first.hot_k if first.hot_len else first.prompt.key.packed).device
        L = nv.lib()
        arr = (nv.Segment * len(segs))(*segs)
        off = (ctypes.c_int32 * len(offsets))(*offsets)
        tb, wb = ctypes.c_size_t(0), ctypes.c_size_t(0)
        sms = _device_sm_count(self.device)
        nv.check(L.pkv_decode_batch_plan(arr, off, self.batch, num_attention_heads, hkv, hd, sms, None, 0,
                                         ctypes.byref(tb), ctypes.byref(wb)))
        self.table_host = torch.empty(tb.value, dtype=torch.uint8, pin_memory=True)
        nv.check(L.pkv_decode_batch_plan(arr, off, self.batch, num_attention_heads, hkv, hd, sms,
                                         self.table_host.data_ptr(), tb.value, ctypes.byref(tb), ctypes.byref(wb)))
        self.workspace_bytes = int(wb.value)
        self.table_device = self.table_host.to(self.device, non_blocking=True)
        self.work_items = int(self.table_host[12:16].view(torch.int32).item())

    def run(self, q: torch.Tensor) -> torch.Tensor:
        nv.require_cuda(q, "q")
        if tuple(q.shape) != (self.batch, self.num_q_heads, self.head_dim) or q.dtype != torch.float16:
            raise ValueError(f"q must be float16 [{self.batch}, {self.num_q_heads}, {self.head_dim}]")
        q = q.contiguous()
        out = torch.empty_like(q)
        with torch.cuda.device(self.device):
            stream = nv.stream_of(self.device)
            ws = _workspace(self.device, stream, self.workspace_bytes)
            nv.check(nv.lib().pkv_decode_attention_batched(
                q.data_ptr(), self.table_host.data_ptr(), self.table_device.data_ptr(),
                1.0 / (self.head_dim ** 0.5), ws.data_ptr(), ws.numel(), out.data_ptr(), stream))
        return out


def fused_phasekv_chunk_decode(q: torch.Tensor, tiers, num_attention_heads: int) -> torch.Tensor:
    """Causal attention of a chunk of ``n`` new tokens against one layer: ``q`` float16 ``[n, Hq, hd]``, ``tiers`` a
    ``LayerTiers`` whose float16 tier ALREADY holds the chunk's ``n`` keys and values at its end
    (``PhaseKVCache.append_rotated`` or ``n`` calls of ``append_prompt_token``).  Row ``i`` of the result
    ``[n, Hq, hd]`` equals what the reference computes token by token (``qwen2_attention.py:99-106``): query
    ``i`` against every packed tier and the float16 tokens up to and including its own.

    All ``n`` queries go through one split-K launch and one merge launch when the layer's layout is the
    tensor-core kernel's (head_dim 128, group 32, GQA group <= 8); other layouts are served query by query."""
    nv.require_cuda(q, "q")
    if q.ndim != 3 or q.dtype != torch.float16 or q.shape[1] != num_attention_heads:
        raise ValueError(f"q must be float16 [n, Hq={num_attention_heads}, hd], got {q.dtype} {tuple(q.shape)}")
    n = q.shape[0]
    if n == 0 or tiers.hot_len < n:
        raise ValueError(f"the float16 tier holds {tiers.hot_len} tokens, fewer than the chunk's {n}")
    q = q.contiguous()
    segs, keep, hkv, hd, origins = _layer_descriptors(tiers)
    if q.shape[2] != hd or num_attention_heads % hkv:
        raise ValueError(f"q {tuple(q.shape)} does not fit Hkv={hkv}, hd={hd}")
    fresh = [(i, o) for i, o in enumerate(origins) if _unread(o)]
    for i, _ in fresh:
        segs[i].flags |= nv.PKV_SEG_FLAG_FRESH
    dev = q.device
    L = nv.lib()
    arr = (nv.Segment * len(segs))(*segs)
    sms = _device_sm_count(dev)
    tb, wb = ctypes.c_size_t(0), ctypes.c_size_t(0)
    rc = L.pkv_decode_chunk_plan(arr, len(segs), n, num_attention_heads, hkv, hd, sms, None, 0,
                                 ctypes.byref(tb), ctypes.byref(wb))
    out = torch.empty_like(q)
    if rc == nv.PKV_E_LAYOUT:
        need = ctypes.c_size_t(0)
        hot_len = arr[len(segs) - 1].seq_len
        for i in range(n):
            arr[len(segs) - 1].seq_len = hot_len - (n - 1 - i)
            nv.check(L.pkv_decode_workspace_bytes(arr, len(segs), num_attention_heads, hkv, hd, sms, ctypes.byref(need)))
            out[i] = _launch_decode(q[i], arr, len(segs), int(need.value), hkv, True, False)[0]
    else:
        nv.check(rc)
        table_host = torch.empty(tb.value, dtype=torch.uint8, pin_memory=True)  # from torch's cached pinned blocks
        nv.check(L.pkv_decode_chunk_plan(arr, len(segs), n, num_attention_heads, hkv, hd, sms, table_host.data_ptr(),
                                         tb.value, ctypes.byref(tb), ctypes.byref(wb)))
        with torch.cuda.device(dev):
            # (torch's pinned-memory allocator keeps the block alive until this asynchronous copy has run)
            table_device = table_host.to(dev, non_blocking=True)
            stream = nv.stream_of(dev)
            ws = _workspace(dev, stream, int(wb.value))
            nv.check(L.pkv_decode_attention_batched(q.data_ptr(), table_host.data_ptr(), table_device.data_ptr(),
                                                    1.0 / (hd ** 0.5), ws.data_ptr(), ws.numel(), out.data_ptr(), stream))
    for _, origin in fresh:
        _mark_read(origin)
    del keep
    return out


def fused_phasekv_decode_batched(q: torch.Tensor, tiers_list, num_attention_heads: int) -> torch.Tensor:
    """``q`` float16 ``[B, Hq, hd]`` against ``tiers_list`` (one ``LayerTiers`` per sequence, or a
    ``BatchDecodePlan`` built from them) -> float16 ``[B, Hq, hd]``, row ``i`` equal to
    ``fused_phasekv_decode(q[i], tiers_list[i], Hq)``."""
    plan = tiers_list if isinstance(tiers_list, BatchDecodePlan) else BatchDecodePlan(tiers_list, num_attention_heads)
    return plan.run(q)
