"""The cold tier of a layer as pre-allocated arenas, filled in place by the cooling kernel.

The reference appends one small ``PackedKVSegment`` per cooling step to a Python list
(``phasekv_cache.py:322-340``); with its defaults (window 32, batch 16, half kept) that is a segment of
8 tokens every 16 generated tokens, each with its own key quantisation group, and a decode step walks all of
them one by one.  Here the steps of a layer land in an *arena*: tensors shaped like ONE packed segment in
which every step owns a slot of ``ceil(keep / group) * group`` tokens.  The step's tokens sit at the start of
its slot, the slot's key groups are the step's own groups, the rest of the slot is zero padding that the
decode kernels mask out (``pkv_segment_t.slot_tokens / slot_valid``).  So

* the decode kernels see one segment per run of equal-sized steps instead of one per step;
* cooling allocates nothing and all layers of a model cool in one launch (``pkv_cold_select_pack_layers``
  reads a device-resident table of the layers' buffers);
* every step is still available as the reference's ``PackedKVSegment`` (``views``): its tensors are views
  into the arena whose contents are bit-identical to what the reference's per-step packing produces.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional

import torch

from . import _native as nv
from .kernels.packing import PackedTensor, _vals_per_byte
from .kernels.tiers import PackedKVSegment


class ColdArena:
    """A run of cooling steps that all kept ``keep`` tokens, for one layer."""

    def __init__(self, like: torch.Tensor, bits: int, group_size: int, keep: int, max_events: int = 64):
        b, hkv, _, hd = like.shape
        self.bits, self.group_size, self.keep = bits, group_size, keep
        self.vpb = _vals_per_byte(bits)
        self.slot_tokens = -(-keep // group_size) * group_size
        if (self.slot_tokens * bits) % 8:
            raise ValueError("a slot must be a whole number of bytes")
        self.slot_bytes = self.slot_tokens * bits // 8
        self.groups_per_event = self.slot_tokens // group_size
        self.gs_k, self.gs_v = min(group_size, keep), min(group_size, hd)
        self.shape = (b, hkv, hd)
        self.device = like.device
        self.events = 0
        self.launched_events = 0   # events a decode launch has already read
        self.views: List[PackedKVSegment] = []
        self._allocate(max_events)

    # ------------------------------------------------------------------ storage
    def _allocate(self, max_events: int) -> None:
        b, hkv, hd = self.shape
        dev = self.device
        tokens = max_events * self.slot_tokens

        def zeros(shape, dtype):
            return torch.zeros(shape, dtype=dtype, device=dev)
        self.max_events = max_events
        self.k_packed = zeros((b, hkv, hd, max_events * self.slot_bytes), torch.uint8)
        self.k_scale = zeros((b, hkv, hd, max_events * self.groups_per_event), torch.float16)
        self.k_mins = zeros((b, hkv, hd, max_events * self.groups_per_event), torch.float16)
        self.v_packed = zeros((b, hkv, tokens, -(-hd // self.vpb)), torch.uint8)
        self.v_scale = zeros((b, hkv, tokens, -(-hd // self.gs_v)), torch.float16)
        self.v_mins = zeros((b, hkv, tokens, -(-hd // self.gs_v)), torch.float16)

    def tensors(self):
        return (self.k_packed, self.k_scale, self.k_mins, self.v_packed, self.v_scale, self.v_mins)

    def grow(self) -> None:
        """Double the capacity (the steps recorded so far are copied; their views are rebuilt)."""
        old = self.tensors()
        old_events, old_tokens = self.max_events, self.max_events * self.slot_tokens
        self._allocate(2 * old_events)
        new = self.tensors()
        for o, n in zip(old[:3], new[:3]):
            n[..., :o.shape[-1]].copy_(o)
        for o, n in zip(old[3:], new[3:]):
            n[:, :, :old_tokens, :].copy_(o)
        self.views = [self._view(e) for e in range(self.events)]
        self.launched_events = 0  # the copies above are the kernels the next decode launch follows

    @property
    def full(self) -> bool:
        return self.events >= self.max_events

    # ------------------------------------------------------------------ the reference's per-step segments
    def _view(self, e: int) -> PackedKVSegment:
        b, hkv, hd = self.shape
        keep, st = self.keep, self.slot_tokens
        kb0, g0, t0 = e * self.slot_bytes, e * self.groups_per_event, e * st
        n_groups = -(-keep // self.gs_k)
        shape = (b, hkv, keep, hd)
        key = PackedTensor(self.k_packed[..., kb0:kb0 + -(-keep // self.vpb)], self.k_scale[..., g0:g0 + n_groups],
                           self.k_mins[..., g0:g0 + n_groups], self.bits, 2, self.gs_k, shape, keep)
        value = PackedTensor(self.v_packed[:, :, t0:t0 + keep, :], self.v_scale[:, :, t0:t0 + keep, :],
                             self.v_mins[:, :, t0:t0 + keep, :], self.bits, 3, self.gs_v, shape, hd)
        seg = PackedKVSegment(key, value)
        seg._arena, seg._arena_event = self, e   # lets the decode entry points read the run as one segment
        return seg

    def commit_event(self) -> PackedKVSegment:
        """Record that the cooling kernel has filled slot ``events``; returns that step's segment."""
        seg = self._view(self.events)
        self.views.append(seg)
        self.events += 1
        return seg

    # ------------------------------------------------------------------ the decode kernels' view
    @property
    def decode_ready(self) -> bool:
        """Whether the tensor-core kernel can take the arena as one segment (otherwise the steps are described
        one by one)."""
        return self.shape[0] == 1 and self.group_size == 32 and self.slot_tokens in (32, 64) and self.shape[2] == 128

    def descriptor(self) -> nv.Segment:
        """One ``pkv_segment_t`` over all recorded steps (batch 1)."""
        tokens = self.max_events * self.slot_tokens
        seg = nv.Segment(self.k_packed.data_ptr(), self.k_scale.data_ptr(), self.k_mins.data_ptr(),
                         self.v_packed.data_ptr(), self.v_scale.data_ptr(), self.v_mins.data_ptr(),
                         self.events * self.slot_tokens, tokens, nv.PKV_SEG_KIVI, self.bits, self.bits,
                         self.group_size, self.gs_v, 0, self.k_packed.shape[-1], self.k_scale.shape[-1], 0,
                         self.slot_tokens, self.keep)
        return seg


class CoolingTable:
    """Device-resident table of the layers' hot buffers and arena bases for the all-layers cooling launch.  It is
    rebuilt (one small host-to-device copy) only when one of the buffers was replaced."""

    def __init__(self):
        self._key = None
        self._table: Optional[torch.Tensor] = None

    def get(self, hot: List[tuple], arenas: List[ColdArena]) -> torch.Tensor:
        rows = []
        for (hk, hv), a in zip(hot, arenas):
            rows.append((hk.data_ptr(), hv.data_ptr(), *(t.data_ptr() for t in a.tensors()), 0))
        key = tuple(rows)
        if key != self._key:
            host = torch.tensor(rows, dtype=torch.int64)
            assert host.shape[1] * 8 == ctypes.sizeof(nv.ColdLayer)
            self._table = host.to(hot[0][0].device)
            self._key = key
        return self._table


def cool_layers_into_arenas(hot: List[tuple], arenas: List[ColdArena], table: CoolingTable, hot_len: int, aged: int,
                            keep: int, bits: int, group_size: int) -> None:
    """One launch: in every layer select the ``keep`` aged tokens with the largest value norm, quantise and pack them
    into the next slot of the layer's arena and move the surviving hot tokens to the front of the hot buffers."""
    first = arenas[0]
    b, hkv, capacity, hd = hot[0][0].shape
    e = first.events
    dev = hot[0][0].device
    with torch.cuda.device(dev):
        nv.check(nv.lib().pkv_cold_select_pack_layers(
            table.get(hot, arenas).data_ptr(), len(arenas), b * hkv, capacity, hd, hot_len, aged, keep, bits, group_size,
            first.k_packed.shape[-1], first.k_scale.shape[-1], first.max_events * first.slot_tokens,
            e * first.slot_bytes, e * first.groups_per_event, e * first.slot_tokens, nv.stream_of(dev)))
