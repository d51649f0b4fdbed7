"""Lazy cold-tier cooling of one layer on the GPU.

``cool_aged_tokens`` does what ``PhaseKVCache._cool_aged_tokens`` (phasekv_cache.py:322-340 of
the reference) does — value-norm top-k among the oldest hot tokens, quantise+pack of the kept
ones into a new frozen cold segment, compaction of the hot buffers — in one kernel launch.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import _native as nv
from .kernels.packing import PackedTensor, _vals_per_byte
from .kernels.tiers import LayerTiers, PackedKVSegment


def select_and_pack_cold(hot_k: torch.Tensor, hot_v: torch.Tensor, hot_len: int, aged: int, keep_count: int,
                         bits: int, group_size: int, return_indices: bool = False):
    """Cool the oldest ``aged`` tokens of ``hot_k``/``hot_v`` (``[B, Hkv, capacity, hd]`` float16,
    contiguous, modified in place: the surviving ``hot_len - aged`` tokens move to the front).

    Returns the new ``PackedKVSegment`` (and the kept positions ``[B, Hkv, keep_count]`` if asked).
    """
    nv.require_cuda(hot_k, "hot_k")
    if hot_k.dtype != torch.float16 or hot_v.dtype != torch.float16:
        raise ValueError("hot buffers must be float16")
    if not (hot_k.is_contiguous() and hot_v.is_contiguous()) or hot_k.shape != hot_v.shape:
        raise ValueError("hot buffers must be contiguous [B, Hkv, capacity, hd] of equal shape")
    vpb = _vals_per_byte(bits)
    b, hkv, capacity, hd = hot_k.shape
    if not (0 < keep_count <= aged <= hot_len <= capacity):
        raise ValueError("need 0 < keep_count <= aged <= hot_len <= capacity")
    dev = hot_k.device
    gs_k, gs_v = min(group_size, keep_count), min(group_size, hd)

    def u8(*shape):
        return torch.empty(shape, dtype=torch.uint8, device=dev)

    def f16(*shape):
        return torch.empty(shape, dtype=torch.float16, device=dev)

    kp, ks, km = u8(b, hkv, hd, -(-keep_count // vpb)), f16(b, hkv, hd, -(-keep_count // gs_k)), f16(b, hkv, hd, -(-keep_count // gs_k))
    vp, vs, vm = u8(b, hkv, keep_count, -(-hd // vpb)), f16(b, hkv, keep_count, -(-hd // gs_v)), f16(b, hkv, keep_count, -(-hd // gs_v))
    idx: Optional[torch.Tensor] = (torch.empty((b, hkv, keep_count), dtype=torch.int64, device=dev)
                                   if return_indices else None)
    with torch.cuda.device(dev):
        nv.check(nv.lib().pkv_cold_select_pack(
            hot_k.data_ptr(), hot_v.data_ptr(), b * hkv, capacity, hd, hot_len, aged, keep_count, bits,
            group_size, kp.data_ptr(), ks.data_ptr(), km.data_ptr(), vp.data_ptr(), vs.data_ptr(),
            vm.data_ptr(), nv.ptr(idx), nv.stream_of(dev)))
    shape = (b, hkv, keep_count, hd)
    seg = PackedKVSegment(
        PackedTensor(kp, ks, km, bits, 2, gs_k, shape, keep_count),
        PackedTensor(vp, vs, vm, bits, 3, gs_v, shape, hd))
    return (seg, idx) if return_indices else seg


def cool_aged_tokens(layer: LayerTiers, recent_window: int, lazy_g: int, decode_keep_ratio: float,
                     cold_bits: int, group_size: int) -> bool:
    """Apply one cooling step to ``layer`` if at least ``lazy_g`` tokens have aged out of the
    recent window; returns whether a cold segment was appended.  Frozen segments are never touched."""
    aged = layer.hot_len - recent_window
    if aged < lazy_g:
        return False
    keep_count = max(1, round(decode_keep_ratio * aged))  # Python's round: half to even
    seg = select_and_pack_cold(layer.hot_k, layer.hot_v, layer.hot_len, aged, keep_count, cold_bits, group_size)
    layer.cold.append(seg)
    layer.hot_len -= aged
    return True
