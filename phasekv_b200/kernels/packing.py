"""Real sub-byte packing for the prompt and cold tiers, on CUDA.

Same surface as the reference's ``src/phasekv/kernels/packing.py``: ``pack_low_bits`` (:41),
``unpack_low_bits`` (:67), ``PackedTensor`` (:85), ``quantize_pack`` (:115) and
``unpack_dequantize`` (:158), with the same layouts, so a ``PackedTensor`` made here can be
handed to the reference's own ``unpack_dequantize`` and vice versa.  Every function runs a
hand-written sm_100a kernel through the C ABI; CPU tensors are rejected (there is no fallback).

Codes, scales and zeros are bit-identical to the reference executed on a CPU.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Tuple

import torch

from .. import _native as nv

_BITS_PER_BYTE = 8
_PACKABLE_BITS = (2, 4, 8)
#: bytes of metadata per quantisation group (float16 scale + float16 zero)
SCALE_MIN_BYTES = 4


def _vals_per_byte(bits: int) -> int:
    if bits not in _PACKABLE_BITS:
        raise ValueError(f"packable bit widths are {_PACKABLE_BITS}, got {bits}")
    return _BITS_PER_BYTE // bits


def pack_low_bits(codes: torch.Tensor, bits: int) -> torch.Tensor:
    """Pack ``bits``-wide integer codes along the last dim into uint8 (little-endian in the byte)."""
    if codes.dtype != torch.uint8:
        raise ValueError(f"codes must be uint8, got {codes.dtype}")
    vpb = _vals_per_byte(bits)
    nv.require_cuda(codes, "codes")
    codes = codes.contiguous()
    if bits == _BITS_PER_BYTE:
        return codes
    length = codes.shape[-1]
    rows = codes.numel() // length if length else 0
    out = torch.empty(*codes.shape[:-1], (length + vpb - 1) // vpb, dtype=torch.uint8, device=codes.device)
    with torch.cuda.device(codes.device):
        nv.check(nv.lib().pkv_pack_low_bits(nv.ptr(codes), rows, length, bits, nv.ptr(out),
                                            nv.stream_of(codes.device)))
    return out


def unpack_low_bits(packed: torch.Tensor, bits: int, length: int) -> torch.Tensor:
    """Inverse of :func:`pack_low_bits`: the first ``length`` codes of every row."""
    if packed.dtype != torch.uint8:
        raise ValueError(f"packed must be uint8, got {packed.dtype}")
    vpb = _vals_per_byte(bits)
    nv.require_cuda(packed, "packed")
    packed = packed.contiguous()
    if bits == _BITS_PER_BYTE:
        return packed[..., :length].contiguous()
    row_bytes = packed.shape[-1]
    length = min(int(length), row_bytes * vpb)  # slicing semantics of the reference
    rows = packed.numel() // row_bytes if row_bytes else 0
    out = torch.empty(*packed.shape[:-1], length, dtype=torch.uint8, device=packed.device)
    with torch.cuda.device(packed.device):
        nv.check(nv.lib().pkv_unpack_low_bits(nv.ptr(packed), rows, row_bytes, length, bits, nv.ptr(out),
                                              nv.stream_of(packed.device)))
    return out


@dataclass
class PackedTensor:
    """A stretch of K or V as it lives in HBM.

    packed     : uint8 codes, the quantisation axis moved last and packed.
    scale, mins: float16 per-group parameters ``[..., n_groups]`` (axis last).
    bits       : code width.
    axis       : quantisation axis of the original tensor (non-negative).
    group_size : group length (clamped to the axis length).
    orig_shape : shape of the original tensor.
    axis_len   : real length of the quantisation axis.
    """

    packed: torch.Tensor
    scale: torch.Tensor
    mins: torch.Tensor
    bits: int
    axis: int
    group_size: int
    orig_shape: Tuple[int, ...]
    axis_len: int

    @property
    def nbytes(self) -> int:
        """Physical bytes: packed codes plus float16 scale and zero."""
        return int(self.packed.numel() + 2 * (self.scale.numel() + self.mins.numel()))


def _axis_view(shape, axis: int):
    outer = 1
    for s in shape[:axis]:
        outer *= int(s)
    inner = 1
    for s in shape[axis + 1:]:
        inner *= int(s)
    return outer, int(shape[axis]), inner


#: tile geometry of the decode kernel that padded key rows are sized for
KEY_TILE_TOKENS, KEY_TILE_GROUP = 64, 32


def quantize_pack(x: torch.Tensor, bits: int, axis: int, group_size: int) -> PackedTensor:
    """Grouped asymmetric min-max quantisation along ``axis`` with the codes really packed.

    ``scale = max(max - min, 1e-8) / qmax``, ``code = round((x - min) / scale)`` (half to even),
    scale and zero stored as float16.  K of a cache uses ``axis=-2`` (per channel, groups of
    tokens), V uses ``axis=-1`` (per token).
    """
    if bits not in _PACKABLE_BITS:
        raise ValueError(f"bits must be one of {_PACKABLE_BITS}, got {bits}")
    nv.require_cuda(x, "x")
    if x.dtype != torch.float16:
        raise ValueError(f"x must be float16 (cast it first, as the cache does), got {x.dtype}")
    if x.dim() == 0 or x.numel() == 0:
        raise ValueError("x must be a non-empty tensor")
    vpb = _vals_per_byte(bits)
    orig_shape = tuple(x.shape)
    axis = axis % x.dim()
    x = x.contiguous()
    outer, length, inner = _axis_view(orig_shape, axis)
    gs = length if group_size is None or group_size <= 0 else min(int(group_size), length)
    moved = tuple(s for i, s in enumerate(orig_shape) if i != axis)
    dev = x.device
    nb, n_groups = (length + vpb - 1) // vpb, (length + gs - 1) // gs
    # Key layout (the axis is not the last dimension, rows are long): pad the rows of the outputs to whole
    # 64-token tiles so that the decode kernel can stream a segment of any length with 16-byte copies.  The
    # tensors handed back are views of the logical shape; the padding is never read as data.
    row_bytes, row_groups = nb, n_groups
    if inner > 1 and gs == KEY_TILE_GROUP:
        tiles = (length + KEY_TILE_TOKENS - 1) // KEY_TILE_TOKENS
        row_bytes = tiles * KEY_TILE_TOKENS // vpb
        row_groups = (tiles * (KEY_TILE_TOKENS // KEY_TILE_GROUP) + 7) // 8 * 8
    packed = torch.empty(*moved, row_bytes, dtype=torch.uint8, device=dev)[..., :nb]
    scale = torch.empty(*moved, row_groups, dtype=torch.float16, device=dev)[..., :n_groups]
    mins = torch.empty(*moved, row_groups, dtype=torch.float16, device=dev)[..., :n_groups]
    with torch.cuda.device(dev):
        nv.check(nv.lib().pkv_quantize_pack_pitched(nv.ptr(x), outer, length, inner, bits, gs, nv.ptr(packed),
                                                    nv.ptr(scale), nv.ptr(mins), row_bytes, row_groups,
                                                    nv.stream_of(dev)))
    return PackedTensor(packed=packed, scale=scale, mins=mins, bits=bits, axis=axis, group_size=gs,
                        orig_shape=orig_shape, axis_len=length)


def unpack_dequantize(pt: PackedTensor) -> torch.Tensor:
    """Inverse of :func:`quantize_pack`: float16 tensor of ``pt.orig_shape``."""
    nv.require_cuda(pt.packed, "pt.packed")
    _vals_per_byte(pt.bits)
    outer, length, inner = _axis_view(pt.orig_shape, pt.axis)
    dev = pt.packed.device
    out = torch.empty(tuple(pt.orig_shape), dtype=torch.float16, device=dev)
    packed, scale, mins = pt.packed.contiguous(), pt.scale.contiguous(), pt.mins.contiguous()
    with torch.cuda.device(dev):
        nv.check(nv.lib().pkv_unpack_dequantize(nv.ptr(packed), nv.ptr(scale), nv.ptr(mins), outer, length,
                                                inner, pt.bits, pt.group_size, nv.ptr(out),
                                                nv.stream_of(dev)))
    return out
