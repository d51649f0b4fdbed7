"""Stage-A quantisation operators on CUDA: quantise-and-dequantise ("fake quantisation") of dense K/V.

Same surface as the reference's ``src/phasekv/quant.py``: ``quantize_key`` (:82), ``quantize_value`` (:94),
``quantize_kv`` (:104), ``_grouped_affine_quant_dequant`` (:34) and the logical-byte accounting
``kv_group_counts`` (:113), ``quantized_tier_bytes`` (:131), ``fp16_tier_bytes`` (:152).  K is quantised per
channel (groups of tokens), V per token (groups along head_dim); scale and zero are float32 here (the packed
path of ``kernels/packing.py`` stores them as float16), so the two differ by up to 0.004 on N(0, 1) data.
One launch per call, bit-identical to the reference executed on a CPU.  ``fake_quant_`` is the in-place form the
tier modules use on a token slice of a cache tensor without copying it out and back.
"""
from __future__ import annotations

from typing import Tuple

import torch

from . import _native as nv

#: metadata bytes per quantisation group (float16 scale + float16 zero in the logical accounting)
SCALE_ZERO_BYTES: int = 4

_DTYPES = {torch.float16: 0, torch.bfloat16: 1, torch.float32: 2}


def _ceil_div(a: int, b: int) -> int:
    return (a + b - 1) // b


def _dtype_code(t: torch.Tensor) -> int:
    try:
        return _DTYPES[t.dtype]
    except KeyError:
        raise ValueError(f"fake quantisation takes float16, bfloat16 or float32, got {t.dtype}") from None


def _launch(src: torch.Tensor, dst: torch.Tensor, outer: int, length: int, inner: int, outer_stride: int,
            bits: int, gs: int) -> None:
    with torch.cuda.device(src.device):
        nv.check(nv.lib().pkv_fake_quant(src.data_ptr(), dst.data_ptr(), _dtype_code(src), outer, length, inner,
                                         outer_stride, int(bits), gs, nv.stream_of(src.device)))


def _grouped_affine_quant_dequant(x: torch.Tensor, bits: int, axis: int, group_size: int) -> torch.Tensor:
    """Asymmetric min-max quantisation along ``axis`` in groups of ``group_size`` (<= 0: the whole axis),
    immediately dequantised; same shape and dtype as ``x``.  ``bits >= 16`` returns ``x`` itself."""
    if bits >= 16:
        return x
    if bits < 1:
        raise ValueError(f"bits must be >= 1, got {bits}")
    nv.require_cuda(x, "x")
    axis = axis % x.dim()
    xc = x.contiguous()
    outer = 1
    for s in xc.shape[:axis]:
        outer *= int(s)
    inner = 1
    for s in xc.shape[axis + 1:]:
        inner *= int(s)
    length = int(xc.shape[axis])
    if xc.numel() == 0:
        return xc.clone()
    gs = length if group_size is None or group_size <= 0 else min(int(group_size), length)
    out = torch.empty_like(xc)
    _launch(xc, out, outer, length, inner, 0, bits, gs)
    return out


def fake_quant_(cache_tensor: torch.Tensor, start: int, stop: int, bits: int, axis: int, group_size: int) -> None:
    """In place on tokens ``[start, stop)`` of a contiguous cache tensor ``[B, Hkv, S, hd]``: what
    ``t[:, :, start:stop, :] = quantize_key/value(t[:, :, start:stop, :], bits, group_size)`` does in the
    reference (prompt_tier.py:107-118, decode_tier.py:78-88), without the copy out and back.
    ``axis`` is -2 (key: groups of tokens) or -1 (value: groups along head_dim)."""
    if bits >= 16 or stop <= start:
        return
    if bits < 1:
        raise ValueError(f"bits must be >= 1, got {bits}")
    nv.require_cuda(cache_tensor, "cache tensor")
    if cache_tensor.dim() != 4 or not cache_tensor.is_contiguous():
        raise ValueError("cache tensor must be a contiguous [B, Hkv, S, hd] tensor")
    b, h, seq, hd = cache_tensor.shape
    if not 0 <= start < stop <= seq:
        raise ValueError(f"token slice [{start}, {stop}) is outside [0, {seq})")
    n = stop - start
    view = cache_tensor[:, :, start:stop, :]
    if axis in (-2, 2):
        gs = n if group_size is None or group_size <= 0 else min(int(group_size), n)
        _launch(view, view, b * h, n, hd, seq * hd, bits, gs)
    elif axis in (-1, 3):
        gs = hd if group_size is None or group_size <= 0 else min(int(group_size), hd)
        if hd % gs == 0:
            # whole groups tile every token row, so the n*hd elements of a (b, h) block are just consecutive
            # groups: one launch over [B*H, n*hd, 1] with the blocks seq*hd apart
            _launch(view, view, b * h, n * hd, 1, seq * hd, bits, gs)
        else:  # a ragged last group per token: token rows one (b, h) block at a time
            for bi in range(b):
                for hi in range(h):
                    rows = view[bi, hi]
                    _launch(rows, rows, n, hd, 1, 0, bits, gs)
    else:
        raise ValueError("axis must be -2 (key) or -1 (value)")


def quantize_key(key: torch.Tensor, bits: int, group_size: int = 32) -> torch.Tensor:
    """Per-channel fake quantisation of K ``[..., seq, head_dim]``: groups of tokens for every channel."""
    if key.dim() < 2:
        raise ValueError("key needs at least [..., seq, head_dim]")
    return _grouped_affine_quant_dequant(key, bits, axis=-2, group_size=group_size)


def quantize_value(value: torch.Tensor, bits: int, group_size: int = 32) -> torch.Tensor:
    """Per-token fake quantisation of V ``[..., seq, head_dim]``: groups along head_dim for every token."""
    if value.dim() < 1:
        raise ValueError("value needs at least one dimension")
    return _grouped_affine_quant_dequant(value, bits, axis=-1, group_size=group_size)


def quantize_kv(key: torch.Tensor, value: torch.Tensor, k_bits: int, v_bits: int,
                group_size: int = 32) -> Tuple[torch.Tensor, torch.Tensor]:
    return quantize_key(key, k_bits, group_size), quantize_value(value, v_bits, group_size)


def kv_group_counts(num_tokens: int, head_dim: int, group_size: int) -> Tuple[int, int]:
    """Quantisation groups of K and of V for one (layer, head): K has ``head_dim * ceil(tokens / gs)``,
    V has ``tokens * ceil(head_dim / gs)``, each group size clamped to its axis (<= 0: whole axis)."""
    if num_tokens <= 0:
        return 0, 0
    whole = group_size is None or group_size <= 0
    gs_token = num_tokens if whole else min(group_size, num_tokens)
    gs_dim = head_dim if whole else min(group_size, head_dim)
    return head_dim * _ceil_div(num_tokens, gs_token), num_tokens * _ceil_div(head_dim, gs_dim)


def quantized_tier_bytes(num_tokens: int, num_layers: int, num_kv_heads: int, head_dim: int, k_bits: int,
                         v_bits: int, group_size: int = 32, batch: int = 1) -> int:
    """Logical bytes of a quantised tier: code bits of K and V plus 4 bytes per group for widths below 16."""
    if num_tokens <= 0:
        return 0
    fan = batch * num_layers * num_kv_heads
    data_bits = fan * num_tokens * head_dim * (k_bits + v_bits)
    k_groups, v_groups = kv_group_counts(num_tokens, head_dim, group_size)
    overhead = 0
    if k_bits < 16:
        overhead += fan * k_groups * SCALE_ZERO_BYTES
    if v_bits < 16:
        overhead += fan * v_groups * SCALE_ZERO_BYTES
    return data_bits // 8 + overhead


def fp16_tier_bytes(num_tokens: int, num_layers: int, num_kv_heads: int, head_dim: int, batch: int = 1) -> int:
    """Logical bytes of a float16 tier (K and V, two bytes each)."""
    if num_tokens <= 0:
        return 0
    return 2 * batch * num_layers * num_kv_heads * num_tokens * head_dim * 2
