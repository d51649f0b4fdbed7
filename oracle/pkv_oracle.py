"""Python face of the CPU oracle (``pkv_oracle.c``).  TEST INFRASTRUCTURE ONLY.

The functions here carry the names and argument order of the reference's
``src/phasekv/kernels/packing.py`` (``pack_low_bits`` :41, ``unpack_low_bits`` :67,
``quantize_pack`` :115, ``unpack_dequantize`` :158) and
``src/phasekv/kernels/reference.py`` (``ThreeTierKV`` :28,
``fused_decode_attention_reference`` :72), so a parity test reads like the
reference's own tests.  They run on CPU tensors only and exist to check the CUDA
path; nothing outside ``tests/``, the smoke check and the benchmark's CPU-baseline
leg may import this module.

Parity of the C restatement with the reference is pinned by ``tests/golden/``.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libpkv_oracle.so")
_PACKABLE_BITS = (2, 4, 8)


def build(force: bool = False) -> str:
    """Compile ``pkv_oracle.c`` with the Makefile next to it and return the library path."""
    src = os.path.join(_HERE, "pkv_oracle.c")
    stale = (not os.path.exists(_LIB_PATH)
             or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src))
    if force or stale:
        subprocess.run(["make", "-C", _HERE, "-B", "libpkv_oracle.so"], check=True,
                       stdout=subprocess.DEVNULL)
    return _LIB_PATH


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(_LIB_PATH)
        i64, i32, vp = ctypes.c_int64, ctypes.c_int, ctypes.c_void_p
        L.pkvo_num_threads.restype = i32
        L.pkvo_set_num_threads.argtypes = [i32]
        L.pkvo_pack_low_bits.argtypes = [vp, i64, i64, i32, vp]
        L.pkvo_unpack_low_bits.argtypes = [vp, i64, i64, i32, vp]
        L.pkvo_quantize_pack.argtypes = [vp, i64, i64, i64, i32, i64, vp, vp, vp]
        L.pkvo_unpack_dequantize.argtypes = [vp, vp, vp, i64, i64, i64, i32, i64, vp]
        L.pkvo_attention_dense.argtypes = [vp, vp, vp, i32, i32, i64, i32, vp, vp, vp, vp, vp]
        L.pkvo_value_norm_topk.argtypes = [vp, i64, i64, i32, i64, vp, vp]
        L.pkvo_fake_quant.argtypes = [vp, i64, i64, i64, i32, i64, vp]
        L.pkvo_fake_quant.restype = None
        for f in (L.pkvo_pack_low_bits, L.pkvo_unpack_low_bits, L.pkvo_quantize_pack,
                  L.pkvo_unpack_dequantize, L.pkvo_attention_dense, L.pkvo_value_norm_topk,
                  L.pkvo_set_num_threads):
            f.restype = None
        _lib = L
    return _lib


def num_threads() -> int:
    return int(lib().pkvo_num_threads())


def set_num_threads(n: int) -> None:
    lib().pkvo_set_num_threads(int(n))


def _ptr(a: np.ndarray) -> ctypes.c_void_p:
    return ctypes.c_void_p(a.ctypes.data)


def _np(t) -> np.ndarray:
    if isinstance(t, torch.Tensor):
        t = t.detach().cpu().contiguous().numpy()
    return np.ascontiguousarray(t)


def _vals_per_byte(bits: int) -> int:
    if bits not in _PACKABLE_BITS:
        raise ValueError(f"packable bit widths are {_PACKABLE_BITS}, got {bits}")
    return 8 // bits


@dataclass
class OraclePacked:
    """Field-for-field image of the reference's ``PackedTensor`` (packing.py:85-112)."""

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
        return int(self.packed.numel() + 2 * (self.scale.numel() + self.mins.numel()))


@dataclass
class ThreeTierKV:
    """Same fields as reference.py:28-40."""

    prompt_k: Optional[object] = None
    prompt_v: Optional[object] = None
    cold_k: Optional[object] = None
    cold_v: Optional[object] = None
    hot_k: Optional[torch.Tensor] = None
    hot_v: Optional[torch.Tensor] = None


def pack_low_bits(codes: torch.Tensor, bits: int) -> torch.Tensor:
    if codes.dtype != torch.uint8:
        raise ValueError(f"codes must be uint8, got {codes.dtype}")
    vpb = _vals_per_byte(bits)
    c = _np(codes)
    length = c.shape[-1]
    rows = c.size // max(length, 1) if length else 0
    out = np.zeros(c.shape[:-1] + ((length + vpb - 1) // vpb,), dtype=np.uint8)
    if c.size:
        lib().pkvo_pack_low_bits(_ptr(c), rows, length, bits, _ptr(out))
    return torch.from_numpy(out)


def unpack_low_bits(packed: torch.Tensor, bits: int, length: int) -> torch.Tensor:
    if packed.dtype != torch.uint8:
        raise ValueError(f"packed must be uint8, got {packed.dtype}")
    vpb = _vals_per_byte(bits)
    p = _np(packed)
    nbytes = p.shape[-1]
    # the reference slices [..., :length] of nbytes*vpb decoded values (packing.py:78-79)
    length_eff = min(int(length), nbytes * vpb)
    need = (length_eff + vpb - 1) // vpb
    rows = p.size // max(nbytes, 1) if nbytes else 0
    src = np.ascontiguousarray(p[..., :need])
    out = np.zeros(p.shape[:-1] + (length_eff,), dtype=np.uint8)
    if out.size:
        lib().pkvo_unpack_low_bits(_ptr(src), rows, length_eff, bits, _ptr(out))
    return torch.from_numpy(out)


def _axis_view(shape: Sequence[int], axis: int) -> Tuple[int, int, int]:
    outer = int(np.prod(shape[:axis], dtype=np.int64)) if axis > 0 else 1
    inner = int(np.prod(shape[axis + 1:], dtype=np.int64)) if axis + 1 < len(shape) else 1
    return outer, int(shape[axis]), inner


def quantize_pack(x: torch.Tensor, bits: int, axis: int, group_size: int) -> OraclePacked:
    vpb = _vals_per_byte(bits)
    orig_shape = tuple(x.shape)
    axis = axis % x.dim()
    # The reference computes on x.float(); for float16/bfloat16 input the float16 image
    # below is exact only for float16, which is what every caller on this path passes
    # (phasekv_cache.py:249 casts to float16 first).
    if x.dtype != torch.float16:
        raise ValueError("the oracle quantises float16 input, as the cache passes it")
    xa = _np(x).view(np.uint16)
    outer, A, inner = _axis_view(orig_shape, axis)
    gs = A if group_size is None or group_size <= 0 else min(int(group_size), A)
    nb, ng = (A + vpb - 1) // vpb, (A + gs - 1) // gs
    moved = tuple(s for i, s in enumerate(orig_shape) if i != axis)
    packed = np.zeros(moved + (nb,), dtype=np.uint8)
    scale = np.zeros(moved + (ng,), dtype=np.uint16)
    mins = np.zeros(moved + (ng,), dtype=np.uint16)
    lib().pkvo_quantize_pack(_ptr(xa), outer, A, inner, bits, gs, _ptr(packed), _ptr(scale), _ptr(mins))
    return OraclePacked(
        packed=torch.from_numpy(packed),
        scale=torch.from_numpy(scale.view(np.float16)),
        mins=torch.from_numpy(mins.view(np.float16)),
        bits=bits, axis=axis, group_size=gs, orig_shape=orig_shape, axis_len=A)


def unpack_dequantize(pt) -> torch.Tensor:
    """Accepts any object with the ``PackedTensor`` attributes (duck typed like reference.py:48-52)."""
    axis = pt.axis
    outer, A, inner = _axis_view(pt.orig_shape, axis)
    assert A == pt.axis_len
    packed = _np(pt.packed)
    scale = _np(pt.scale).view(np.uint16)
    mins = _np(pt.mins).view(np.uint16)
    out = np.zeros(tuple(pt.orig_shape), dtype=np.uint16)
    lib().pkvo_unpack_dequantize(_ptr(packed), _ptr(scale), _ptr(mins), outer, A, inner,
                                 pt.bits, pt.group_size, _ptr(out))
    return torch.from_numpy(out.view(np.float16))


def attention_dense(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, num_attention_heads: int,
                    want_partial: bool = False):
    """q [Hq, hd], k/v [Hkv, S, hd], all float16 -> out float16 [Hq, hd] (+ (m, l, acc) float32)."""
    hq, hd = q.shape
    hkv, S, _ = k.shape
    if hq != num_attention_heads or hq % hkv:
        raise ValueError("query heads must be a multiple of KV heads")
    qa, ka, va = (_np(t.to(torch.float16)).view(np.uint16) for t in (q, k, v))
    out = np.zeros((hq, hd), dtype=np.uint16)
    outf = np.zeros((hq, hd), dtype=np.float32)
    m = np.zeros((hq,), dtype=np.float32)
    l = np.zeros((hq,), dtype=np.float32)
    acc = np.zeros((hq, hd), dtype=np.float32)
    lib().pkvo_attention_dense(_ptr(qa), _ptr(ka), _ptr(va), hq, hkv, S, hd, _ptr(out), _ptr(outf),
                               _ptr(m), _ptr(l), _ptr(acc))
    o = torch.from_numpy(out.view(np.float16))
    if want_partial:
        return o, torch.from_numpy(outf), (torch.from_numpy(m), torch.from_numpy(l), torch.from_numpy(acc))
    return o


def _dequant_concat(kv: ThreeTierKV) -> Tuple[torch.Tensor, torch.Tensor]:
    ks: List[torch.Tensor] = []
    vs: List[torch.Tensor] = []
    if kv.prompt_k is not None:
        ks.append(unpack_dequantize(kv.prompt_k)); vs.append(unpack_dequantize(kv.prompt_v))
    if kv.cold_k is not None:
        ks.append(unpack_dequantize(kv.cold_k)); vs.append(unpack_dequantize(kv.cold_v))
    if kv.hot_k is not None:
        ks.append(kv.hot_k.cpu().to(torch.float16)); vs.append(kv.hot_v.cpu().to(torch.float16))
    if not ks:
        raise ValueError("all three tiers are empty")
    return torch.cat(ks, dim=-2), torch.cat(vs, dim=-2)


def fused_decode_attention_reference(q: torch.Tensor, kv: ThreeTierKV,
                                     num_attention_heads: int) -> torch.Tensor:
    """reference.py:72-96: q [b, Hq, q_len, hd] float16 -> [b, Hq, q_len, hd] float16."""
    if q.dim() != 4:
        raise ValueError(f"q must be [b, Hq, q_len, hd], got {tuple(q.shape)}")
    k_all, v_all = _dequant_concat(kv)
    b, hq, qlen, hd = q.shape
    out = torch.empty((b, hq, qlen, hd), dtype=torch.float16)
    qc = q.detach().cpu()
    for bi in range(b):
        for t in range(qlen):
            out[bi, :, t, :] = attention_dense(qc[bi, :, t, :], k_all[bi], v_all[bi], num_attention_heads)
    return out


def segments_decode_reference(q: torch.Tensor, segments, hot_k: Optional[torch.Tensor],
                              hot_v: Optional[torch.Tensor], num_attention_heads: int,
                              want_partial: bool = False):
    """Attention over a list of ``(key, value)`` packed segments (each ``[1, Hkv, S_i, hd]``)
    plus an optional float16 hot tier ``[1, Hkv, hot, hd]``, i.e. what
    ``fused_phasekv_decode`` (attention_triton.py:643-669) computes for ``LayerTiers``.
    q is ``[Hq, hd]``."""
    ks = [unpack_dequantize(k)[0] for k, _ in segments]
    vs = [unpack_dequantize(v)[0] for _, v in segments]
    if hot_k is not None and hot_k.shape[-2] > 0:
        ks.append(hot_k.cpu().to(torch.float16)[0]); vs.append(hot_v.cpu().to(torch.float16)[0])
    k_all, v_all = torch.cat(ks, dim=-2), torch.cat(vs, dim=-2)
    return attention_dense(q.cpu(), k_all, v_all, num_attention_heads, want_partial=want_partial)


def value_norm_topk(value: torch.Tensor, keep: int):
    """phasekv_cache.py:331-332 for value ``[..., aged, hd]`` float16: ascending indices of the
    ``keep`` rows with the largest L2 norm, and the relative gap at the keep boundary."""
    v = _np(value.to(torch.float16)).view(np.uint16)
    *lead, aged, hd = v.shape
    rows = int(np.prod(lead, dtype=np.int64)) if lead else 1
    idx = np.zeros(tuple(lead) + (keep,), dtype=np.int64)
    gap = np.zeros(tuple(lead), dtype=np.float64)
    lib().pkvo_value_norm_topk(_ptr(v), rows, aged, hd, keep, _ptr(idx), _ptr(gap))
    return torch.from_numpy(idx), torch.from_numpy(gap)


def fake_quant(x: torch.Tensor, bits: int, axis: int, group_size: int) -> torch.Tensor:
    """quant.py:34-79 ``_grouped_affine_quant_dequant``: quantise and dequantise along ``axis`` with float32
    scale and zero; same shape and dtype as ``x``; ``bits >= 16`` returns ``x``."""
    if bits >= 16:
        return x
    if bits < 1:
        raise ValueError(f"bits must be >= 1, got {bits}")
    axis = axis % x.dim()
    outer, length, inner = _axis_view(tuple(x.shape), axis)
    gs = length if group_size is None or group_size <= 0 else min(int(group_size), length)
    xf = np.ascontiguousarray(x.detach().cpu().float().contiguous().numpy())
    out = np.empty_like(xf)
    lib().pkvo_fake_quant(_ptr(xf), outer, length, inner, int(bits), gs, _ptr(out))
    return torch.from_numpy(out).to(x.dtype)


def quantize_key(key: torch.Tensor, bits: int, group_size: int = 32) -> torch.Tensor:
    """quant.py:82-91: per channel, groups of tokens (axis -2)."""
    return fake_quant(key, bits, -2, group_size)


def quantize_value(value: torch.Tensor, bits: int, group_size: int = 32) -> torch.Tensor:
    """quant.py:94-101: per token, groups along head_dim (axis -1)."""
    return fake_quant(value, bits, -1, group_size)
