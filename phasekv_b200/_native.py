"""ctypes binding of ``libphasekv_b200.so`` (declared in include/phasekv_b200.h).

There is no fallback of any kind: if the library is missing or a call fails, an exception is
raised.  torch is used only to own device memory and name the current stream.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libphasekv_b200.so")

PKV_SEG_KIVI, PKV_SEG_PER_TOKEN, PKV_SEG_FP16 = 0, 1, 2
PKV_SEG_FLAG_FRESH = 1
PKV_DTYPE_F16, PKV_DTYPE_BF16, PKV_DTYPE_F32 = 0, 1, 2
PKV_E_BITS, PKV_E_SHAPE, PKV_E_NULL, PKV_E_LAYOUT = -1, -2, -3, -4
PKV_E_WORKSPACE, PKV_E_CUDA, PKV_E_LIMIT = -5, -6, -7


class Segment(ctypes.Structure):
    """``pkv_segment_t``."""

    _fields_ = [
        ("k_packed", ctypes.c_void_p), ("k_scale", ctypes.c_void_p), ("k_mins", ctypes.c_void_p),
        ("v_packed", ctypes.c_void_p), ("v_scale", ctypes.c_void_p), ("v_mins", ctypes.c_void_p),
        ("seq_len", ctypes.c_int64), ("head_stride", ctypes.c_int64),
        ("kind", ctypes.c_int32), ("k_bits", ctypes.c_int32), ("v_bits", ctypes.c_int32),
        ("k_group", ctypes.c_int32), ("v_group", ctypes.c_int32), ("num_splits", ctypes.c_int32),
        ("k_row_pitch", ctypes.c_int64), ("k_meta_pitch", ctypes.c_int64),
        ("flags", ctypes.c_int32), ("slot_tokens", ctypes.c_int16), ("slot_valid", ctypes.c_int16),
        ("seq_len_dev", ctypes.c_void_p),
    ]


class ColdLayer(ctypes.Structure):
    """``pkv_cold_layer_t``: one layer's hot buffers and the base pointers of its cooling outputs."""

    _fields_ = [(name, ctypes.c_void_p) for name in ("hot_k", "hot_v", "k_packed", "k_scale", "k_mins",
                                                       "v_packed", "v_scale", "v_mins", "indices")]


class NativeError(RuntimeError):
    def __init__(self, code: int, what: str, cuda_error: int = 0):
        self.code = code
        self.cuda_error = cuda_error
        extra = f" (cudaError {cuda_error})" if cuda_error else ""
        super().__init__(f"phasekv_b200: {what}{extra} [code {code}]")


_lib: Optional[ctypes.CDLL] = None

_I64, _I32, _VP, _F32 = ctypes.c_int64, ctypes.c_int, ctypes.c_void_p, ctypes.c_float

_SIGNATURES = {
    "pkv_abi_version": ([], _I32),
    "pkv_last_cuda_error": ([], _I32),
    "pkv_strerror": ([_I32], ctypes.c_char_p),
    "pkv_device_sm_count": ([_I32, ctypes.POINTER(_I32)], _I32),
    "pkv_pack_low_bits": ([_VP, _I64, _I64, _I32, _VP, _VP], _I32),
    "pkv_unpack_low_bits": ([_VP, _I64, _I64, _I64, _I32, _VP, _VP], _I32),
    "pkv_quantize_pack": ([_VP, _I64, _I64, _I64, _I32, _I64, _VP, _VP, _VP, _VP], _I32),
    "pkv_quantize_pack_pitched": ([_VP, _I64, _I64, _I64, _I32, _I64, _VP, _VP, _VP, _I64, _I64, _VP], _I32),
    "pkv_unpack_dequantize": ([_VP, _VP, _VP, _I64, _I64, _I64, _I32, _I64, _VP, _VP], _I32),
    "pkv_decode_workspace_bytes": ([ctypes.POINTER(Segment), _I32, _I32, _I32, _I32, _I32,
                                    ctypes.POINTER(ctypes.c_size_t)], _I32),
    "pkv_decode_launches": ([ctypes.POINTER(Segment), _I32, _I32, _I32, _I32, _I32, ctypes.POINTER(_I32)], _I32),
    "pkv_decode_attention": ([_VP, ctypes.POINTER(Segment), _I32, _I32, _I32, _I32, _F32, _I32, _VP,
                              ctypes.c_size_t, _VP, _VP, _VP, _VP, _VP], _I32),
    "pkv_decode_attention_static": ([_VP, ctypes.POINTER(Segment), _I32, _I32, _I32, _I32, _F32, _I32,
                                     _VP, _VP, _VP, _VP, _VP], _I32),
    "pkv_decode_batch_plan": ([ctypes.POINTER(Segment), ctypes.POINTER(ctypes.c_int32), _I32, _I32, _I32, _I32, _I32,
                               _VP, ctypes.c_size_t, ctypes.POINTER(ctypes.c_size_t),
                               ctypes.POINTER(ctypes.c_size_t)], _I32),
    "pkv_decode_attention_batched": ([_VP, _VP, _VP, _F32, _VP, ctypes.c_size_t, _VP, _VP], _I32),
    "pkv_decode_chunk_plan": ([ctypes.POINTER(Segment), _I32, _I32, _I32, _I32, _I32, _I32, _VP, ctypes.c_size_t,
                               ctypes.POINTER(ctypes.c_size_t), ctypes.POINTER(ctypes.c_size_t)], _I32),
    "pkv_rope_append": ([_VP, _VP, _VP, _I32, _I64, _I64, _I64, _VP, _VP, _I32, _I64, _I32, _I32, _I32, _I32,
                         _VP, _VP, _VP, _I64, _I64, _VP, _VP], _I32),
    "pkv_merge_partials": ([_VP, _VP, _VP, _I32, _I32, _I32, _VP, _VP, _VP, _VP, _VP], _I32),
    "pkv_merge_partials_strided": ([_VP, _VP, _VP, _I32, _I64, _I64, _I32, _I32, _VP, _VP, _VP, _VP, _VP], _I32),
    "pkv_exchange_create": ([_I32, _I32, _I32, _I32, ctypes.POINTER(_VP), _VP], _I32),
    "pkv_exchange_connect": ([_VP, _VP], _I32),
    "pkv_exchange_connect_loopback": ([_VP], _I32),
    "pkv_exchange_set_spin_limit": ([_VP, ctypes.c_uint], _I32),
    "pkv_exchange_set_wait_us": ([_VP, ctypes.c_uint], _I32),
    "pkv_exchange_status": ([_VP, ctypes.POINTER(_I32)], _I32),
    "pkv_exchange_destroy": ([_VP], _I32),
    "pkv_decode_attention_sharded": ([_VP, ctypes.POINTER(Segment), _I32, _I32, _I32, _I32, _F32, _I32, _VP,
                                      ctypes.c_size_t, _VP, _VP, _VP], _I32),
    "pkv_fake_quant": ([_VP, _VP, _I32, _I64, _I64, _I64, _I64, _I32, _I64, _VP], _I32),
    "pkv_value_norm": ([_VP, _I32, _I64, _I64, _I64, _I32, _VP, _VP], _I32),
    "pkv_topk_rows": ([_VP, _I64, _I64, _I64, _VP, _VP], _I32),
    "pkv_gather_tokens": ([_VP, _VP, _VP, _I64, _I64, _I64, _I64, _VP], _I32),
    "pkv_cold_select_pack": ([_VP, _VP, _I64, _I64, _I32, _I64, _I64, _I64, _I32, _I64,
                              _VP, _VP, _VP, _VP, _VP, _VP, _VP, _VP], _I32),
    "pkv_cold_select_pack_layers": ([_VP, _I32, _I64, _I64, _I32, _I64, _I64, _I64, _I32, _I64, _I64, _I64, _I64,
                                     _I64, _I64, _I64, _VP], _I32),
}

#: every symbol include/phasekv_b200.h declares
EXPORTED_SYMBOLS = tuple(_SIGNATURES)


def lib() -> ctypes.CDLL:
    """Load the CUDA library, failing loudly when it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m phasekv_b200.build`. "
                "phasekv_b200 has no CPU or PyTorch fallback.")
        L = ctypes.CDLL(LIB_PATH)
        for name, (argtypes, restype) in _SIGNATURES.items():
            fn = getattr(L, name)  # AttributeError if the library lacks a declared symbol
            fn.argtypes = argtypes
            fn.restype = restype
        _lib = L
    return _lib


def check(code: int) -> None:
    if code == 0:
        return
    L = lib()
    what = L.pkv_strerror(code).decode()
    raise NativeError(code, what, L.pkv_last_cuda_error() if code == PKV_E_CUDA else 0)


def ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def stream_of(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def require_cuda(t: torch.Tensor, what: str) -> None:
    if not t.is_cuda:
        raise RuntimeError(f"{what} must be a CUDA tensor: phasekv_b200 has no CPU path")


_SM_COUNT: dict = {}


def sm_count(device: torch.device) -> int:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _SM_COUNT:
        out = ctypes.c_int(0)
        check(lib().pkv_device_sm_count(idx, ctypes.byref(out)))
        _SM_COUNT[idx] = int(out.value)
    return _SM_COUNT[idx]
