"""Triton-free stand-in for the reference's ``src/phasekv/kernels/attention_triton.py``.

Callers of the reference import their decode entry points from this module path
(qwen2_attention.py:96, examples/llama_phasekv_adapter.py:13, scripts/bench_*.py); this module
re-exports the CUDA implementations under the same names.  Nothing here imports triton.
"""
from .attention_cuda import (  # noqa: F401
    _device_sm_count,
    _fp16_layer_partial,
    _kivi_layer_partial,
    _merge_partials,
    _reduce_splits,
    decode_attention_packed,
    decode_attention_packed_splitk,
    fused_phasekv_chunk_decode,
    fused_phasekv_decode,
    fused_three_tier_decode,
    fused_three_tier_decode_single,
)
from .launch_config import plan_kivi_decode  # noqa: F401
from .packing import PackedTensor, _vals_per_byte  # noqa: F401
