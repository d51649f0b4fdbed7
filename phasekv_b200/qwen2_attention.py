"""Attention adapter that lets a Hugging Face Qwen2 (or Llama-style) model decode over a ``PhaseKVCache``.

Same contract as the reference's ``src/phasekv/qwen2_attention.py:19-122`` (and its Llama example,
``examples/llama_phasekv_adapter.py``): call ``install_qwen2_phasekv_attention(model)`` once after loading; the
first prefill still runs through the original attention module; with a ``PhaseKVCache`` as the model's cache a
forward pass is either one generated token or one chunk of new prompt tokens announced with
``begin_prompt_chunk``.  The layer only writes KV and attends; ``finish_decode_step`` / ``finish_prompt_chunk``
belong to the caller, after the whole model has returned (``decode_token`` / ``append_prompt_chunk`` below do
both).  Batch 1, CUDA, no padding.

What differs from the reference is how much is launched.  There, rotary embedding, three dtype conversions and
the append are separate torch operations, and a chunk of N tokens is N rounds of "append one token, attend with
one query" (``qwen2_attention.py:99-106``).  Here one kernel rotates q and k, converts and appends the whole
chunk (``PhaseKVCache.append_rotated``), and one split-K launch plus one merge launch attend for all N queries
with the causal rule applied by length (``fused_phasekv_chunk_decode``).

The module works with the attention classes of transformers 4.46 (``num_heads`` attributes, a 3-tuple result,
``past_key_value``) and 5.x (``config`` attributes, a 2-tuple result, ``past_key_values``).
"""
from __future__ import annotations

import inspect
from typing import List

import torch
from torch import nn

from .kernels.attention_cuda import fused_phasekv_chunk_decode, fused_phasekv_decode
from .phasekv_cache import PhaseKVCache


def _geometry(attention: nn.Module):
    """(query heads, KV heads, head_dim) of an attention module of either transformers generation."""
    config = getattr(attention, "config", None)
    heads = getattr(attention, "num_heads", None) or config.num_attention_heads
    kv_heads = getattr(attention, "num_key_value_heads", None) or config.num_key_value_heads
    head_dim = getattr(attention, "head_dim", None) or config.hidden_size // heads
    return int(heads), int(kv_heads), int(head_dim)


class PhaseKVQwen2Attention(nn.Module):
    """Wraps the original attention module and reuses its projection weights."""

    def __init__(self, original: nn.Module):
        super().__init__()
        self.original = original
        self.layer_idx = getattr(original, "layer_idx", None)
        parameters = inspect.signature(original.forward).parameters
        self._legacy_result = "past_key_value" in parameters   # 4.x returns (output, weights, cache)
        self.train(original.training)

    def forward(self, hidden_states, attention_mask=None, position_ids=None, past_key_value=None,
                output_attentions=False, use_cache=False, cache_position=None, position_embeddings=None,
                past_key_values=None, **kwargs):
        cache = past_key_values if past_key_values is not None else past_key_value
        if not isinstance(cache, PhaseKVCache):
            passed = dict(hidden_states=hidden_states, attention_mask=attention_mask, position_ids=position_ids,
                          output_attentions=output_attentions, use_cache=use_cache, cache_position=cache_position,
                          position_embeddings=position_embeddings, **kwargs)
            passed["past_key_value" if self._legacy_result else "past_key_values"] = cache
            accepted = inspect.signature(self.original.forward).parameters
            if not any(p.kind is inspect.Parameter.VAR_KEYWORD for p in accepted.values()):
                passed = {k: v for k, v in passed.items() if k in accepted}
            return self.original(**passed)

        batch, q_len, _ = hidden_states.shape
        if batch != 1 or hidden_states.dtype not in (torch.float16, torch.bfloat16):
            raise ValueError("PhaseKV attention serves batch=1 in float16/bfloat16 (目前只支持 batch=1、float16/bfloat16)")
        if hidden_states.device.type != "cuda":
            raise ValueError("PhaseKV decode 需要 CUDA (needs CUDA)")
        if self.training or output_attentions or not use_cache:
            raise ValueError("PhaseKV decode 需要 eval()、use_cache=True、output_attentions=False")
        if self.layer_idx is None:
            raise ValueError("the attention module has no layer_idx (缺少 layer_idx)")
        # decide the phase before anything is projected or written; new input goes through the chunk interface
        # even when it is a single token
        if cache.prompt_chunk_len:
            if q_len != cache.prompt_chunk_len:
                raise ValueError(f"新增 prompt 需要 {cache.prompt_chunk_len} 个 token，实际为 {q_len} "
                                 "(the announced prompt chunk and the input differ in length)")
        elif q_len != 1:
            raise ValueError(f"普通 PhaseKV decode 需要 q_len=1，实际为 {q_len}; announce new input with "
                             "begin_prompt_chunk(length) first")

        base = self.original
        heads, kv_heads, head_dim = _geometry(base)
        query = base.q_proj(hidden_states)[0].view(q_len, heads, head_dim)
        key = base.k_proj(hidden_states)[0].view(q_len, kv_heads, head_dim)
        value = base.v_proj(hidden_states)[0].view(q_len, kv_heads, head_dim)
        if position_embeddings is None:
            if position_ids is None or not hasattr(base, "rotary_emb"):
                raise ValueError("必须提供真实绝对 position_ids 以计算 RoPE (true absolute positions are needed)")
            cos, sin = base.rotary_emb(value, position_ids)
        else:
            cos, sin = position_embeddings
        query = cache.append_rotated(self.layer_idx, query, key, value, cos[0], sin[0])
        tiers = cache.layer_tiers(self.layer_idx)
        if cache.prompt_chunk_len:
            context = fused_phasekv_chunk_decode(query, tiers, heads)
        else:
            context = fused_phasekv_decode(query[0], tiers, heads)
        output = base.o_proj(context.reshape(1, q_len, heads * head_dim).to(hidden_states.dtype))
        return (output, None, cache) if self._legacy_result else (output, None)


def _install(model, model_type: str) -> None:
    if getattr(model.config, "model_type", None) != model_type:
        raise TypeError(f"当前适配器仅支持 model_type='{model_type}' 的模型 (this adapter serves {model_type} models)")
    for layer in model.model.layers:
        original = layer.self_attn
        if isinstance(original, PhaseKVQwen2Attention):
            continue
        if not all(hasattr(original, name) for name in ("q_proj", "k_proj", "v_proj", "o_proj")):
            raise TypeError(f"不支持的 attention 类型 (unsupported attention module): {type(original).__name__}")
        layer.self_attn = PhaseKVQwen2Attention(original)


def install_qwen2_phasekv_attention(model) -> None:
    """Wrap the attention of every layer of a ``Qwen2ForCausalLM`` in place; installed files are not touched."""
    _install(model, "qwen2")


def install_llama_phasekv_attention(model) -> None:
    """The same for a Llama model (rotary embedding, grouped-query projections without bias)."""
    if getattr(model.config, "pretraining_tp", 1) != 1:
        raise ValueError("pretraining_tp > 1 splits the projections; not supported")
    _install(model, "llama")


# --------------------------------------------------------------------------- driving a model over the cache
def _positions(model, start: int, length: int) -> torch.Tensor:
    return torch.arange(start, start + length, device=next(model.parameters()).device).unsqueeze(0)


@torch.inference_mode()
def decode_token(model, cache: PhaseKVCache, token: torch.Tensor) -> torch.Tensor:
    """Forward one generated token and commit the step once every layer has returned; the next token's logits."""
    output = model(input_ids=token.reshape(1, 1), past_key_values=cache, use_cache=True,
                   position_ids=_positions(model, cache.true_seq_length, 1))
    cache.finish_decode_step()
    return output.logits[:, -1, :]


@torch.inference_mode()
def append_prompt_chunk(model, cache: PhaseKVCache, token_ids: List[int]) -> torch.Tensor:
    """Forward only the new input tokens; the old prompt and the generated KV stay where they are."""
    if not token_ids:
        raise ValueError("新增 prompt 不能为空 (the new prompt chunk is empty)")
    device = next(model.parameters()).device
    start = cache.true_seq_length
    cache.begin_prompt_chunk(len(token_ids))
    output = model(input_ids=torch.tensor([token_ids], device=device), past_key_values=cache, use_cache=True,
                   position_ids=_positions(model, start, len(token_ids)))
    cache.finish_prompt_chunk()
    return output.logits[:, -1, :].clone()
