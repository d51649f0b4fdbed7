"""The attention adapter is transparent to ordinary forward passes (no PhaseKVCache involved): the scenario of the
reference's tests/test_qwen2_attention_adapter.py:73-91, which needs neither weights nor a GPU."""
import pytest
import torch

transformers = pytest.importorskip("transformers")


def tiny_qwen2(**over):
    from transformers import Qwen2Config, Qwen2ForCausalLM
    args = dict(vocab_size=97, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4,
                num_key_value_heads=2, max_position_embeddings=128, attention_dropout=0.0, attn_implementation="eager")
    args.update(over)
    torch.manual_seed(7)
    return Qwen2ForCausalLM(Qwen2Config(**args))


def test_install_preserves_uncompressed_prefill_and_is_idempotent():
    from phasekv_b200.qwen2_attention import PhaseKVQwen2Attention, install_qwen2_phasekv_attention
    model = tiny_qwen2().eval()
    input_ids = torch.tensor([[1, 2, 3]])
    with torch.no_grad():
        original = model(input_ids=input_ids, use_cache=False).logits
        install_qwen2_phasekv_attention(model)
        wrapped = model(input_ids=input_ids, use_cache=False).logits
        cached = model(input_ids=input_ids, use_cache=True)      # a dense cache still goes to the original module
    assert isinstance(model.model.layers[0].self_attn, PhaseKVQwen2Attention)
    assert not model.model.layers[0].self_attn.training
    assert torch.equal(original, wrapped) and torch.equal(original, cached.logits)
    assert cached.past_key_values.get_seq_length() == 3
    first = model.model.layers[0].self_attn
    install_qwen2_phasekv_attention(model)
    assert model.model.layers[0].self_attn is first


def test_install_refuses_other_model_types():
    from phasekv_b200.qwen2_attention import install_llama_phasekv_attention, install_qwen2_phasekv_attention
    model = tiny_qwen2()
    with pytest.raises(TypeError):
        install_llama_phasekv_attention(model)
    model.config.model_type = "other"
    with pytest.raises(TypeError):
        install_qwen2_phasekv_attention(model)
