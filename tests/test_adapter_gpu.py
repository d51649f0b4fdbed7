"""The model adapter on the GPU: the fused rotary-embedding + append kernel against the torch formulation, the
one-launch causal chunk attention against the reference's token-by-token order and the oracle, and the scenario of
the reference's tests/test_qwen2_attention_adapter.py:20-68 on a randomly initialised Qwen2."""
import types

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def rotate_half(x):
    return torch.cat((-x[..., x.shape[-1] // 2:], x[..., :x.shape[-1] // 2]), dim=-1)


def make_prefill(layers, length, heads, hd, seed=5):
    gen = torch.Generator().manual_seed(seed)
    c = types.SimpleNamespace(key_cache=[], value_cache=[])
    for _ in range(layers):
        c.key_cache.append(torch.randn(1, heads, length, hd, generator=gen, dtype=torch.float16).to(DEV))
        c.value_cache.append(torch.randn(1, heads, length, hd, generator=gen, dtype=torch.float16).to(DEV))
    return c


@pytest.mark.parametrize("dtype,rope_dtype", [(torch.float16, torch.float16), (torch.bfloat16, torch.bfloat16),
                                              (torch.bfloat16, torch.float32)])
@pytest.mark.parametrize("n,hq,hkv,hd", [(1, 28, 4, 128), (37, 28, 4, 128), (5, 14, 2, 64), (3, 4, 2, 8)])
def test_rope_append_equals_the_torch_formulation_bit_for_bit(dtype, rope_dtype, n, hq, hkv, hd):
    """apply_rotary_pos_emb as transformers writes it (q * cos + rotate_half(q) * sin in the model's dtype), then
    .to(float16) and the copy into the hot buffers: one launch, the same bits."""
    from phasekv_b200.phasekv_cache import PhaseKVCache
    gen = torch.Generator().manual_seed(n * 100 + hd)
    cache = PhaseKVCache.from_dense_prefill(make_prefill(1, 40, hkv, hd), prompt_len=40, group_size=min(32, hd),
                                            recent_window=64, lazy_g=8)
    layer = cache.layer_tiers(0)
    layer.hot_k.fill_(7.0), layer.hot_v.fill_(7.0)
    if n > 1:
        cache.begin_prompt_chunk(n)
        layer = cache.layer_tiers(0)
    start = layer.hot_len
    # the projections' outputs: one fused [n, (Hq + 2 Hkv) * hd] buffer, so the views have a token stride
    fused = torch.randn(n, (hq + 2 * hkv) * hd, generator=gen).to(DEV, dtype)
    q = fused[:, :hq * hd].view(n, hq, hd)
    k = fused[:, hq * hd:(hq + hkv) * hd].view(n, hkv, hd)
    v = fused[:, (hq + hkv) * hd:].view(n, hkv, hd)
    pos = torch.arange(1000, 1000 + n, dtype=torch.float32)
    inv = 1.0 / (10000.0 ** (torch.arange(0, hd, 2, dtype=torch.float32) / hd))
    emb = torch.cat([pos[:, None] * inv[None, :]] * 2, dim=-1)
    cos, sin = emb.cos().to(DEV, rope_dtype), emb.sin().to(DEV, rope_dtype)
    got_q = cache.append_rotated(0, q, k, v, cos, sin)
    c, s = cos.to(dtype)[:, None, :], sin.to(dtype)[:, None, :]
    want_q = ((q * c) + (rotate_half(q) * s)).to(torch.float16)
    want_k = ((k * c) + (rotate_half(k) * s)).to(torch.float16)
    assert got_q.dtype == torch.float16 and torch.equal(got_q, want_q)
    layer = cache.layer_tiers(0)
    assert layer.hot_len == start + n
    assert torch.equal(layer.hot_k[0, :, start:start + n], want_k.transpose(0, 1))
    assert torch.equal(layer.hot_v[0, :, start:start + n], v.to(torch.float16).transpose(0, 1))
    assert bool((layer.hot_k[0, :, start + n:] == 7).all()) and bool((layer.hot_k[0, :, :start] == 7).all())
    if n == 1:
        with pytest.raises(RuntimeError, match="已追加"):
            cache.append_rotated(0, q, k, v, cos, sin)
    else:
        with pytest.raises(RuntimeError, match="已写满"):
            cache.append_rotated(0, q[:1], k[:1], v[:1], cos[:1], sin[:1])
        cache.finish_prompt_chunk()
        assert cache.layer_tiers(0).prompt_extensions[-1].length == n


@pytest.mark.parametrize("prompt,steps,n", [(4096, 100, 37), (300, 0, 1), (1000, 40, 130), (64, 20, 8)])
def test_chunk_attention_equals_token_by_token_order_and_the_oracle(oracle, prompt, steps, n):
    """7B geometry: all queries of a chunk in one launch pair.  Each row must equal the single-query entry point run
    in the reference's order (append token i, attend with query i) and meet the parity bar against the oracle."""
    from phasekv_b200 import workloads
    from phasekv_b200.kernels.attention_cuda import fused_phasekv_chunk_decode, fused_phasekv_decode
    from phasekv_b200.phasekv_cache import PhaseKVCache
    from tests.conftest import attention_close
    from tests.util import to_cpu_packed
    shape = workloads.QWEN2_5_7B
    gen = torch.Generator().manual_seed(prompt + n)

    def tok(count=1):
        return torch.randn(1, 4, count, 128, generator=gen, dtype=torch.float16).to(DEV)
    caches = [PhaseKVCache.from_dense_prefill(make_prefill(1, prompt, 4, 128, seed=n), prompt_len=prompt) for _ in range(2)]
    for _ in range(steps):
        k, v = tok(), tok()
        for cache in caches:
            cache.append_hot(0, k, v)
            cache.finish_decode_step()
    block, serial = caches
    ks, vs = tok(n), tok(n)
    q = torch.randn(n, shape.num_q_heads, 128, generator=gen).half().to(DEV)
    block.begin_prompt_chunk(n), serial.begin_prompt_chunk(n)
    for i in range(n):
        block.append_prompt_token(0, ks[:, :, i:i + 1], vs[:, :, i:i + 1])
    out = fused_phasekv_chunk_decode(q, block.layer_tiers(0), shape.num_q_heads)
    assert out.shape == q.shape and out.dtype == torch.float16
    tiers = serial.layer_tiers(0)
    frozen = [(to_cpu_packed(s.key), to_cpu_packed(s.value)) for s in [tiers.prompt, *tiers.cold]]
    for i in range(n):
        serial.append_prompt_token(0, ks[:, :, i:i + 1], vs[:, :, i:i + 1])
        one = fused_phasekv_decode(q[i], tiers, shape.num_q_heads)
        assert (out[i].float() - one.float()).abs().max().item() <= 1e-3, i
        if i in (0, n // 2, n - 1):
            hk, hv = tiers.hot_views()
            attention_close(out[i], oracle.segments_decode_reference(q[i].cpu(), frozen, hk.cpu(), hv.cpu(), shape.num_q_heads))
    block.finish_prompt_chunk(), serial.finish_prompt_chunk()
    for a, b in zip(block.layer_tiers(0).prompt_extensions, serial.layer_tiers(0).prompt_extensions):
        assert torch.equal(a.key.packed, b.key.packed) and torch.equal(a.value.packed, b.value.packed)


def test_chunk_attention_on_other_layouts_is_the_token_loop():
    """head_dim 64: served query by query by the general kernel, bit-identical to the loop."""
    from phasekv_b200.kernels.attention_cuda import fused_phasekv_chunk_decode, fused_phasekv_decode
    from phasekv_b200.phasekv_cache import PhaseKVCache
    gen = torch.Generator().manual_seed(3)
    caches = [PhaseKVCache.from_dense_prefill(make_prefill(1, 200, 2, 64), prompt_len=200) for _ in range(2)]
    n = 6
    ks = torch.randn(1, 2, n, 64, generator=gen, dtype=torch.float16).to(DEV)
    q = torch.randn(n, 14, 64, generator=gen).half().to(DEV)
    for cache in caches:
        cache.begin_prompt_chunk(n)
    for i in range(n):
        caches[0].append_prompt_token(0, ks[:, :, i:i + 1], ks[:, :, i:i + 1])
    out = fused_phasekv_chunk_decode(q, caches[0].layer_tiers(0), 14)
    for i in range(n):
        caches[1].append_prompt_token(0, ks[:, :, i:i + 1], ks[:, :, i:i + 1])
        assert torch.equal(out[i], fused_phasekv_decode(q[i], caches[1].layer_tiers(0), 14))


def tiny_qwen2(hidden, heads, kv_heads):
    from transformers import Qwen2Config, Qwen2ForCausalLM
    torch.manual_seed(7)
    config = Qwen2Config(vocab_size=97, hidden_size=hidden, intermediate_size=2 * hidden, num_hidden_layers=2,
                         num_attention_heads=heads, num_key_value_heads=kv_heads, max_position_embeddings=128,
                         attention_dropout=0.0, attn_implementation="eager")
    return Qwen2ForCausalLM(config).to(device=DEV, dtype=torch.float16).eval()


@pytest.mark.parametrize("hidden,heads,kv_heads,group,prompt_len,kept", [(32, 4, 2, 4, 6, 3), (512, 4, 2, 32, 70, 64)])
@torch.inference_mode()
def test_prompt_block_matches_causal_token_forwards_and_preserves_hot(hidden, heads, kv_heads, group, prompt_len, kept):
    """head_dim 8 with a 6-token prompt is the reference's own test model (general kernel, query by query);
    head_dim 128 with 64 kept prompt tokens takes the tensor-core chunk path.  Per-head selection makes true and
    physical positions differ; a generated token is left in the hot tier before the chunk; then decode steps and
    single-token chunks alternate."""
    pytest.importorskip("transformers")
    from transformers.cache_utils import DynamicCache
    from phasekv_b200.kernels import attention_cuda
    from phasekv_b200.phasekv_cache import PhaseKVCache
    from phasekv_b200.qwen2_attention import append_prompt_chunk, decode_token, install_qwen2_phasekv_attention
    model = tiny_qwen2(hidden, heads, kv_heads)
    install_qwen2_phasekv_attention(model)
    gen = torch.Generator().manual_seed(1)
    prompt = torch.randint(1, 97, (1, prompt_len), generator=gen).to(DEV)
    try:
        prefill = model(input_ids=prompt, past_key_values=DynamicCache(config=model.config), use_cache=True)
    except TypeError:
        prefill = model(input_ids=prompt, past_key_values=DynamicCache(), use_cache=True)
    keep = torch.stack([torch.randperm(prompt_len, generator=gen)[:kept].sort().values for _ in range(kv_heads)]).unsqueeze(0).to(DEV)
    options = dict(prompt_len=prompt_len, keep_indices=[keep, keep], group_size=group, recent_window=8, lazy_g=2)
    block_cache = PhaseKVCache.from_dense_prefill(prefill.past_key_values, **options)
    serial_cache = PhaseKVCache.from_dense_prefill(prefill.past_key_values, **options)
    for cache in (block_cache, serial_cache):
        decode_token(model, cache, torch.tensor([7], device=DEV))
    old_hot = [(k.clone(), v.clone()) for k, v in (layer.hot_views() for layer in block_cache.layers)]
    new_ids = torch.tensor([[8, 9, 10]], device=DEV)
    block_cache.begin_prompt_chunk(3)
    block_output = model(input_ids=new_ids, past_key_values=block_cache, use_cache=True,
                         position_ids=torch.arange(prompt_len + 1, prompt_len + 4, device=DEV).unsqueeze(0))
    # a token-by-token forward cannot read later input: the control for causality inside the block
    serial_logits = [decode_token(model, serial_cache, token) for token in new_ids[0]]
    torch.testing.assert_close(block_output.logits, torch.stack(serial_logits, dim=1), atol=0.002, rtol=0.002)
    block_cache.finish_prompt_chunk()
    assert block_cache.true_seq_length == prompt_len + 4
    for layer, (key, value) in zip(block_cache.layers, old_hot):
        assert layer.hot_len == 1 and layer.cold_len == 0 and layer.prompt_extensions[-1].length == 3
        assert torch.equal(layer.hot_views()[0], key) and torch.equal(layer.hot_views()[1], value)
    logits = decode_token(model, block_cache, torch.tensor([11], device=DEV))
    assert torch.isfinite(logits).all()
    logits = append_prompt_chunk(model, block_cache, [12])
    assert torch.isfinite(logits).all()
    assert block_cache.true_seq_length == prompt_len + 6 and block_cache.layer_tiers(0).hot_len == 2
    with pytest.raises(ValueError, match="q_len=1"):
        model(input_ids=new_ids, past_key_values=block_cache, use_cache=True,
              position_ids=torch.arange(prompt_len + 6, prompt_len + 9, device=DEV).unsqueeze(0))
