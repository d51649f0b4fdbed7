"""PhaseKVCache lifecycle on the GPU: the scenarios of the reference's tests/test_phasekv_cache.py (which run on
a CPU there) against this package's CUDA-backed cache, plus decode attention over the cache's tiers."""
import types

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def make_prefill(layers=2, length=20, batch=1, dtype=torch.float16, heads=2, hd=8, seed=7):
    gen = torch.Generator().manual_seed(seed)
    c = types.SimpleNamespace(key_cache=[], value_cache=[])
    for _ in range(layers):
        c.key_cache.append(torch.randn(batch, heads, length, hd, generator=gen, dtype=dtype).to(DEV))
        c.value_cache.append(torch.randn(batch, heads, length, hd, generator=gen, dtype=dtype).to(DEV))
    return c


def step_all(cache, key, value=None):
    for layer_idx in range(len(cache)):
        cache.append_hot(layer_idx, key, key if value is None else value)
    cache.finish_decode_step()


@pytest.fixture(scope="module")
def PhaseKVCache():
    from phasekv_b200.phasekv_cache import PhaseKVCache
    return PhaseKVCache


def test_bf16_prefill_is_packed_for_fp16_decode(PhaseKVCache):
    from phasekv_b200.kernels.packing import unpack_dequantize
    cache = PhaseKVCache.from_dense_prefill(make_prefill(dtype=torch.bfloat16), prompt_len=20, prompt_bits=2, group_size=4)
    layer = cache.layer_tiers(0)
    assert layer.hot_k.dtype == layer.hot_v.dtype == torch.float16 and layer.prompt.key.packed.dtype == torch.uint8
    assert torch.isfinite(unpack_dequantize(layer.prompt.key)).all()


def test_prefill_selection_packs_key_and_value_on_different_axes(PhaseKVCache):
    from phasekv_b200.kernels.packing import unpack_dequantize
    from phasekv_b200.quant import quantize_key, quantize_value
    dense = make_prefill()
    indices = torch.tensor([[[0, 1, 4, 6, 9, 11, 15, 19], [0, 2, 3, 7, 9, 13, 17, 19]]])
    cache = PhaseKVCache.from_dense_prefill(dense, prompt_len=20, keep_indices=[indices, indices], prompt_bits=2,
                                            group_size=4, recent_window=2, lazy_g=2)
    assert cache.get_seq_length() == 8 and cache.true_seq_length == 20 and len(cache) == 2
    layer = cache.layer_tiers(0)
    assert layer.prompt.key.axis == 2 and layer.prompt.value.axis == 3
    sel = indices.sort(dim=-1).values.unsqueeze(-1).expand(1, 2, 8, 8).to(DEV)
    raw_k, raw_v = dense.key_cache[0].gather(2, sel), dense.value_cache[0].gather(2, sel)
    # packed (float16 scale/zero) and stage-A fake quantisation (float32 scale/zero) agree to 0.004
    assert torch.allclose(unpack_dequantize(layer.prompt.key), quantize_key(raw_k, 2, 4), atol=0.004)
    assert torch.allclose(unpack_dequantize(layer.prompt.value), quantize_value(raw_v, 2, 4), atol=0.004)
    assert dense.key_cache[0].shape[2] == 20
    try:
        from transformers.cache_utils import Cache
        assert isinstance(cache, Cache)
    except ImportError:
        pass


def test_decode_cools_batches_without_repacking_old_segments(PhaseKVCache):
    cache = PhaseKVCache.from_dense_prefill(make_prefill(), prompt_len=20, prompt_bits=2, cold_bits=4, group_size=4,
                                            recent_window=2, lazy_g=2, decode_keep_ratio=0.5)
    gen = torch.Generator().manual_seed(9)

    def tok():
        return torch.randn(1, 2, 1, 8, generator=gen, dtype=torch.float16).to(DEV)
    for _ in range(4):
        for l in range(len(cache)):
            cache.append_hot(l, tok(), tok())
        cache.finish_decode_step()
    first_cold = cache.layer_tiers(0).cold[0]
    assert first_cold.length == 1 and cache.layer_tiers(0).hot_len == 2
    for _ in range(2):
        for l in range(len(cache)):
            cache.append_hot(l, tok(), tok())
        cache.finish_decode_step()
    assert cache.layer_tiers(0).cold[0] is first_cold and len(cache.layer_tiers(0).cold) == 2
    assert cache.get_seq_length() == 24 and cache.true_seq_length == 26
    assert cache.physical_nbytes() > 0 and cache.get_max_cache_shape() is None


def test_standard_update_is_refused_and_a_step_needs_every_layer(PhaseKVCache):
    cache = PhaseKVCache.from_dense_prefill(make_prefill(), prompt_len=20)
    key = torch.ones(1, 2, 1, 8, dtype=torch.float16, device=DEV)
    with pytest.raises(RuntimeError, match="不返回稠密"):
        cache.update(key, key, 0)
    cache.append_hot(0, key, key)
    with pytest.raises(RuntimeError, match="每一层"):
        cache.finish_decode_step()


def test_new_prompt_is_packed_without_rebuilding_old_cache(PhaseKVCache):
    cache = PhaseKVCache.from_dense_prefill(make_prefill(), prompt_len=20, prompt_bits=4, recent_window=2, lazy_g=2)
    old_prompt = cache.layer_tiers(0).prompt
    key = torch.ones(1, 2, 1, 8, dtype=torch.float16, device=DEV)
    step_all(cache, key)
    cache.begin_prompt_chunk(3)
    for l in range(len(cache)):
        for _ in range(3):
            cache.append_prompt_token(l, key, key)
    cache.finish_prompt_chunk()
    layer = cache.layer_tiers(0)
    assert layer.prompt is old_prompt and cache.true_seq_length == 24 and cache.get_seq_length() == 24
    assert layer.hot_len == 1 and layer.cold == []
    assert torch.equal(layer.hot_views()[0], key) and torch.equal(layer.hot_views()[1], key)
    assert [s.length for s in layer.prompt_extensions] == [3] and layer.prompt_extensions[-1].key.bits == 4


def test_invalid_config_and_fractional_indices_fail_before_packing(PhaseKVCache):
    dense = make_prefill()
    for name, value in (("prompt_bits", 3), ("cold_bits", 4.0), ("group_size", 1.5), ("recent_window", True),
                        ("lazy_g", 0), ("decode_keep_ratio", float("nan"))):
        with pytest.raises(ValueError, match=name):
            PhaseKVCache.from_dense_prefill(dense, prompt_len=20, **{name: value})
    indices = torch.tensor([[[0.5, 3.0], [1.0, 4.0]]])
    with pytest.raises(ValueError, match="整数张量"):
        PhaseKVCache.from_dense_prefill(dense, prompt_len=20, keep_indices=[indices, indices])
    with pytest.raises(ValueError, match="第 0 层.*prompt_len=19.*20"):
        PhaseKVCache.from_dense_prefill(dense, prompt_len=19)
    with pytest.raises(TypeError):
        PhaseKVCache.from_dense_prefill(object(), prompt_len=20)


def test_invalid_layer_and_failed_writes_do_not_advance_state(PhaseKVCache):
    cache = PhaseKVCache.from_dense_prefill(make_prefill(), prompt_len=20, recent_window=2, lazy_g=2)
    key = torch.ones(1, 2, 1, 8, dtype=torch.float16, device=DEV)
    for layer_idx in (-1, 2, 0.0, True):
        with pytest.raises(IndexError, match="layer_idx"):
            cache.append_hot(layer_idx, key, key)
    with pytest.raises(ValueError, match="float16"):
        cache.append_hot(0, key.float(), key.float())
    assert cache.get_seq_length() == 20
    cache.append_hot(0, key, key)
    with pytest.raises(RuntimeError, match="第 0 层.*已追加"):
        cache.append_hot(0, key, key)
    with pytest.raises(RuntimeError, match=r"尚未追加的层为 \[1\]"):
        cache.finish_decode_step()
    with pytest.raises(RuntimeError, match="decode 步内"):
        cache.begin_prompt_chunk(2)
    cache.append_hot(1, key, key)
    cache.finish_decode_step()
    with pytest.raises(RuntimeError, match=r"\[0, 1\]"):
        cache.finish_decode_step()


def test_cooling_threshold_selection_and_hot_tail(PhaseKVCache):
    """Known answer: the aged batch holds tokens 0 and 1; head 0 keeps token 0 (value norm 9 > 1), head 1 token 1."""
    from phasekv_b200.kernels.packing import unpack_dequantize
    cache = PhaseKVCache.from_dense_prefill(make_prefill(layers=1), prompt_len=20, group_size=4, recent_window=2,
                                            lazy_g=2, decode_keep_ratio=0.5)
    prompt, tokens = cache.layer_tiers(0).prompt, []
    for step, strengths in enumerate(((9, 1), (1, 9), (3, 3), (4, 4))):
        value = torch.tensor(strengths, dtype=torch.float16, device=DEV).view(1, 2, 1, 1).expand(1, 2, 1, 8).contiguous()
        key = torch.full_like(value, step + 1)
        tokens.append((key, value))
        cache.append_hot(0, key, value)
        assert cache.layer_tiers(0).hot_len == step + 1 and cache.layer_tiers(0).cold_len == 0  # the query reads before cooling
        cache.finish_decode_step()
        if step < 3:
            assert cache.layer_tiers(0).cold_len == 0
    layer = cache.layer_tiers(0)
    cold_key = unpack_dequantize(layer.cold[0].key)
    assert torch.equal(cold_key[0, :, 0, 0].cpu(), torch.tensor([1., 2.], dtype=torch.float16))
    assert torch.equal(unpack_dequantize(layer.cold[0].value), torch.full_like(cold_key, 9))
    hot_k, hot_v = layer.hot_views()
    assert torch.equal(hot_k, torch.cat([t[0] for t in tokens[2:]], dim=2))
    assert torch.equal(hot_v, torch.cat([t[1] for t in tokens[2:]], dim=2))
    assert layer.prompt is prompt and cache.true_seq_length == 24 and cache.get_seq_length() == 23


def test_prompt_chunk_state_errors_and_decode_after_finish(PhaseKVCache):
    cache = PhaseKVCache.from_dense_prefill(make_prefill(), prompt_len=20, recent_window=2, lazy_g=2)
    key = torch.ones(1, 2, 1, 8, dtype=torch.float16, device=DEV)
    with pytest.raises(RuntimeError, match="begin_prompt_chunk"):
        cache.append_prompt_token(0, key, key)
    for length in (0, 1.5, True):
        with pytest.raises(ValueError, match="length"):
            cache.begin_prompt_chunk(length)
    cache.begin_prompt_chunk(5)  # more than the hot capacity: the buffers grow
    with pytest.raises(RuntimeError, match="prompt 块内"):
        cache.begin_prompt_chunk(1)
    with pytest.raises(RuntimeError, match="prompt 块内"):
        cache.reorder_cache(torch.tensor([0]))
    with pytest.raises(RuntimeError, match="finish_prompt_chunk"):
        cache.append_hot(0, key, key)
    with pytest.raises(RuntimeError, match="finish_prompt_chunk"):
        cache.finish_decode_step()
    with pytest.raises(ValueError, match="同一设备"):
        cache.append_prompt_token(0, key.to("meta"), key.to("meta"))
    with pytest.raises(ValueError, match="float16"):
        cache.append_prompt_token(0, key.float(), key.float())
    for _ in range(5):
        cache.append_prompt_token(0, key, key)
    with pytest.raises(RuntimeError, match="第 0 层已写满"):
        cache.append_prompt_token(0, key, key)
    with pytest.raises(RuntimeError, match="第 1 层.*期望 5 个，实际 0 个"):
        cache.finish_prompt_chunk()
    assert cache.true_seq_length == 20 and cache.layer_tiers(0).prompt_extensions == []
    for _ in range(5):
        cache.append_prompt_token(1, key, key)
    cache.finish_prompt_chunk()
    assert cache.true_seq_length == 25 and cache.layer_tiers(0).hot_k.shape[2] == 4
    step_all(cache, key)
    assert cache.true_seq_length == 26


def test_reorder_keeps_all_tiers_and_rejects_invalid_indices(PhaseKVCache):
    from phasekv_b200.kernels.packing import unpack_dequantize
    cache = PhaseKVCache.from_dense_prefill(make_prefill(batch=2), prompt_len=20, recent_window=2, lazy_g=2)
    key = torch.arange(32, dtype=torch.float16, device=DEV).reshape(2, 2, 1, 8)
    for _ in range(4):
        step_all(cache, key)
    cache.begin_prompt_chunk(1)
    for l in range(len(cache)):
        cache.append_prompt_token(l, key, key)
    cache.finish_prompt_chunk()
    step_all(cache, key)
    for bad in (torch.tensor([-1]), torch.tensor([2]), torch.tensor([0.])):
        with pytest.raises(ValueError, match="beam_idx"):
            cache.reorder_cache(bad.to(DEV))
    layer = cache.layer_tiers(0)
    originals = [unpack_dequantize(s.key) for s in [layer.prompt, *layer.prompt_extensions, *layer.cold]]
    original_hot = layer.hot_views()[0].clone()
    order = torch.tensor([1, 0, 1], device=DEV)
    cache.reorder_cache(order)
    for original, seg in zip(originals, [layer.prompt, *layer.prompt_extensions, *layer.cold]):
        assert torch.equal(unpack_dequantize(seg.key), original.index_select(0, order))
    assert torch.equal(layer.hot_views()[0], original_hot.index_select(0, order)) and cache.true_seq_length == 26


@pytest.mark.parametrize("keep_ratio", [0.5, 1.0])
def test_prompt_chunks_preserve_decode_window_and_cooling_schedule(PhaseKVCache, keep_ratio):
    """The same generated KV stream with and without interleaved prompt chunks must give identical hot and cold tiers."""
    options = dict(prompt_len=20, group_size=4, recent_window=2, lazy_g=2, decode_keep_ratio=keep_ratio)
    baseline = PhaseKVCache.from_dense_prefill(make_prefill(), **options)
    cache = PhaseKVCache.from_dense_prefill(make_prefill(), **options)
    gen = torch.Generator().manual_seed(23)

    def tok():
        return torch.randn(1, 2, 1, 8, generator=gen, dtype=torch.float16).to(DEV)
    added = 0
    for step in range(8):
        for l in range(len(cache)):
            key, value = tok(), tok()
            baseline.append_hot(l, key, value)
            cache.append_hot(l, key, value)
        baseline.finish_decode_step()
        cache.finish_decode_step()
        if step in (0, 2, 3, 6):
            length = 1 if step == 0 else 5
            frozen = [[layer.prompt, *layer.prompt_extensions, *layer.cold] for layer in cache.layers]
            cache.begin_prompt_chunk(length)
            for l in range(len(cache)):
                for _ in range(length):
                    cache.append_prompt_token(l, tok(), tok())
            cache.finish_prompt_chunk()
            added += length
            assert cache.prompt_chunk_len == 0
            for layer, old in zip(cache.layers, frozen):
                kept = [layer.prompt, *layer.prompt_extensions[:-1], *layer.cold]
                assert len(kept) == len(old) and all(a is b for a, b in zip(old, kept))
                assert layer.prompt_extensions[-1].length == length
        for actual, expected in zip(cache.layers, baseline.layers):
            assert actual.hot_len == expected.hot_len and actual.hot_k.shape[2] == 4
            for a, e in zip(actual.hot_views(), expected.hot_views()):
                assert a.dtype == torch.float16 and torch.equal(a, e)
            assert len(actual.cold) == len(expected.cold)
            for sa, se in zip(actual.cold, expected.cold):
                for name in ("key", "value"):
                    for field in ("packed", "scale", "mins"):
                        assert torch.equal(getattr(getattr(sa, name), field), getattr(getattr(se, name), field))
        assert cache.true_seq_length == 20 + step + 1 + added
        assert cache.get_seq_length() == baseline.get_seq_length() + added


def test_decode_attention_over_a_lived_in_cache(oracle):
    """Prefill 300 tokens of the 7B shape with per-head selection, decode 70 steps (cooling every 16 with half kept),
    add a prompt chunk, then attend: the kernel over cache.layer_tiers() must match the oracle over the same tiers
    read back to the CPU."""
    from phasekv_b200 import workloads
    from phasekv_b200.kernels.attention_triton import fused_phasekv_decode
    from phasekv_b200.phasekv_cache import PhaseKVCache
    from tests.util import to_cpu_packed
    shape = workloads.QWEN2_5_7B
    dense = make_prefill(layers=2, length=300, heads=4, hd=128, seed=31)
    keep = [torch.stack([torch.randperm(300, generator=torch.Generator().manual_seed(l * 10 + h))[:200] for h in range(4)]).unsqueeze(0)
            for l in range(2)]
    cache = PhaseKVCache.from_dense_prefill(dense, prompt_len=300, keep_indices=keep, recent_window=32, lazy_g=16,
                                            decode_keep_ratio=0.5)
    gen = torch.Generator().manual_seed(4)

    def tok():
        return torch.randn(1, 4, 1, 128, generator=gen, dtype=torch.float16).to(DEV)
    for _ in range(70):
        for l in range(2):
            cache.append_hot(l, tok(), tok())
        cache.finish_decode_step()
    cache.begin_prompt_chunk(37)
    for l in range(2):
        for _ in range(37):
            cache.append_prompt_token(l, tok(), tok())
    cache.finish_prompt_chunk()
    for l in range(2):
        cache.append_hot(l, tok(), tok())
    tiers = cache.layer_tiers(1)
    assert tiers.prompt.length == 200 and len(tiers.prompt_extensions) == 1 and len(tiers.cold) >= 2 and tiers.hot_len > 0
    q = torch.randn(shape.num_q_heads, 128, generator=gen).half()
    out = fused_phasekv_decode(q.to(DEV), tiers, shape.num_q_heads)
    segs = [(to_cpu_packed(s.key), to_cpu_packed(s.value)) for s in [tiers.prompt, *tiers.prompt_extensions, *tiers.cold]]
    hk, hv = tiers.hot_views()
    ref = oracle.segments_decode_reference(q, segs, hk.cpu(), hv.cpu(), shape.num_q_heads)
    from tests.conftest import attention_close
    attention_close(out, ref)


def test_decode_directly_behind_the_kernel_that_wrote_a_segment(oracle):
    """One layer, one stream, 200 decode steps that cool every fourth step: the decode call that follows
    finish_decode_step() is enqueued directly behind the cooling kernel that has just written a new cold segment
    (no other kernel in between).  Decode launches are programmatic dependents of the previous kernel and fetch
    settled packed segments before that kernel's writes are guaranteed visible, so the first launch over a new
    segment must carry the "fresh" flag and read it only after the dependency is resolved.  Every output is
    compared with the oracle over the same tiers read back to the CPU."""
    from phasekv_b200 import workloads
    from phasekv_b200.kernels.attention_triton import fused_phasekv_decode
    from phasekv_b200.phasekv_cache import PhaseKVCache
    from tests.conftest import attention_close
    from tests.util import to_cpu_packed
    shape = workloads.QWEN2_5_7B
    dense = make_prefill(layers=1, length=256, heads=4, hd=128, seed=3)
    cache = PhaseKVCache.from_dense_prefill(dense, prompt_len=256, recent_window=4, lazy_g=4, decode_keep_ratio=0.5)
    gen = torch.Generator().manual_seed(8)
    cold_cpu = []  # frozen segments are read back once
    tiers = cache.layer_tiers(0)
    prompt_cpu = (to_cpu_packed(tiers.prompt.key), to_cpu_packed(tiers.prompt.value))
    worst = 0.0
    for step in range(200):
        k = torch.randn(1, 4, 1, 128, generator=gen, dtype=torch.float16).to(DEV)
        v = torch.randn(1, 4, 1, 128, generator=gen, dtype=torch.float16).to(DEV)
        cache.append_hot(0, k, v)
        cache.finish_decode_step()          # every fourth step this ends with the cooling kernel ...
        tiers = cache.layer_tiers(0)
        q = torch.randn(shape.num_q_heads, 128, generator=gen).half()
        out = fused_phasekv_decode(q.to(DEV), tiers, shape.num_q_heads)  # ... and this is the next launch
        while len(cold_cpu) < len(tiers.cold):
            seg = tiers.cold[len(cold_cpu)]
            cold_cpu.append((to_cpu_packed(seg.key), to_cpu_packed(seg.value)))
        hk, hv = tiers.hot_views()
        ref = oracle.segments_decode_reference(q, [prompt_cpu, *cold_cpu], hk.cpu(), hv.cpu(), shape.num_q_heads)
        worst = max(worst, attention_close(out, ref))
    assert len(cold_cpu) >= 45 and worst <= 2e-3
