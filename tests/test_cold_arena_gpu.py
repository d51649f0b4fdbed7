"""The cold tier as arenas: every cooling step is bit-identical to the per-step packing, and decode attention that
reads a run of steps as ONE masked segment agrees with decode over the steps one by one and with the oracle."""
import types

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def make_prefill(layers, length, heads=4, hd=128, seed=5):
    gen = torch.Generator().manual_seed(seed)
    c = types.SimpleNamespace(key_cache=[], value_cache=[])
    for _ in range(layers):
        c.key_cache.append(torch.randn(1, heads, length, hd, generator=gen, dtype=torch.float16).to(DEV))
        c.value_cache.append(torch.randn(1, heads, length, hd, generator=gen, dtype=torch.float16).to(DEV))
    return c


def detached(tiers):
    """The same tiers with every cold step in tensors of its own: the decode entry point describes them one by one."""
    from dataclasses import replace
    from phasekv_b200.kernels.tiers import LayerTiers, PackedKVSegment

    def own(pt):
        return replace(pt, packed=pt.packed.clone(), scale=pt.scale.clone(), mins=pt.mins.clone())
    return LayerTiers(prompt=tiers.prompt, prompt_extensions=list(tiers.prompt_extensions),
                      cold=[PackedKVSegment(own(s.key), own(s.value)) for s in tiers.cold],
                      hot_k=tiers.hot_k, hot_v=tiers.hot_v, hot_len=tiers.hot_len)


def descriptor_count(tiers):
    from phasekv_b200.kernels.attention_cuda import layer_segments
    return len(layer_segments(tiers)[0])


@pytest.mark.parametrize("window,lazy_g,ratio,cold_bits,steps", [
    (32, 16, 0.5, 4, 180),    # the reference's defaults: 8 of 16 kept, slots of 32 tokens with 8 valid
    (32, 16, 1.0, 2, 120),    # 16 kept
    (8, 48, 1.0, 4, 200),     # 48 kept: slots of 64 tokens, two key groups per step, the second one ragged
    (16, 40, 0.8, 8, 170),    # 32 kept: a slot with no padding at all
])
def test_arena_steps_equal_per_step_packing_and_decode_agrees(oracle, window, lazy_g, ratio, cold_bits, steps):
    from phasekv_b200 import workloads
    from phasekv_b200.cold_tier import select_and_pack_cold
    from phasekv_b200.kernels.attention_cuda import fused_phasekv_decode
    from phasekv_b200.phasekv_cache import PhaseKVCache
    from tests.conftest import attention_close
    from tests.util import assert_packed_equal, to_cpu_packed
    shape = workloads.QWEN2_5_7B
    cache = PhaseKVCache.from_dense_prefill(make_prefill(2, 320), prompt_len=320, recent_window=window, lazy_g=lazy_g,
                                            decode_keep_ratio=ratio, cold_bits=cold_bits)
    gen = torch.Generator().manual_seed(11)
    expected = []     # per-step segments from the single-layer entry point, on copies of layer 1's hot buffers
    checked = 0
    for step in range(steps):
        for l in range(2):
            k = torch.randn(1, 4, 1, 128, generator=gen, dtype=torch.float16).to(DEV)
            v = torch.randn(1, 4, 1, 128, generator=gen, dtype=torch.float16).to(DEV)
            cache.append_hot(l, k, v)
        layer = cache.layer_tiers(1)
        aged = layer.hot_len - window
        if aged >= lazy_g:
            keep = max(1, round(ratio * aged))
            hk, hv = layer.hot_k.clone(), layer.hot_v.clone()
            expected.append((select_and_pack_cold(hk, hv, layer.hot_len, aged, keep, cold_bits, 32), hk, hv, layer.hot_len - aged))
        cache.finish_decode_step()
        layer = cache.layer_tiers(1)
        assert len(layer.cold) == len(expected)
        if expected and len(layer.cold) != checked:
            seg, hk, hv, left = expected[-1]
            assert_packed_equal(layer.cold[-1].key, seg.key, f"step {step} key")
            assert_packed_equal(layer.cold[-1].value, seg.value, f"step {step} value")
            assert layer.hot_len == left
            assert torch.equal(layer.hot_k[:, :, :left], hk[:, :, :left]) and torch.equal(layer.hot_v[:, :, :left], hv[:, :, :left])
            checked = len(layer.cold)
        if step % 7 == 0 or step == steps - 1:
            q = torch.randn(shape.num_q_heads, 128, generator=gen).half()
            out = fused_phasekv_decode(q.to(DEV), layer, shape.num_q_heads)
            apart = fused_phasekv_decode(q.to(DEV), detached(layer), shape.num_q_heads)
            assert (out.float() - apart.float()).abs().max().item() <= 5e-4
            if step % 28 == 0 or step == steps - 1:
                segs = [(to_cpu_packed(s.key), to_cpu_packed(s.value)) for s in [layer.prompt, *layer.cold]]
                hk, hv = layer.hot_views()
                attention_close(out, oracle.segments_decode_reference(q, segs, hk.cpu(), hv.cpu(), shape.num_q_heads))
    layer = cache.layer_tiers(1)
    assert len(layer.cold) >= 3
    # all steps of the run are read as one segment: prompt + one arena + hot
    assert descriptor_count(layer) == 3 and descriptor_count(detached(layer)) == 2 + len(layer.cold)
    # earlier steps were never rewritten
    for got, (seg, *_rest) in zip(layer.cold, expected):
        assert_packed_equal(got.key, seg.key) and assert_packed_equal(got.value, seg.value)


def test_arena_grows_and_survives_a_prompt_chunk(oracle, monkeypatch):
    """A small arena (4 steps) that has to double twice; growing and a prompt chunk between decode steps change
    nothing about the steps recorded so far, and cooling continues in the same arena afterwards."""
    from phasekv_b200 import cold_arena, workloads
    from phasekv_b200.kernels.attention_cuda import fused_phasekv_decode
    from phasekv_b200.phasekv_cache import PhaseKVCache
    from tests.conftest import attention_close
    from tests.util import to_cpu_packed
    real_init = cold_arena.ColdArena.__init__
    monkeypatch.setattr(cold_arena.ColdArena, "__init__",
                        lambda self, like, bits, group, keep, max_events=4: real_init(self, like, bits, group, keep, max_events))
    shape = workloads.QWEN2_5_7B
    cache = PhaseKVCache.from_dense_prefill(make_prefill(1, 200, seed=2), prompt_len=200, recent_window=8, lazy_g=4,
                                            decode_keep_ratio=0.75)
    gen = torch.Generator().manual_seed(13)

    def tok():
        return torch.randn(1, 4, 1, 128, generator=gen, dtype=torch.float16).to(DEV)
    snapshots = []
    for step in range(60):
        cache.append_hot(0, tok(), tok())
        cache.finish_decode_step()
        layer = cache.layer_tiers(0)
        while len(snapshots) < len(layer.cold):
            s = layer.cold[len(snapshots)]
            snapshots.append((to_cpu_packed(s.key), to_cpu_packed(s.value)))
        q = torch.randn(shape.num_q_heads, 128, generator=gen).half()
        out = fused_phasekv_decode(q.to(DEV), layer, shape.num_q_heads)
        hk, hv = layer.hot_views()
        ref = oracle.segments_decode_reference(q, [(to_cpu_packed(layer.prompt.key), to_cpu_packed(layer.prompt.value)),
                                                   *snapshots], hk.cpu(), hv.cpu(), shape.num_q_heads)
        attention_close(out, ref)
    layer = cache.layer_tiers(0)
    assert len(layer.cold) == 13 and layer._cold_runs[0].max_events == 16 and descriptor_count(layer) == 3
    for (k, v), s in zip(snapshots, layer.cold):      # growing moved the steps without changing a bit
        assert torch.equal(k.packed, s.key.packed.cpu()) and torch.equal(v.packed, s.value.packed.cpu())
        assert torch.equal(k.scale, s.key.scale.cpu()) and torch.equal(v.mins, s.value.mins.cpu())
    cache.begin_prompt_chunk(5)
    for _ in range(5):
        cache.append_prompt_token(0, tok(), tok())
    cache.finish_prompt_chunk()
    for _ in range(20):
        cache.append_hot(0, tok(), tok())
        cache.finish_decode_step()
    layer = cache.layer_tiers(0)
    assert len(layer._cold_runs) == 1 and len(layer.cold) == 18 and descriptor_count(layer) == 4
    q = torch.randn(shape.num_q_heads, 128, generator=gen).half()
    out = fused_phasekv_decode(q.to(DEV), layer, shape.num_q_heads)
    segs = [(to_cpu_packed(s.key), to_cpu_packed(s.value)) for s in [layer.prompt, *layer.prompt_extensions, *layer.cold]]
    hk, hv = layer.hot_views()
    attention_close(out, oracle.segments_decode_reference(q, segs, hk.cpu(), hv.cpu(), shape.num_q_heads))


def test_batched_and_sharded_entry_points_read_arenas(oracle):
    from phasekv_b200 import workloads
    from phasekv_b200.kernels.attention_cuda import BatchDecodePlan, fused_phasekv_decode
    from phasekv_b200.phasekv_cache import PhaseKVCache
    from tests.conftest import attention_close
    shape = workloads.QWEN2_5_7B
    gen = torch.Generator().manual_seed(17)
    tiers = []
    for i, (length, steps) in enumerate([(500, 100), (4096, 40), (64, 333)]):
        cache = PhaseKVCache.from_dense_prefill(make_prefill(1, length, seed=20 + i), prompt_len=length)
        for _ in range(steps):
            k = torch.randn(1, 4, 1, 128, generator=gen, dtype=torch.float16).to(DEV)
            cache.append_hot(0, k, k.flip(-1).contiguous())
            cache.finish_decode_step()
        tiers.append(cache.layer_tiers(0))
    q = torch.randn(3, shape.num_q_heads, 128, generator=gen).half().to(DEV)
    out = BatchDecodePlan(tiers, shape.num_q_heads).run(q)
    for i, t in enumerate(tiers):
        single = fused_phasekv_decode(q[i], t, shape.num_q_heads)
        apart = fused_phasekv_decode(q[i], detached(t), shape.num_q_heads)
        assert (out[i].float() - single.float()).abs().max().item() <= 1e-3
        assert (single.float() - apart.float()).abs().max().item() <= 5e-4


def test_layouts_the_tensor_core_kernel_cannot_take_fall_back_to_one_descriptor_per_step(oracle):
    """head_dim 64 and group 16: still arenas (one cooling launch for all layers), described step by step."""
    from phasekv_b200.kernels.attention_cuda import fused_phasekv_decode
    from phasekv_b200.phasekv_cache import PhaseKVCache
    from tests.conftest import attention_close
    from tests.util import to_cpu_packed
    gen = torch.Generator().manual_seed(19)
    for hd, group in ((64, 32), (128, 16)):
        cache = PhaseKVCache.from_dense_prefill(make_prefill(2, 96, heads=2, hd=hd), prompt_len=96, group_size=group,
                                                recent_window=4, lazy_g=4, decode_keep_ratio=0.5)
        for _ in range(30):
            for l in range(2):
                k = torch.randn(1, 2, 1, hd, generator=gen, dtype=torch.float16).to(DEV)
                cache.append_hot(l, k, k * 0.5)
            cache.finish_decode_step()
        layer = cache.layer_tiers(1)
        assert len(layer._cold_runs) == 1 and descriptor_count(layer) == 2 + len(layer.cold)
        q = torch.randn(8, hd, generator=gen).half()
        out = fused_phasekv_decode(q.to(DEV), layer, 8)
        segs = [(to_cpu_packed(s.key), to_cpu_packed(s.value)) for s in [layer.prompt, *layer.cold]]
        hk, hv = layer.hot_views()
        attention_close(out, oracle.segments_decode_reference(q, segs, hk.cpu(), hv.cpu(), 8))
