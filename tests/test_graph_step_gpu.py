"""A decode step captured once as a CUDA graph (device-resident lengths) against the same steps made eagerly."""
import types

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def make_prefill(layers, length, seed=5):
    gen = torch.Generator().manual_seed(seed)
    c = types.SimpleNamespace(key_cache=[], value_cache=[])
    for _ in range(layers):
        c.key_cache.append(torch.randn(1, 4, length, 128, generator=gen, dtype=torch.float16).to(DEV))
        c.value_cache.append(torch.randn(1, 4, length, 128, generator=gen, dtype=torch.float16).to(DEV))
    return c


def rope_tables(position, hd=128):
    inv = 1.0 / (10000.0 ** (torch.arange(0, hd, 2, dtype=torch.float32) / hd))
    emb = torch.cat([position * inv] * 2)
    return emb.cos().to(DEV), emb.sin().to(DEV)


def run_both(steps, layers, prompt_len, chunk_at=None, **options):
    from phasekv_b200.graph_step import GraphedDecodeStep
    from phasekv_b200.kernels.attention_cuda import fused_phasekv_decode
    from phasekv_b200.phasekv_cache import PhaseKVCache
    graphed = PhaseKVCache.from_dense_prefill(make_prefill(layers, prompt_len), prompt_len=prompt_len, **options)
    eager = PhaseKVCache.from_dense_prefill(make_prefill(layers, prompt_len), prompt_len=prompt_len, **options)
    runner = GraphedDecodeStep(graphed, 28, dtype=torch.bfloat16)
    gen = torch.Generator().manual_seed(21)
    worst = 0.0
    for step in range(steps):
        if chunk_at is not None and step == chunk_at:   # new input between decode steps: the hot buffers are replaced
            for cache in (graphed, eager):
                cache.begin_prompt_chunk(70)
                for l in range(layers):
                    for _ in range(70):
                        t = torch.randn(1, 4, 1, 128, generator=torch.Generator().manual_seed(l), dtype=torch.float16).to(DEV)
                        cache.append_prompt_token(l, t, t)
                cache.finish_prompt_chunk()
        q = torch.randn(layers, 28, 128, generator=gen).to(DEV, torch.bfloat16)
        k = torch.randn(layers, 4, 128, generator=gen).to(DEV, torch.bfloat16)
        v = torch.randn(layers, 4, 128, generator=gen).to(DEV, torch.bfloat16)
        cos, sin = rope_tables(float(graphed.true_seq_length))
        out = runner.step(q, k, v, cos, sin).clone()
        for l in range(layers):
            q_rot = eager.append_rotated(l, q[l:l + 1], k[l:l + 1], v[l:l + 1], cos[None], sin[None])
            want = fused_phasekv_decode(q_rot[0], eager.layer_tiers(l), 28)
            worst = max(worst, (out[l].float() - want.float()).abs().max().item())
        eager.finish_decode_step()
        assert graphed.true_seq_length == eager.true_seq_length
        assert graphed.layer_tiers(0).hot_len == eager.layer_tiers(0).hot_len
    for a, b in zip(graphed.layers, eager.layers):
        assert a.hot_len == b.hot_len and len(a.cold) == len(b.cold) and len(a.prompt_extensions) == len(b.prompt_extensions)
        assert torch.equal(a.hot_k[:, :, :a.hot_len], b.hot_k[:, :, :b.hot_len])
        assert torch.equal(a.hot_v[:, :, :a.hot_len], b.hot_v[:, :, :b.hot_len])
        for sa, sb in zip(a.cold, b.cold):
            assert torch.equal(sa.key.packed, sb.key.packed) and torch.equal(sa.value.packed, sb.value.packed)
            assert torch.equal(sa.key.scale, sb.key.scale) and torch.equal(sa.value.mins, sb.value.mins)
    return runner, worst, graphed


def test_one_capture_serves_growth_and_cooling():
    """130 tokens with the reference's defaults: the float16 tier fills and is cooled six times; the graph is captured
    once, and every output agrees with the eager path (split points differ: the captured launch is sized for the
    tiers' capacities)."""
    runner, worst, cache = run_both(130, 3, 700)
    assert runner.captures == 1 and len(cache.layer_tiers(0).cold) >= 6
    assert worst <= 5e-4


def test_recapture_when_a_buffer_is_replaced(monkeypatch):
    """A small arena that has to grow, and a prompt chunk between decode steps: both replace buffers the captured
    launches point at, and both are noticed."""
    from phasekv_b200 import cold_arena
    real_init = cold_arena.ColdArena.__init__
    monkeypatch.setattr(cold_arena.ColdArena, "__init__",
                        lambda self, like, bits, group, keep, max_events=2: real_init(self, like, bits, group, keep, max_events))
    runner, worst, cache = run_both(60, 2, 300, chunk_at=25, recent_window=8, lazy_g=4, decode_keep_ratio=0.5)
    assert runner.captures >= 4          # first capture, arena growth (2 -> 4 -> 8 -> 16 events), the prompt chunk
    assert len(cache.layer_tiers(0).cold) >= 10 and worst <= 5e-4


def test_layouts_without_an_arena_are_refused():
    from phasekv_b200.graph_step import GraphedDecodeStep
    from phasekv_b200.phasekv_cache import PhaseKVCache
    gen = torch.Generator().manual_seed(1)
    dense = types.SimpleNamespace(key_cache=[torch.randn(1, 2, 64, 64, generator=gen, dtype=torch.float16).to(DEV)],
                                  value_cache=[torch.randn(1, 2, 64, 64, generator=gen, dtype=torch.float16).to(DEV)])
    cache = PhaseKVCache.from_dense_prefill(dense, prompt_len=64)
    runner = GraphedDecodeStep(cache, 14)
    z = torch.zeros(1, 14, 64, device=DEV, dtype=torch.float16)
    with pytest.raises(ValueError, match="arena"):
        runner.step(z, z[:, :2], z[:, :2], torch.zeros(64, device=DEV), torch.zeros(64, device=DEV))
