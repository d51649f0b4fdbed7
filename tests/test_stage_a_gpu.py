"""Stage-A operators on the GPU against the reference's vectors and the CPU oracle."""
import types

import numpy as np
import pytest
import torch

from tests.conftest import GOLDEN as GOLDEN_DIR
from tests.test_stage_a_cpu import _cases

pytestmark = pytest.mark.gpu


def test_fake_quant_matches_the_reference_bit_for_bit():
    from phasekv_b200 import quant
    for i, x, y, axis, bits, gs in _cases():
        got = quant._grouped_affine_quant_dequant(x.cuda(), bits, axis, gs)
        assert got.dtype == x.dtype and got.shape == x.shape
        assert torch.equal(got.float().cpu(), y), f"case {i}: {(got.float().cpu() != y).sum().item()} elements differ"
    z = np.load(f"{GOLDEN_DIR}/fake_quant.npz")
    k = torch.from_numpy(z["key.x"].view(np.float16)).cuda()
    assert torch.equal(quant.quantize_key(k, 2, 32).cpu(), torch.from_numpy(z["key.y"].view(np.float16)))
    assert torch.equal(quant.quantize_value(k, 4, 32).cpu(), torch.from_numpy(z["value.y"].view(np.float16)))
    qk, qv = quant.quantize_kv(k, k, 2, 4)
    assert torch.equal(qk, quant.quantize_key(k, 2)) and torch.equal(qv, quant.quantize_value(k, 4))
    assert quant.quantize_key(k, 16) is k
    with pytest.raises(ValueError):
        quant.quantize_key(k, 0)
    with pytest.raises(RuntimeError):
        quant.quantize_key(k.cpu(), 2)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_in_place_slices_equal_the_copy_out_and_back_of_the_reference(oracle, dtype):
    """t[:, :, a:b, :] = quantize(t[:, :, a:b, :]) for K and V, group sizes that do and do not divide head_dim."""
    from phasekv_b200 import quant
    gen = torch.Generator().manual_seed(5)
    for (b, h, s, hd, a, e, bits, gs) in [(1, 4, 300, 128, 64, 203, 4, 32), (2, 2, 50, 64, 0, 50, 2, 32),
                                          (1, 2, 40, 24, 3, 37, 3, 16), (1, 2, 64, 128, 10, 11, 8, 0)]:
        k = torch.randn(b, h, s, hd, generator=gen).to(dtype)
        v = torch.randn(b, h, s, hd, generator=gen).to(dtype)
        want_k, want_v = k.clone(), v.clone()
        want_k[:, :, a:e, :] = oracle.quantize_key(k[:, :, a:e, :], bits, gs)
        want_v[:, :, a:e, :] = oracle.quantize_value(v[:, :, a:e, :], bits, gs)
        gk, gv = k.cuda(), v.cuda()
        quant.fake_quant_(gk, a, e, bits, -2, gs)
        quant.fake_quant_(gv, a, e, bits, -1, gs)
        assert torch.equal(gk.cpu(), want_k), (b, h, s, hd, a, e, bits, gs)
        assert torch.equal(gv.cpu(), want_v), (b, h, s, hd, a, e, bits, gs)


def test_signal_topk_and_gather(oracle):
    from phasekv_b200 import hetero_cache as hc
    gen = torch.Generator().manual_seed(8)
    v = torch.randn(2, 4, 200, 128, generator=gen).half()
    sig = hc.value_norm_signal(v.cuda(), slice(40, 104))
    want = torch.linalg.vector_norm(v[:, :, 40:104, :].float(), dim=-1)
    assert sig.shape == (2, 4, 64) and torch.allclose(sig.cpu(), want, rtol=1e-5, atol=1e-6)
    idx = hc.topk_per_head(sig, 32)
    want_idx, gap = oracle.value_norm_topk(v[:, :, 40:104, :], 32)
    assert gap.min() > 1e-5, "seeded data has a near-tie at the selection boundary"
    assert torch.equal(idx.cpu(), want_idx)
    assert hc.topk_per_head(sig, 0).shape == (2, 4, 0) and hc.topk_per_head(sig, 1000).shape == (2, 4, 64)
    # ties go to the lower position
    flat = torch.zeros(1, 1, 10, device="cuda")
    assert hc.topk_per_head(flat, 3).tolist() == [[[0, 1, 2]]]
    # NaN ranks as the largest value (torch.topk's order) and exactly `keep` positions come back
    nan_row = torch.tensor([[[1.0, float("nan"), 3.0, float("nan"), 2.0, -1.0]]], device="cuda")
    assert hc.topk_per_head(nan_row, 3).tolist() == [[[1, 2, 3]]]
    with pytest.raises(RuntimeError):
        hc.topk_per_head(torch.zeros(1, 1, 8), 2)  # host tensors are refused: there is no CPU path
    # a whole prompt's candidates per head (radix select): same positions as a sort, ties to the lower position
    gen = torch.Generator().manual_seed(5)
    long = torch.randn(2, 4, 40000, generator=gen)
    long[0, 0, 100:4000] = 0.5          # a long run of equal scores across the selection boundary
    long[1, 2, 17] = float("nan")
    for keep in (1, 777, 20000, 39999):
        got = hc.topk_per_head(long.cuda(), keep).cpu()
        key = torch.where(torch.isnan(long), torch.full_like(long, float("inf")), long)
        order = torch.sort(key, dim=-1, descending=True, stable=True).indices[..., :keep]
        assert torch.equal(got, order.sort(dim=-1).values), keep
    g = hc.gather_tokens(v.cuda(), idx + 40)
    want_g = v.gather(2, (want_idx + 40).unsqueeze(-1).expand(2, 4, 32, 128))
    assert torch.equal(g.cpu(), want_g)


def _fake_cache(layers, b, h, s, hd, seed, dtype=torch.float16):
    gen = torch.Generator().manual_seed(seed)
    c = types.SimpleNamespace(key_cache=[], value_cache=[])
    for _ in range(layers):
        c.key_cache.append(torch.randn(b, h, s, hd, generator=gen).to(dtype))
        c.value_cache.append(torch.randn(b, h, s, hd, generator=gen).to(dtype))
    return c


def test_decode_tier_and_prompt_tier_lifecycle_against_a_cpu_restatement(oracle):
    """Prompt packing, then decode steps that append a token per layer and call maintain(): the dense cache must end
    up bit-identical to the same procedure restated on the CPU with the oracle's operators
    (decode_tier.py:25-88, prompt_tier.py:78-118 of the reference)."""
    from phasekv_b200 import decode_tier, hetero_cache as hc, prompt_tier
    layers, b, h, hd, prompt = 2, 1, 2, 64, 70
    cpu = _fake_cache(layers, b, h, prompt, hd, seed=3)
    gpu = types.SimpleNamespace(key_cache=[t.cuda() for t in cpu.key_cache], value_cache=[t.cuda() for t in cpu.value_cache])
    keep = [torch.stack([torch.randperm(prompt, generator=torch.Generator().manual_seed(10 + l + 7 * i))[:48]
                         for i in range(h)]).unsqueeze(0) for l in range(layers)]
    st_gpu = hc.HeteroTierState(prompt_bits=2, cold_bits=4, group_size=32, recent_window=4)
    st_cpu = hc.HeteroTierState(prompt_bits=2, cold_bits=4, group_size=32, recent_window=4)
    prompt_tier.pack_selected(gpu, [k.cuda() for k in keep], st_gpu)

    def cpu_gather(t, idx):
        return t.gather(2, idx.unsqueeze(-1).expand(*idx.shape, t.shape[-1])).contiguous()

    for l in range(layers):
        idx = keep[l].sort(dim=-1).values
        cpu.key_cache[l], cpu.value_cache[l] = cpu_gather(cpu.key_cache[l], idx), cpu_gather(cpu.value_cache[l], idx)
        cpu.key_cache[l] = oracle.quantize_key(cpu.key_cache[l], 2, 32)
        cpu.value_cache[l] = oracle.quantize_value(cpu.value_cache[l], 2, 32)
    st_cpu.prompt_len_phys = 48
    assert st_gpu.prompt_len_phys == 48
    gen = torch.Generator().manual_seed(77)
    for step in range(14):
        for l in range(layers):
            nk, nv_ = torch.randn(b, h, 1, hd, generator=gen).half(), torch.randn(b, h, 1, hd, generator=gen).half()
            cpu.key_cache[l] = torch.cat([cpu.key_cache[l], nk], dim=2)
            cpu.value_cache[l] = torch.cat([cpu.value_cache[l], nv_], dim=2)
            gpu.key_cache[l] = torch.cat([gpu.key_cache[l], nk.cuda()], dim=2)
            gpu.value_cache[l] = torch.cat([gpu.value_cache[l], nv_.cuda()], dim=2)
        decode_tier.maintain(gpu, step=step, model_config=None, state=st_gpu, decode_keep_ratio=0.5, lazy_g=4)
        # the same on the CPU
        seq = cpu.key_cache[0].shape[2]
        aged = seq - st_cpu.prompt_len_phys - st_cpu.cold_len - st_cpu.recent_window
        if aged >= 4:
            base = st_cpu.prompt_len_phys + st_cpu.cold_len
            keep_b = max(1, int(round(0.5 * aged)))
            for l in range(layers):
                sel, gap = oracle.value_norm_topk(cpu.value_cache[l][:, :, base:base + aged, :], keep_b)
                assert gap.min() > 1e-5
                idx = torch.cat([torch.arange(base).view(1, 1, -1).expand(b, h, -1), sel + base,
                                 torch.arange(base + aged, seq).view(1, 1, -1).expand(b, h, -1)], dim=-1)
                cpu.key_cache[l], cpu.value_cache[l] = cpu_gather(cpu.key_cache[l], idx), cpu_gather(cpu.value_cache[l], idx)
                cpu.key_cache[l][:, :, base:base + keep_b, :] = oracle.quantize_key(cpu.key_cache[l][:, :, base:base + keep_b, :], 4, 32)
                cpu.value_cache[l][:, :, base:base + keep_b, :] = oracle.quantize_value(cpu.value_cache[l][:, :, base:base + keep_b, :], 4, 32)
            st_cpu.cold_len += keep_b
        assert st_gpu.cold_len == st_cpu.cold_len, step
    assert st_gpu.cold_len > 0
    for l in range(layers):
        assert torch.equal(gpu.key_cache[l].cpu(), cpu.key_cache[l]), l
        assert torch.equal(gpu.value_cache[l].cpu(), cpu.value_cache[l]), l
    assert st_gpu.logical_bytes(gpu) == st_cpu.logical_bytes(cpu) > 0


def test_prompt_selection_matches_the_reference():
    """prompt_tier.select_prompt_indices on seeded causal attention matrices: the kept positions per layer and
    head are the reference's (prompt_tier.py:24-75), including short prompts where sinks and the recent window
    fill the budget.  The vectors were made by the reference's own function."""
    import os
    import types

    import numpy as np

    from phasekv_b200 import hetero_cache as hc
    from phasekv_b200 import prompt_tier
    z = np.load(os.path.join(os.path.dirname(__file__), "golden", "prompt_select.npz"))
    ties = 0
    for i in range(int(z["n_cases"][0])):
        plen, hq, hkv, layers, batch, sink, obs, kernel, avg = (int(v) for v in z[f"c{i}.args"])
        atts = [torch.from_numpy(a).cuda() for a in z[f"c{i}.att"]]
        cfg = types.SimpleNamespace(num_key_value_heads=hkv, num_attention_heads=hq)
        keep = prompt_tier.select_prompt_indices(
            atts, prompt_len=plen, model_config=cfg, prefill_keep_ratio=float(z[f"c{i}.ratio"][0]), sink_tokens=sink,
            obs_window=obs, pool_kernel=kernel, pooling="avgpool" if avg else "maxpool")
        want = torch.from_numpy(z[f"c{i}.keep"])
        assert len(keep) == layers
        for l in range(layers):
            got = keep[l].cpu()
            assert keep[l].dtype == torch.long and got.shape == want[l].shape
            assert bool((got[..., 1:] > got[..., :-1]).all())
            if torch.equal(got, want[l]):
                continue
            # Max-pooled votes of neighbouring positions are often EQUAL, and which of several equal votes fills the
            # last places is not defined by the reference (it is whatever torch.topk does on the device at hand).
            # Here equal votes go to the lowest position.  The two selections must then hold the same votes:
            ratio = float(z[f"c{i}.ratio"][0])
            budget = min(plen, max(1, min(sink, plen), round(plen * ratio)))
            first = min(sink, plen, budget)                                  # candidates: behind the sinks ...
            last = plen - min(obs, budget - first, plen - first)             # ... and before the recent window
            votes = hc.pool_scores(hc.observation_votes(atts[l], hkv, min(obs, plen))[..., first:last], kernel,
                                   "avgpool" if avg else "maxpool").cpu()

            def chosen_votes(idx):
                inside = (idx >= first) & (idx < last)
                per_head = budget - first - (plen - last)
                assert bool((inside.sum(-1) == per_head).all())
                picked = votes.gather(-1, (idx - first).clamp(0, last - first - 1))[inside]
                return picked.view(*idx.shape[:2], per_head).sort(-1).values
            ties += 1
            assert torch.equal(chosen_votes(got), chosen_votes(want[l])), (i, l)
    assert ties <= 4


@torch.inference_mode()
def test_compressor_hooks_drive_a_transformers_cache_of_this_generation():
    """PhaseKVCompressor.on_prefill / on_decode_step (compressor.py:134-148 of the reference) over the dense cache a
    randomly initialised Qwen2 returns: whatever cache class the installed transformers uses (per-layer lists in 4.x,
    layer objects in 5.x), the result equals the same hooks run on plain per-layer lists of the same tensors."""
    transformers = pytest.importorskip("transformers")
    from transformers import Qwen2Config, Qwen2ForCausalLM
    from phasekv_b200 import hetero_cache as hc
    from phasekv_b200.compressor import PhaseKVCompressor
    torch.manual_seed(3)
    config = Qwen2Config(vocab_size=97, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                         num_key_value_heads=2, max_position_embeddings=256, attention_dropout=0.0, attn_implementation="eager")
    model = Qwen2ForCausalLM(config).to("cuda", torch.float16).eval()
    ids = torch.randint(1, 97, (1, 80), generator=torch.Generator().manual_seed(5)).cuda()
    out = model(input_ids=ids, use_cache=True, output_attentions=True)
    cache = out.past_key_values
    settings = types.SimpleNamespace(prefill_keep_ratio=0.5, decode_keep_ratio=0.5, recent_window=4, sink_tokens=2, bits=2,
                                     extra={"cold_bits": 4, "group_size": 16, "lazy_g": 4, "obs_window": 8, "pool_kernel": 5})
    ours, plain = PhaseKVCompressor(settings), PhaseKVCompressor(settings)
    lists = types.SimpleNamespace(key_cache=[hc.layer_kv(cache, l)[0].clone() for l in range(2)],
                                  value_cache=[hc.layer_kv(cache, l)[1].clone() for l in range(2)])
    ours.reset(config), plain.reset(config)
    ours.on_prefill(cache, attentions=out.attentions, prompt_len=80, model_config=config)
    plain.on_prefill(lists, attentions=out.attentions, prompt_len=80, model_config=config)
    assert hc.cache_seq_len(cache) == 40 == ours.state.prompt_len_phys and cache.get_seq_length() == 40
    token = out.logits[:, -1].argmax(-1, keepdim=True)
    for step in range(12):
        before = hc.cache_seq_len(cache)
        step_out = model(input_ids=token, past_key_values=cache, use_cache=True,
                         position_ids=torch.tensor([[80 + step]], device="cuda"))
        assert hc.cache_seq_len(cache) == before + 1
        for l in range(2):       # the plain lists receive the very same new token
            k, v = hc.layer_kv(cache, l)
            lists.key_cache[l] = torch.cat([lists.key_cache[l], k[:, :, -1:, :]], dim=2)
            lists.value_cache[l] = torch.cat([lists.value_cache[l], v[:, :, -1:, :]], dim=2)
        ours.on_decode_step(cache, step=step, model_config=config)
        plain.on_decode_step(lists, step=step, model_config=config)
        token = step_out.logits[:, -1].argmax(-1, keepdim=True)
        assert torch.isfinite(step_out.logits).all()
    assert ours.state.cold_len == plain.state.cold_len > 0
    for l in range(2):
        k, v = hc.layer_kv(cache, l)
        assert torch.equal(k, lists.key_cache[l]) and torch.equal(v, lists.value_cache[l])
    assert ours.cache_memory_bytes(cache) == plain.cache_memory_bytes(lists) > 0
    assert ours.describe()["phasekv"]["cold_bits"] == 4
    with pytest.raises(ValueError):
        PhaseKVCompressor(types.SimpleNamespace(extra={"use_planner": True}))
