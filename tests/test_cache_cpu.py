"""The cache's state machine on the CPU: every refusal that the reference's tests/test_phasekv_cache.py:84-222 checks
by its wording happens before any kernel is launched, so it can be exercised with hand-made tiers on CPU tensors
(packing, cooling and attention themselves are GPU tests)."""
import pytest
import torch


def make_cache(layers=2, heads=2, hd=8, prompt=20, capacity=6, **options):
    from phasekv_b200.kernels.packing import PackedTensor
    from phasekv_b200.kernels.tiers import LayerTiers, PackedKVSegment
    from phasekv_b200.phasekv_cache import PhaseKVCache
    shape = (1, heads, prompt, hd)

    def packed(axis):
        moved = [s for i, s in enumerate(shape) if i != axis]
        length = shape[axis]
        return PackedTensor(torch.zeros(*moved, (length + 3) // 4, dtype=torch.uint8), torch.ones(*moved, 1, dtype=torch.float16),
                            torch.zeros(*moved, 1, dtype=torch.float16), 2, axis, length, shape, length)
    tiers = [LayerTiers(prompt=PackedKVSegment(packed(2), packed(3)),
                        hot_k=torch.zeros(1, heads, capacity, hd, dtype=torch.float16),
                        hot_v=torch.zeros(1, heads, capacity, hd, dtype=torch.float16)) for _ in range(layers)]
    settings = dict(seen_tokens=prompt, prompt_bits=2, cold_bits=4, group_size=32, recent_window=4, lazy_g=2,
                    decode_keep_ratio=1.0)
    settings.update(options)
    return PhaseKVCache(tiers, **settings)


def test_dense_update_is_rejected_and_a_step_needs_every_layer():
    cache = make_cache()
    with pytest.raises(RuntimeError, match="不返回稠密"):
        cache.update(torch.zeros(1), torch.zeros(1), 0)
    with pytest.raises(RuntimeError, match="每一层"):
        cache.finish_decode_step()
    with pytest.raises(RuntimeError, match=r"\[0, 1\]"):
        cache.finish_decode_step()
    assert cache.get_seq_length() == 20 and cache.true_seq_length == 20 and len(cache) == 2
    assert cache.get_max_cache_shape() is None and cache.get_mask_sizes(3, 0) == (23, 0)
    assert cache.get_mask_sizes(torch.arange(5), 1) == (25, 0) and cache.is_compileable is False


def test_invalid_config_fails_in_the_constructor():
    for bad in (dict(prompt_bits=3), dict(cold_bits=16), dict(group_size=0), dict(recent_window=1.5), dict(lazy_g=True),
                dict(decode_keep_ratio=0.0), dict(decode_keep_ratio=1.5), dict(seen_tokens=0)):
        with pytest.raises(ValueError, match=next(iter(bad))):
            make_cache(**bad)


def test_invalid_layer_and_failed_writes_do_not_advance_state():
    cache = make_cache()
    key = torch.ones(1, 2, 1, 8, dtype=torch.float16)
    for layer_idx in (-1, 2, 0.5, True):
        with pytest.raises(IndexError, match="layer_idx"):
            cache.append_hot(layer_idx, key, key)
    with pytest.raises(ValueError, match="float16"):
        cache.append_hot(0, key.float(), key.float())
    with pytest.raises(ValueError, match="shape"):
        cache.append_hot(0, key[:, :1], key[:, :1])
    assert cache.get_seq_length() == 20 and cache.layer_tiers(0).hot_len == 0
    cache.append_hot(0, key, key)
    assert cache.true_seq_length == 20 and cache.get_seq_length(0) == 21 and cache.get_seq_length(1) == 20
    with pytest.raises(RuntimeError, match="第 0 层.*已追加"):
        cache.append_hot(0, key, key)
    with pytest.raises(RuntimeError, match=r"尚未追加的层为 \[1\]"):
        cache.finish_decode_step()
    with pytest.raises(RuntimeError, match="decode 步内"):
        cache.begin_prompt_chunk(2)
    with pytest.raises(RuntimeError, match="decode 步内"):
        cache.reorder_cache(torch.tensor([0]))
    cache.append_hot(1, key * 3, key * 5)
    cache.finish_decode_step()          # one hot token: nothing has aged out of the window of four
    assert cache.true_seq_length == 21 and cache.layer_tiers(1).hot_len == 1 and cache.layer_tiers(1).cold == []
    hk, hv = cache.layer_tiers(1).hot_views()
    assert torch.equal(hk, key * 3) and torch.equal(hv, key * 5)
    with pytest.raises(RuntimeError, match=r"\[0, 1\]"):
        cache.finish_decode_step()


def test_prompt_chunk_state_errors():
    cache = make_cache(capacity=4, recent_window=2, lazy_g=2)
    key = torch.ones(1, 2, 1, 8, dtype=torch.float16)
    with pytest.raises(RuntimeError, match="begin_prompt_chunk"):
        cache.append_prompt_token(0, key, key)
    with pytest.raises(RuntimeError, match="begin_prompt_chunk"):
        cache.finish_prompt_chunk()
    for length in (0, 1.5, True):
        with pytest.raises(ValueError, match="length"):
            cache.begin_prompt_chunk(length)
    assert cache.prompt_chunk_len == 0
    cache.begin_prompt_chunk(5)          # more than the hot capacity: the buffers grow
    assert cache.prompt_chunk_len == 5 and cache.layer_tiers(0).hot_k.shape[2] == 5
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


def test_reorder_rejects_invalid_indices_before_touching_anything():
    cache = make_cache()
    for bad in (torch.tensor([[0]]), torch.tensor([0.0]), torch.tensor([], dtype=torch.long), torch.tensor([1]), torch.tensor([-1]), [0]):
        with pytest.raises(ValueError, match="beam_idx"):
            cache.reorder_cache(bad)
    prompt = cache.layer_tiers(0).prompt
    assert cache.layer_tiers(0).prompt is prompt
