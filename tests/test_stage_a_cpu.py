"""Stage-A fake quantisation: the C oracle against vectors produced by the reference's quant.py."""
import numpy as np
import torch

from tests.conftest import GOLDEN as GOLDEN_DIR

DTYPES = [torch.float16, torch.bfloat16, torch.float32]


def _cases():
    z = np.load(f"{GOLDEN_DIR}/fake_quant.npz")
    for i in range(int(z["n_cases"][0])):
        axis, bits, gs, dt = (int(v) for v in z[f"c{i}.args"])
        yield i, torch.from_numpy(z[f"c{i}.x"]).to(DTYPES[dt]), torch.from_numpy(z[f"c{i}.y"]), axis, bits, gs
    return z


def test_oracle_fake_quant_matches_the_reference_bit_for_bit(oracle):
    n = 0
    for i, x, y, axis, bits, gs in _cases():
        got = oracle.fake_quant(x, bits, axis, gs)
        assert got.dtype == x.dtype and got.shape == x.shape
        assert torch.equal(got.float(), y), f"case {i}: {(got.float() != y).sum().item()} elements differ"
        n += 1
    assert n >= 10
    z = np.load(f"{GOLDEN_DIR}/fake_quant.npz")
    k = torch.from_numpy(z["key.x"].view(np.float16))
    assert torch.equal(oracle.quantize_key(k, 2, 32), torch.from_numpy(z["key.y"].view(np.float16)))
    assert torch.equal(oracle.quantize_value(k, 4, 32), torch.from_numpy(z["value.y"].view(np.float16)))
    assert oracle.fake_quant(k, 16, -1, 32) is k


def test_logical_byte_accounting_matches_the_reference():
    from phasekv_b200 import quant
    z = np.load(f"{GOLDEN_DIR}/fake_quant.npz")
    want = [int(v) for v in z["bytes"]]
    got = [quant.quantized_tier_bytes(1000, 28, 4, 128, 2, 2, 32, 1),
           quant.quantized_tier_bytes(77, 2, 2, 64, 4, 16, 0, 3),
           quant.fp16_tier_bytes(128, 28, 4, 128, 2),
           *quant.kv_group_counts(1000, 128, 32), *quant.kv_group_counts(5, 8, 0)]
    assert got == want
    assert quant.quantized_tier_bytes(0, 1, 1, 8, 2, 2) == 0 and quant.kv_group_counts(0, 8, 32) == (0, 0)


def test_prompt_selection_refuses_bad_arguments_before_any_launch():
    import types

    import pytest

    from phasekv_b200 import prompt_tier
    cfg = types.SimpleNamespace(num_key_value_heads=2, num_attention_heads=4)
    for bad in (dict(attentions=None), dict(prompt_len=0), dict(prefill_keep_ratio=0.0), dict(sink_tokens=-1), dict(obs_window=0)):
        args = dict(attentions=[torch.rand(1, 4, 8, 8)], prompt_len=8, model_config=cfg, prefill_keep_ratio=0.5,
                    sink_tokens=1, obs_window=2, pool_kernel=3, pooling="maxpool")
        args.update(bad)
        with pytest.raises(ValueError):
            prompt_tier.select_prompt_indices(args.pop("attentions"), **args)


def test_compressor_reads_and_validates_its_configuration():
    """compressor.py:41-100 of the reference: defaults, the extra dictionary, and the refusals of _validate()."""
    import types

    import pytest

    from phasekv_b200.compressor import PhaseKVCompressor
    c = PhaseKVCompressor(types.SimpleNamespace(prefill_keep_ratio=None, decode_keep_ratio=None, recent_window=None,
                                                sink_tokens=4, bits=None, extra={}))
    assert (c.prefill_keep_ratio, c.decode_keep_ratio, c.recent_window, c.sink_tokens) == (0.5, 1.0, 32, 4)
    assert (c.prompt_bits, c.cold_bits, c.group_size, c.lazy_g, c.obs_window, c.pool_kernel, c.pooling) == (2, 4, 32, 16, 32, 7, "maxpool")
    assert c.requires_attention and c.physically_evicts
    c = PhaseKVCompressor(types.SimpleNamespace(bits=4, extra={"prompt_bits": 3, "cold_bits": 8, "lazy_g": 5}))
    assert (c.prompt_bits, c.cold_bits, c.lazy_g) == (3, 8, 5) and c.state.prompt_bits == 3 and c.state.cold_bits == 8
    c.state.prompt_len_phys = 9
    c.reset()
    assert c.state.prompt_len_phys == 0 and c.describe()["phasekv"]["lazy_g"] == 5
    for bad in (dict(bits=5), dict(extra={"cold_bits": 6}), dict(prefill_keep_ratio=0.0), dict(decode_keep_ratio=1.2),
                dict(recent_window=0), dict(extra={"group_size": 0}), dict(extra={"lazy_g": -1}), dict(extra={"obs_window": 0}),
                dict(extra={"use_planner": True}), dict(extra={"target_memory_ratio": 0.3})):
        with pytest.raises(ValueError):
            PhaseKVCompressor(types.SimpleNamespace(**bad))
