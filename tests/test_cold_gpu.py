"""Cold-tier cooling kernel (selection + pack + hot compaction) against the golden fixtures
(reference arithmetic) and the oracle."""
import pytest
import torch

from conftest import from_f16, load_packed
from util import assert_packed_equal

pytestmark = pytest.mark.gpu


def test_golden_cold_cases(golden):
    from phasekv_b200.cold_tier import select_and_pack_cold
    z = golden("cold_select.npz")
    for i in range(int(z["n_cases"][0])):
        window, keep, aged, bits, gs = (int(v) for v in z[f"k{i}.args"])
        hot_k, hot_v = from_f16(z[f"k{i}.hot_k"]), from_f16(z[f"k{i}.hot_v"])
        hot_len = hot_k.shape[2]
        cap = hot_len + 5
        bk = torch.zeros(hot_k.shape[0], hot_k.shape[1], cap, hot_k.shape[3], dtype=torch.float16, device="cuda")
        bv = torch.zeros_like(bk)
        bk[:, :, :hot_len], bv[:, :, :hot_len] = hot_k.cuda(), hot_v.cuda()
        seg, idx = select_and_pack_cold(bk, bv, hot_len, aged, keep, bits, gs, return_indices=True)
        if keep < aged:
            assert torch.equal(idx.cpu(), torch.from_numpy(z[f"k{i}.indices"])), f"case {i}: selection"
        assert_packed_equal(seg.key, load_packed(z, f"k{i}.key"), f"case {i} key")
        assert_packed_equal(seg.value, load_packed(z, f"k{i}.value"), f"case {i} value")
        # surviving hot tokens moved to the front, bit for bit
        rest = hot_len - aged
        assert torch.equal(bk[:, :, :rest].cpu(), hot_k[:, :, aged:])
        assert torch.equal(bv[:, :, :rest].cpu(), hot_v[:, :, aged:])


def test_known_answer_selection():
    """tests/test_phasekv_cache.py:155-182 of the reference."""
    from phasekv_b200.cold_tier import cool_aged_tokens
    from phasekv_b200.kernels.packing import unpack_dequantize
    from phasekv_b200.kernels.tiers import LayerTiers
    hot_k = torch.zeros(1, 2, 4, 8, dtype=torch.float16, device="cuda")
    hot_v = torch.zeros_like(hot_k)
    layer = LayerTiers(prompt=None, hot_k=hot_k, hot_v=hot_v, hot_len=0)
    tokens = []
    for step, strengths in enumerate(((9, 1), (1, 9), (3, 3), (4, 4))):
        value = torch.tensor(strengths, dtype=torch.float16).view(1, 2, 1, 1).expand(1, 2, 1, 8)
        key = torch.full_like(value, step + 1)
        tokens.append((key, value))
        hot_k[:, :, layer.hot_len:layer.hot_len + 1] = key.cuda()
        hot_v[:, :, layer.hot_len:layer.hot_len + 1] = value.cuda()
        layer.hot_len += 1
        cooled = cool_aged_tokens(layer, recent_window=2, lazy_g=2, decode_keep_ratio=0.5, cold_bits=4, group_size=4)
        assert cooled == (step == 3)
    cold_key = unpack_dequantize(layer.cold[0].key).cpu()
    assert torch.equal(cold_key[0, :, 0, 0], torch.tensor([1., 2.], dtype=torch.float16))
    assert torch.equal(unpack_dequantize(layer.cold[0].value).cpu(), torch.full_like(cold_key, 9))
    hk, hv = layer.hot_views()
    assert torch.equal(hk.cpu(), torch.cat([t[0] for t in tokens[2:]], dim=2))
    assert torch.equal(hv.cpu(), torch.cat([t[1] for t in tokens[2:]], dim=2))


def test_cold_batch_of_64_against_oracle(oracle):
    """The lazy cold batch configuration: 64 aged tokens, top-50% by value norm, 4-bit, per KV head."""
    from phasekv_b200 import workloads
    from phasekv_b200.cold_tier import select_and_pack_cold
    for seed in range(4):
        gen = torch.Generator().manual_seed(100 + seed)
        hk, hv = workloads.make_kv(gen, 4, 192, 128)
        idx_ref, gap = oracle.value_norm_topk(hv[:, :, :64], 32)
        bk, bv = hk.cuda().clone(), hv.cuda().clone()
        seg, idx = select_and_pack_cold(bk, bv, 192, 64, 32, 4, 32, return_indices=True)
        assert torch.equal(idx.cpu(), idx_ref), f"selection differs; boundary gap {gap.min().item():.2e}"
        gi = idx_ref.unsqueeze(-1).expand(1, 4, 32, 128)
        assert_packed_equal(seg.key, oracle.quantize_pack(hk[:, :, :64].gather(2, gi).contiguous(), 4, -2, 32))
        assert_packed_equal(seg.value, oracle.quantize_pack(hv[:, :, :64].gather(2, gi).contiguous(), 4, -1, 32))
        assert torch.equal(bk[:, :, :128].cpu(), hk[:, :, 64:])
