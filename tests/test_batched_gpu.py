"""Batched serving decode: many sequences through one split-K launch and one merge launch."""
import pytest
import torch

from tests.conftest import attention_close
from tests.test_decode_gpu import _pack_tiers
from tests.util import make_tiers, remove_batch, to_gpu_packed

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def attn():
    from phasekv_b200.kernels import attention_cuda
    return attention_cuda


def _batch(oracle, shape, specs, bits=2, cold_bits=4):
    """specs: (prompt, [cold...], hot) per sequence -> tiers list, q [B, Hq, hd] (CPU), oracle outputs."""
    tiers, qs, refs = [], [], []
    for i, (p, cold, h) in enumerate(specs):
        segs, hk, hv, q = _pack_tiers(oracle, shape, p, bits, cold, cold_bits, h, seed=4242 + 17 * i)
        q2 = q[0, :, 0, :]
        refs.append(oracle.segments_decode_reference(q2, segs, hk if h else None, hv if h else None,
                                                     shape.num_q_heads))
        tiers.append(make_tiers(segs, hk if h else None, hv if h else None, hot_len=h))
        qs.append(q2)
    return tiers, torch.stack(qs), refs


def test_batched_equals_per_sequence_and_oracle(oracle, attn):
    """Ragged batch: lengths on and off the 64-token grid, with and without cold / hot tiers, several cold
    segments.  Every row must meet the parity bar against the oracle and agree with the batch-1 entry point
    (the split points differ, so agreement is to float32 merge accuracy, not bit for bit)."""
    from phasekv_b200 import workloads
    shape = workloads.QWEN2_5_7B
    specs = [(8192, [512], 128), (6150, [384], 97), (10240, [640], 160), (64, [], 0), (1, [], 1),
             (4097, [64, 64, 64], 33), (7000, [500], 0), (12288, [], 128), (9999, [777], 191)]
    tiers, q, refs = _batch(oracle, shape, specs)
    plan = attn.BatchDecodePlan(tiers, shape.num_q_heads)
    assert plan.batch == len(specs) and plan.work_items >= len(specs)
    out = plan.run(q.cuda())
    assert out.shape == q.shape and torch.isfinite(out).all()
    for i in range(len(specs)):
        attention_close(out[i], refs[i])
        single = attn.fused_phasekv_decode(q[i].cuda(), tiers[i], shape.num_q_heads)
        assert (out[i].float() - single.float()).abs().max().item() <= 1e-3, i
    # the plan is reusable: other queries, same tiers
    q2 = torch.roll(q, 1, dims=0).contiguous()
    out2 = attn.fused_phasekv_decode_batched(q2.cuda(), plan, shape.num_q_heads)
    for i in (0, 3, 8):
        single = attn.fused_phasekv_decode(q2[i].cuda(), tiers[i], shape.num_q_heads)
        assert (out2[i].float() - single.float()).abs().max().item() <= 1e-3, i


@pytest.mark.parametrize("bits", [4, 8])
def test_batched_other_bit_widths(oracle, attn, bits):
    from phasekv_b200 import workloads
    shape = workloads.QWEN2_5_7B
    specs = [(2048, [256], 64), (1500, [], 10), (3000, [128], 128)]
    tiers, q, refs = _batch(oracle, shape, specs, bits=bits, cold_bits=bits)
    out = attn.fused_phasekv_decode_batched(q.cuda(), tiers, shape.num_q_heads)
    for i in range(len(specs)):
        attention_close(out[i], refs[i])


def test_batched_serving_configuration_sample(oracle, attn):
    """64 sequences of the batched-serving configuration (8192 @2-bit + 512 @4-bit + 128 hot, +-25 % jitter)
    in one launch; a sample of rows is checked against the oracle, all rows against each other's finiteness."""
    from phasekv_b200 import workloads
    shape = workloads.QWEN2_5_7B
    lengths = workloads.jittered_lengths(0, 64, 8192, 512, 128, hot_capacity=192)
    order = sorted(range(64), key=lambda i: lengths[i][0])
    sample = {order[0], order[-1], order[20], order[41]}
    tiers, qs, refs = [], [], {}
    for i, (p, c, h) in enumerate(lengths):
        if i in sample:
            segs, hk, hv, q = _pack_tiers(oracle, shape, p, 2, [c], 4, h, seed=workloads.layer_seed(0, 5, i))
            refs[i] = oracle.segments_decode_reference(q[0, :, 0, :], segs, hk, hv, shape.num_q_heads)
            tiers.append(make_tiers(segs, hk, hv, hot_len=h))
            qs.append(q[0, :, 0, :].cuda())
        else:  # packed on the GPU: these rows only have to be finite and stay out of the others' way
            t, q = workloads.gpu_three_tier(shape, p, 2, c, 4, h, workloads.layer_seed(0, 5, i), "cuda")
            tiers.append(t)
            qs.append(q)
    out = attn.fused_phasekv_decode_batched(torch.stack(qs), tiers, shape.num_q_heads)
    assert torch.isfinite(out).all()
    for i, ref in refs.items():
        attention_close(out[i], ref)


def test_batched_rejects_what_it_cannot_take(oracle, attn):
    from phasekv_b200 import _native as nv
    from phasekv_b200 import workloads
    shape = workloads.QWEN2_0_5B  # head_dim 64: not a tensor-core shape
    tiers, q, _ = _batch(oracle, shape, [(256, [], 8)])
    with pytest.raises(nv.NativeError) as err:
        attn.BatchDecodePlan(tiers, shape.num_q_heads)
    assert err.value.code == nv.PKV_E_LAYOUT
    big = workloads.QWEN2_5_7B
    tiers, q, _ = _batch(oracle, big, [(256, [], 8), (128, [], 0)])
    plan = attn.BatchDecodePlan(tiers, big.num_q_heads)
    with pytest.raises(ValueError):
        plan.run(q[:1].cuda())
    with pytest.raises(ValueError):
        plan.run(q.cuda().float())
    with pytest.raises(ValueError):
        attn.BatchDecodePlan([], big.num_q_heads)
