"""Parity of the CUDA decode attention (through the C ABI) with the oracle and the golden fixtures.

The bar for attention is max-abs <= 2e-3 and max-abs / max|ref| <= 1e-2 against the
dequantise-then-attend semantics (conftest.attention_close)."""
import pytest
import torch

from conftest import attention_close, from_f16, load_packed
from util import make_tiers, remove_batch, to_gpu_packed

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def attn():
    from phasekv_b200.kernels import attention_triton
    return attention_triton


def _pack_tiers(oracle, shape, prompt, pbits, cold_lens, cbits, hot, seed, gsk=32, gsv=32):
    """Dense seeded tiers -> oracle-packed segments (CPU) in prompt, cold... order plus hot."""
    from phasekv_b200 import workloads
    gen = torch.Generator().manual_seed(seed)
    segs = []
    for length, bits in [(prompt, pbits)] + [(c, cbits) for c in cold_lens]:
        k, v = workloads.make_kv(gen, shape.num_kv_heads, length, shape.head_dim)
        segs.append((oracle.quantize_pack(k, bits, -2, gsk), oracle.quantize_pack(v, bits, -1, gsv)))
    hk = hv = None
    if hot:
        hk, hv = workloads.make_kv(gen, shape.num_kv_heads, hot, shape.head_dim)
    q = workloads.make_query(gen, shape.num_q_heads, shape.head_dim)
    return segs, hk, hv, q


def test_golden_c1_plumbing_case(golden, attn):
    z = golden("attention_c1.npz")
    segs = [(load_packed(z, "prompt_k"), load_packed(z, "prompt_v")),
            (load_packed(z, "cold_k"), load_packed(z, "cold_v"))]
    hk, hv = from_f16(z["hot_k"]), from_f16(z["hot_v"])
    tiers = make_tiers(segs, hk, hv, hot_len=hk.shape[2])
    q = from_f16(z["q"])
    out = attn.fused_phasekv_decode(q[0, :, 0, :].cuda(), tiers, q.shape[1])
    assert out.shape == (14, 64) and out.dtype == torch.float16
    attention_close(out, from_f16(z["out"])[0, :, 0, :])


def test_golden_small_ragged_cases(golden, attn):
    z = golden("attention_small.npz")
    for i in range(int(z["n_cases"][0])):
        segs = []
        for tier in ("prompt", "cold"):
            if f"a{i}.{tier}_k.meta" in z:
                segs.append((load_packed(z, f"a{i}.{tier}_k"), load_packed(z, f"a{i}.{tier}_v")))
        hk = hv = None
        if f"a{i}.hot_k" in z:
            hk, hv = from_f16(z[f"a{i}.hot_k"]), from_f16(z[f"a{i}.hot_v"])
        q = from_f16(z[f"a{i}.q"])
        if not segs:
            continue
        tiers = make_tiers(segs, hk, hv, hot_len=0 if hk is None else hk.shape[2])
        out = attn.fused_phasekv_decode(q[0, :, 0, :].cuda(), tiers, q.shape[1])
        attention_close(out, from_f16(z[f"a{i}.out"])[0, :, 0, :])


@pytest.mark.parametrize("length,heads,dim,kb,vb", [
    (1, 4, 8, 2, 4), (10, 4, 64, 8, 8), (127, 12, 128, 4, 4), (513, 12, 128, 2, 2),
    (8193, 12, 128, 4, 4), (28672, 12, 128, 4, 4), (129, 4, 256, 8, 4)])
def test_kivi_layer_partial_shapes_of_the_reference_test(oracle, attn, length, heads, dim, kb, vb):
    """The seven shapes and three launch options of the reference's
    tests/test_phasekv_launch_config.py:64-79 against a float32 dense-quantised softmax built in the
    test.  Every shape, on either kernel, meets the reference's own tolerance (atol 3e-4, rtol 1e-3); the
    largest excess measured on a B200 is -1.5e-4 (shape 513 x 12 x 128 at 2 bits: max-abs 2.5e-4)."""
    gen = torch.Generator().manual_seed(42)
    q = torch.randn(heads, dim, generator=gen).half()
    kd = torch.randn(2, length, dim, generator=gen).half()
    vd = torch.randn(2, length, dim, generator=gen).half()
    k, v = oracle.quantize_pack(kd, kb, 1, 32), oracle.quantize_pack(vd, vb, 2, 32)

    def dense_float(pt):
        codes = oracle.unpack_low_bits(pt.packed, pt.bits, pt.axis_len).float()
        groups = torch.arange(pt.axis_len) // pt.group_size
        return (codes * pt.scale.float()[..., groups] + pt.mins.float()[..., groups]).movedim(-1, pt.axis)

    dk = dense_float(k).repeat_interleave(heads // 2, dim=0)
    dv = dense_float(v).repeat_interleave(heads // 2, dim=0)
    probs = torch.softmax(torch.einsum("hd,hsd->hs", q.float(), dk) / dim ** 0.5, dim=-1)
    expected = torch.einsum("hs,hsd->hd", probs, dv)
    kg, vg = to_gpu_packed(k), to_gpu_packed(v)
    for options in ({}, {"num_splits": 8, "block_n": 64, "num_warps": 4}, {"num_splits": 3}):
        m, total, acc = attn._kivi_layer_partial(q.cuda(), kg, vg, heads, **options)
        assert m.shape == (heads,) and acc.shape == (heads, dim)
        torch.testing.assert_close((acc / total[:, None]).cpu(), expected, atol=3e-4, rtol=1e-3)


@pytest.mark.parametrize("prompt", [4096, 8192, 16384, 32768, 131072])
def test_qwen7b_single_layer_contexts(oracle, attn, prompt):
    """2-bit prompt of 4K..128K tokens + 256 cold tokens at 4 bits + 128 hot tokens (7B shape)."""
    from phasekv_b200 import workloads
    shape = workloads.QWEN2_5_7B
    segs, hk, hv, q = _pack_tiers(oracle, shape, prompt, 2, [256], 4, 128, seed=prompt)
    ref = oracle.segments_decode_reference(q[0, :, 0, :], segs, hk, hv, shape.num_q_heads)
    tiers = make_tiers(segs, hk, hv, hot_len=128)
    out = attn.fused_phasekv_decode(q[0, :, 0, :].cuda(), tiers, shape.num_q_heads)
    attention_close(out, ref)


def _exact_attention(oracle, q, key, value, heads):
    """float64 softmax attention over the exactly dequantised codes (no float16 rounding of K or V)."""
    def dense(pt):
        codes = oracle.unpack_low_bits(pt.packed, pt.bits, pt.axis_len).double()
        groups = torch.arange(pt.axis_len) // pt.group_size
        return (codes * pt.scale.double()[..., groups] + pt.mins.double()[..., groups]).movedim(-1, pt.axis)
    dk, dv = dense(key), dense(value)
    if dk.ndim == 4:  # a batch dimension of one
        dk, dv = dk[0], dv[0]
    rep = heads // dk.shape[0]
    dk, dv = dk.repeat_interleave(rep, 0), dv.repeat_interleave(rep, 0)
    probs = torch.softmax(torch.einsum("hd,hsd->hs", q.double(), dk) / q.shape[-1] ** 0.5, dim=-1)
    return torch.einsum("hs,hsd->hd", probs, dv).float()


# (bits, S) -> measured |out - oracle| of the cases that exceed the 2e-3 bar, with the oracle's own distance from the
# exact attention over the codes beside it.  In each of them the kernel is the one nearer the exact result (the
# oracle rounds K and V to float16 before the softmax, as reference.py does): the oracle sits 2.8e-3 from exact
# there, the kernel 5.2e-4.
RAGGED_EXCEPTIONS = {(4, 127): {"kernel_vs_oracle": 2.93e-3, "oracle_vs_exact": 2.79e-3}}


@pytest.mark.parametrize("bits", [2, 4, 8])
def test_ragged_lengths_on_the_tensor_core_path(oracle, attn, bits):
    """Any segment length: rows that start on odd bytes, partial last groups, partial last bytes.

    Every case is held to the parity bar itself (max-abs <= 2e-3 and <= 1e-2 of max|ref| against the oracle)
    except the enumerated ones above, and every case, the exceptions included, to 1.5e-3 from the exact
    float64 attention over the codes (with a handful of tokens the output is of order |v| ~ 2..3, where half a
    float16 step is 1e-3)."""
    from phasekv_b200 import workloads
    shape = workloads.QWEN2_5_7B
    for S in (1, 3, 31, 63, 64, 65, 127, 129, 1000, 4097, 8193):
        segs, hk, hv, q = _pack_tiers(oracle, shape, S, bits, [], 4, 0, seed=1000 * bits + S)
        q2 = q[0, :, 0, :]
        ref = oracle.segments_decode_reference(q2, segs, None, None, shape.num_q_heads).float()
        exact = _exact_attention(oracle, q2, segs[0][0], segs[0][1], shape.num_q_heads)
        out = attn.fused_phasekv_decode(q2.cuda(), make_tiers(segs), shape.num_q_heads).float().cpu()
        assert torch.isfinite(out).all(), S
        e_exact = (out - exact).abs().max().item()
        e_oracle = (out - ref).abs().max().item()
        where = f"S={S} bits={bits}"
        assert e_exact <= 1.5e-3, f"{where}: {e_exact:.2e} from the exact attention"
        known = RAGGED_EXCEPTIONS.get((bits, S))
        if known is None:
            assert e_oracle <= 2e-3, f"{where}: {e_oracle:.2e} from the oracle"
            assert e_oracle <= 1e-2 * ref.abs().max().item(), f"{where}: {e_oracle:.2e} is over 1e-2 of max|ref|"
        else:
            slack = (ref - exact).abs().max().item()
            assert e_oracle <= known["kernel_vs_oracle"] * 1.05, f"{where}: {e_oracle:.2e} from the oracle"
            assert e_exact < slack, f"{where}: the kernel should be nearer the exact result than the oracle is"


def test_batched_serving_shapes_with_jittered_lengths(oracle, attn):
    """The batched-serving configuration (8192 prompt @2-bit + 512 cold @4-bit + 128 hot, lengths jittered
    by +-25 % per sequence): sequences are independent, so the batch is a loop over sequences; a sample of
    them (shortest, longest, six more) is checked against the oracle."""
    from phasekv_b200 import workloads
    shape = workloads.QWEN2_5_7B
    lengths = workloads.jittered_lengths(0, 64, 8192, 512, 128, hot_capacity=192)
    order = sorted(range(64), key=lambda i: lengths[i][0])
    sample = [order[0], order[-1]] + order[5:60:10]
    assert len({lengths[i] for i in sample}) >= 6 and any(lengths[i][0] % 64 for i in sample)
    for i in sample:
        p, c, h = lengths[i]
        segs, hk, hv, q = _pack_tiers(oracle, shape, p, 2, [c], 4, h, seed=workloads.layer_seed(0, 3, i))
        ref = oracle.segments_decode_reference(q[0, :, 0, :], segs, hk, hv, shape.num_q_heads)
        out = attn.fused_phasekv_decode(q[0, :, 0, :].cuda(), make_tiers(segs, hk, hv, hot_len=h), shape.num_q_heads)
        attention_close(out, ref)


def test_long_context_262144_tokens(oracle, attn):
    """The long-context configuration on one GPU: 262144 prompt tokens @2-bit + 1024 cold @4-bit + 128 hot."""
    from phasekv_b200 import workloads
    shape = workloads.QWEN2_5_7B
    segs, hk, hv, q = _pack_tiers(oracle, shape, 262144, 2, [1024], 4, 128, seed=262144)
    ref = oracle.segments_decode_reference(q[0, :, 0, :], segs, hk, hv, shape.num_q_heads)
    out = attn.fused_phasekv_decode(q[0, :, 0, :].cuda(), make_tiers(segs, hk, hv, hot_len=128), shape.num_q_heads)
    attention_close(out, ref)


def test_many_cold_segments_and_hot_capacity(oracle, attn):
    """cold = 8 frozen segments of 64 tokens, hot buffer with spare capacity (only hot_len valid)."""
    from phasekv_b200 import workloads
    shape = workloads.QWEN2_5_7B
    segs, hk, hv, q = _pack_tiers(oracle, shape, 1000, 2, [64] * 8, 4, 77, seed=99)
    ref = oracle.segments_decode_reference(q[0, :, 0, :], segs, hk, hv, shape.num_q_heads)
    cap_k = torch.full((1, 4, 192, 128), float("nan"), dtype=torch.float16)
    cap_v = torch.full((1, 4, 192, 128), float("nan"), dtype=torch.float16)
    cap_k[:, :, :77], cap_v[:, :, :77] = hk, hv
    tiers = make_tiers(segs, cap_k, cap_v, hot_len=77)
    out = attn.fused_phasekv_decode(q[0, :, 0, :].cuda(), tiers, shape.num_q_heads)
    assert torch.isfinite(out).all()
    attention_close(out, ref)
    # more segments than one launch carries inline
    segs2, hk2, hv2, q2 = _pack_tiers(oracle, workloads.QWEN2_0_5B, 300, 2, [32] * 40, 4, 9, seed=98)
    ref2 = oracle.segments_decode_reference(q2[0, :, 0, :], segs2, hk2, hv2, 14)
    out2 = attn.fused_phasekv_decode(q2[0, :, 0, :].cuda(), make_tiers(segs2, hk2, hv2, hot_len=9), 14)
    attention_close(out2, ref2)


def test_split_count_does_not_change_the_result(oracle, attn):
    from phasekv_b200 import workloads
    shape = workloads.QWEN2_5_7B
    segs, hk, hv, q = _pack_tiers(oracle, shape, 5000, 2, [], 4, 0, seed=7)
    kg, vg = remove_batch(to_gpu_packed(segs[0][0])), remove_batch(to_gpu_packed(segs[0][1]))
    outs = []
    for ns in (1, 2, 7, 64, 128, None):
        m, l, acc = attn._kivi_layer_partial(q[0, :, 0, :].cuda(), kg, vg, 28, num_splits=ns)
        outs.append((acc / l[:, None]).cpu())
    for o in outs[1:]:
        # only the float16 rounding of the probabilities depends on where the running maximum sits
        torch.testing.assert_close(o, outs[0], atol=3e-4, rtol=5e-3)


@pytest.mark.parametrize("bits", [2, 4, 8])
def test_per_token_layout_entry_points(oracle, attn, bits):
    """decode_attention_packed[_splitk] and fused_three_tier_decode take K and V both packed along
    head_dim (the layout of the reference's published micro-benchmark)."""
    from phasekv_b200.kernels.tiers import ThreeTierKV
    gen = torch.Generator().manual_seed(1234)
    hkv, hq, hd, S = 4, 28, 128, 1500
    K, V = torch.randn(hkv, S, hd, generator=gen).half(), torch.randn(hkv, S, hd, generator=gen).half()
    Kc, Vc = torch.randn(hkv, 90, hd, generator=gen).half(), torch.randn(hkv, 90, hd, generator=gen).half()
    Kh, Vh = torch.randn(hkv, 33, hd, generator=gen).half(), torch.randn(hkv, 33, hd, generator=gen).half()
    q = torch.randn(hq, hd, generator=gen).half()
    pk, pv = oracle.quantize_pack(K, bits, -1, 32), oracle.quantize_pack(V, bits, -1, 32)
    ck, cv = oracle.quantize_pack(Kc, 4, -1, 32), oracle.quantize_pack(Vc, 4, -1, 32)
    ref1 = oracle.attention_dense(q, oracle.unpack_dequantize(pk), oracle.unpack_dequantize(pv), hq)
    out_single = attn.decode_attention_packed(q.cuda(), to_gpu_packed(pk), to_gpu_packed(pv), hq)
    out_split = attn.decode_attention_packed_splitk(q.cuda(), to_gpu_packed(pk), to_gpu_packed(pv), hq, num_splits=16)
    attention_close(out_single, ref1)
    attention_close(out_split, ref1)
    kv_o = oracle.ThreeTierKV(pk, pv, ck, cv, Kh, Vh)
    k_all, v_all = oracle._dequant_concat(kv_o)
    ref3 = oracle.attention_dense(q, k_all, v_all, hq)
    kv = ThreeTierKV(to_gpu_packed(pk), to_gpu_packed(pv), to_gpu_packed(ck), to_gpu_packed(cv), Kh.cuda(), Vh.cuda())
    attention_close(attn.fused_three_tier_decode(q.cuda(), kv, hq), ref3)
    attention_close(attn.fused_three_tier_decode_single(q.cuda(), kv, hq), ref3)


# (bits, Hq, S) -> the per-token cases beyond the 2e-3 bar, as in RAGGED_EXCEPTIONS: the oracle's own float16
# rounding of the dequantised keys (keys with x8 outlier channels, a 64-token context) puts IT 3.0e-3 from the exact
# attention; the kernel is 6.1e-4 from it.
PER_TOKEN_EXCEPTIONS = {(4, 28, 64): {"kernel_vs_oracle": 3.17e-3, "oracle_vs_exact": 2.97e-3}}


@pytest.mark.parametrize("bits", [2, 4, 8])
@pytest.mark.parametrize("hq,hkv", [(28, 4), (8, 4), (32, 4)])
def test_per_token_layout_sizes_splits_and_outlier_channels(oracle, attn, bits, hq, hkv):
    """The tensor-core kernel of the per-token layout: lengths on and off the 64-token tile grid (odd lengths make
    the scale rows of odd heads 8-byte aligned only), one token, library-sized and forced grids, GQA groups of
    7, 2 and 8, keys with outlier channels (which make the softmax peaky: the hard case for the probabilities).
    Every case is held to the parity bar against the oracle except the enumerated one, and every case to 1.5e-3
    from the exact float64 attention over the codes."""
    gen = torch.Generator().manual_seed(bits * 100 + hq)
    for S, splits in ((1, None), (31, 8), (64, None), (65, 1), (1501, None), (4113, 128), (20000, None), (20000, 3)):
        K, V = torch.randn(hkv, S, 128, generator=gen).half(), torch.randn(hkv, S, 128, generator=gen).half()
        K[:, :, [5, 40, 77, 100]] *= 8
        q = torch.randn(hq, 128, generator=gen).half()
        pk, pv = oracle.quantize_pack(K, bits, -1, 32), oracle.quantize_pack(V, bits, -1, 32)
        ref = oracle.attention_dense(q, oracle.unpack_dequantize(pk), oracle.unpack_dequantize(pv), hq).float()
        exact = _exact_attention(oracle, q, pk, pv, hq)
        out = attn.decode_attention_packed_splitk(q.cuda(), to_gpu_packed(pk), to_gpu_packed(pv), hq,
                                                  num_splits=splits).float().cpu()
        where = f"S={S} bits={bits} Hq={hq}"
        e_exact, e_oracle = (out - exact).abs().max().item(), (out - ref).abs().max().item()
        assert e_exact <= 1.5e-3, f"{where}: {e_exact:.2e} from the exact attention"
        known = PER_TOKEN_EXCEPTIONS.get((bits, hq, S))
        if known is None:
            attention_close(out, ref)
        else:
            assert e_oracle <= known["kernel_vs_oracle"] * 1.05, f"{where}: {e_oracle:.2e} from the oracle"
            assert e_exact < (ref - exact).abs().max().item(), f"{where}: the kernel should be nearer the exact result"


def test_per_token_and_kivi_segments_in_one_call_use_the_general_kernel(oracle, attn):
    """No caller of the reference mixes the two layouts in one attention; the C entry point still takes such a list
    (the per-token segments are then served by the general kernel) and the result is the same attention."""
    import ctypes

    from phasekv_b200 import _native as nv
    gen = torch.Generator().manual_seed(77)
    hkv, hq, hd = 4, 28, 128
    K1, V1 = torch.randn(hkv, 700, hd, generator=gen).half(), torch.randn(hkv, 700, hd, generator=gen).half()
    K2, V2 = torch.randn(hkv, 300, hd, generator=gen).half(), torch.randn(hkv, 300, hd, generator=gen).half()
    q = torch.randn(hq, hd, generator=gen).half()
    k1, v1 = oracle.quantize_pack(K1, 2, -2, 32), oracle.quantize_pack(V1, 2, -1, 32)      # KIVI
    k2, v2 = oracle.quantize_pack(K2, 4, -1, 32), oracle.quantize_pack(V2, 4, -1, 32)      # per token
    k_all = torch.cat([oracle.unpack_dequantize(k1), oracle.unpack_dequantize(k2)], dim=1)
    v_all = torch.cat([oracle.unpack_dequantize(v1), oracle.unpack_dequantize(v2)], dim=1)
    ref = oracle.attention_dense(q, k_all, v_all, hq)
    from phasekv_b200.kernels import attention_cuda
    s1, keep1 = attention_cuda._packed_segment(to_gpu_packed(k1), to_gpu_packed(v1), None)
    s2, keep2 = attention_cuda._packed_segment(to_gpu_packed(k2), to_gpu_packed(v2), None)
    assert (s1.kind, s2.kind) == (nv.PKV_SEG_KIVI, nv.PKV_SEG_PER_TOKEN)
    out, _ = attention_cuda._run_decode(q.cuda(), [s1, s2], [keep1, keep2], hq, hkv, True, False)
    attention_close(out, ref)


def test_partials_merge_like_the_reference_algebra(oracle, attn):
    """_fp16_layer_partial + _kivi_layer_partial + _merge_partials == one fused call; _reduce_splits
    accepts the reference's [Hq, splits] layout."""
    from phasekv_b200 import workloads
    shape = workloads.QWEN2_0_5B
    segs, hk, hv, q = _pack_tiers(oracle, shape, 700, 2, [100], 4, 50, seed=5)
    qg = q[0, :, 0, :].cuda()
    parts = [attn._kivi_layer_partial(qg, remove_batch(to_gpu_packed(k)), remove_batch(to_gpu_packed(v)), 14)
             for k, v in segs]
    parts.append(attn._fp16_layer_partial(qg, hk[0].cuda(), hv[0].cuda(), 14))
    merged = attn._merge_partials(parts)
    fused = attn.fused_phasekv_decode(qg, make_tiers(segs, hk, hv, hot_len=50), 14)
    torch.testing.assert_close(merged.float(), fused.float(), atol=1e-3, rtol=1e-3)
    attention_close(merged, oracle.segments_decode_reference(q[0, :, 0, :], segs, hk, hv, 14))
    pm = torch.stack([p[0] for p in parts], dim=1)
    pl = torch.stack([p[1] for p in parts], dim=1)
    pacc = torch.stack([p[2] for p in parts], dim=1)
    m, l, acc = attn._reduce_splits(pm, pl, pacc)
    torch.testing.assert_close((acc / l[:, None]).half().float(), merged.float(), atol=1e-3, rtol=1e-3)


def test_argument_errors(oracle, attn):
    from phasekv_b200 import workloads
    segs, hk, hv, q = _pack_tiers(oracle, workloads.QWEN2_0_5B, 64, 2, [], 4, 0, seed=1)
    k, v = remove_batch(to_gpu_packed(segs[0][0])), remove_batch(to_gpu_packed(segs[0][1]))
    qg = q[0, :, 0, :].cuda()
    with pytest.raises(ValueError):
        attn._kivi_layer_partial(qg.float(), k, v, 14)          # query must be float16
    with pytest.raises(ValueError):
        attn._kivi_layer_partial(qg[:13], k, v, 13)             # 13 heads over 2 KV heads
    with pytest.raises(ValueError):
        attn._kivi_layer_partial(qg, v, v, 14)                  # K packed along the wrong axis
    with pytest.raises(ValueError):
        attn._kivi_layer_partial(qg, k, v, 14, num_splits=0)
    with pytest.raises(ValueError):
        attn._kivi_layer_partial(qg, k, v, 14, block_n=3)
    batched = to_gpu_packed(segs[0][0])
    batched.orig_shape = (2,) + tuple(batched.orig_shape[1:])
    from phasekv_b200.kernels.tiers import LayerTiers, PackedKVSegment
    with pytest.raises(ValueError):
        attn.fused_phasekv_decode(qg, LayerTiers(PackedKVSegment(batched, batched)), 14)


@pytest.mark.parametrize("bits", [2, 4, 8])
def test_padded_key_rows_take_any_length(oracle, attn, bits):
    """Keys packed on the GPU come with rows padded to whole 64-token tiles (views with a row stride), which
    lets segments of any length stream through the 16-byte copy path.  Codes, scales and zeros seen through
    the views are the oracle's bit for bit, and the attention over them meets the same bars as the dense
    layout does."""
    from phasekv_b200 import workloads
    from phasekv_b200.kernels import packing
    from phasekv_b200.kernels.tiers import LayerTiers, PackedKVSegment
    from tests.util import assert_packed_equal
    shape = workloads.QWEN2_5_7B
    over_the_bar = []
    for S in (1, 31, 65, 1000, 4097, 8193):
        segs, hk, hv, q = _pack_tiers(oracle, shape, S, bits, [], 4, 0, seed=77 * bits + S)
        (pk, pv), _, _, _ = workloads.three_tier_dense(77 * bits + S, shape, S, 0, 0)
        key = packing.quantize_pack(pk.cuda(), bits, -2, 32)
        value = packing.quantize_pack(pv.cuda(), bits, -1, 32)
        assert_packed_equal(key, segs[0][0], f"K S={S}")
        assert_packed_equal(value, segs[0][1], f"V S={S}")
        if S >= 32:
            assert key.packed.stride(2) % 16 == 0 and key.packed.stride(2) * (8 // bits) % 64 == 0
            assert key.scale.stride(2) % 8 == 0 and key.scale.stride(2) == key.mins.stride(2)
        q2 = q[0, :, 0, :]
        ref = oracle.segments_decode_reference(q2, segs, None, None, shape.num_q_heads).float()
        exact = _exact_attention(oracle, q2, segs[0][0], segs[0][1], shape.num_q_heads)
        tiers = LayerTiers(prompt=PackedKVSegment(key, value))
        out = attn.fused_phasekv_decode(q2.cuda(), tiers, shape.num_q_heads).float().cpu()
        dense = attn.fused_phasekv_decode(q2.cuda(), make_tiers(segs), shape.num_q_heads).float().cpu()
        assert torch.isfinite(out).all(), S
        e_exact, e_oracle = (out - exact).abs().max().item(), (out - ref).abs().max().item()
        assert e_exact <= 1.5e-3, f"S={S} bits={bits}: {e_exact:.2e} from the exact attention"
        if e_oracle > 2e-3 or e_oracle > 1e-2 * ref.abs().max().item():
            over_the_bar.append((S, bits, e_oracle, (ref - exact).abs().max().item()))
        assert (out - dense).abs().max().item() <= 1e-3, f"S={S} bits={bits}: padded and dense rows disagree"
    # the parity bar itself (2e-3 and 1e-2 of max|ref| against the oracle), no exception among these cases
    assert not over_the_bar, f"(S, bits, |out - oracle|, |oracle - exact|): {over_the_bar}"
