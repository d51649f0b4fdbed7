"""Pins the CPU oracle (oracle/pkv_oracle.c) against fixtures produced by the reference's
own packing.py / reference.py / phasekv_cache.py arithmetic (tests/golden/make_golden.py)."""
import numpy as np
import torch

from conftest import attention_close, from_f16, load_packed


def test_quantize_pack_bit_exact(golden, oracle):
    z = golden("pack_cases.npz")
    for i in range(int(z["n_cases"][0])):
        x = from_f16(z[f"c{i}.x"])
        axis, bits, gs = (int(v) for v in z[f"c{i}.args"])
        ref = load_packed(z, f"c{i}.pt")
        got = oracle.quantize_pack(x, bits, axis, gs)
        assert (got.bits, got.axis, got.group_size, got.axis_len, got.orig_shape) == \
            (ref.bits, ref.axis, ref.group_size, ref.axis_len, ref.orig_shape), i
        assert torch.equal(got.packed, ref.packed), f"codes differ in case {i}"
        assert torch.equal(got.scale.view(torch.int16), ref.scale.view(torch.int16)), f"scale, case {i}"
        assert torch.equal(got.mins.view(torch.int16), ref.mins.view(torch.int16)), f"mins, case {i}"


def test_unpack_dequantize_and_low_bits_bit_exact(golden, oracle):
    z = golden("pack_cases.npz")
    for i in range(int(z["n_cases"][0])):
        ref = load_packed(z, f"c{i}.pt")
        deq = oracle.unpack_dequantize(ref)
        assert torch.equal(deq.view(torch.int16), from_f16(z[f"c{i}.deq"]).view(torch.int16)), i
        codes = oracle.unpack_low_bits(ref.packed, ref.bits, ref.axis_len)
        assert torch.equal(codes, torch.from_numpy(z[f"c{i}.codes"])), i
        assert torch.equal(oracle.pack_low_bits(codes, ref.bits), ref.packed), i


def test_attention_c1_matches_reference(golden, oracle):
    z = golden("attention_c1.npz")
    kv = oracle.ThreeTierKV(
        prompt_k=load_packed(z, "prompt_k"), prompt_v=load_packed(z, "prompt_v"),
        cold_k=load_packed(z, "cold_k"), cold_v=load_packed(z, "cold_v"),
        hot_k=from_f16(z["hot_k"]), hot_v=from_f16(z["hot_v"]))
    q = from_f16(z["q"])
    out = oracle.fused_decode_attention_reference(q, kv, q.shape[1])
    ref = from_f16(z["out"])
    assert out.shape == ref.shape == (1, 14, 1, 64)
    # the oracle and the reference differ only by float32 summation order
    assert attention_close(out, ref, atol=2e-4, rel=1e-3) < 2e-4


def test_attention_small_cases_match_reference(golden, oracle):
    z = golden("attention_small.npz")
    for i in range(int(z["n_cases"][0])):
        kv = oracle.ThreeTierKV()
        if f"a{i}.prompt_k.meta" in z:
            kv.prompt_k, kv.prompt_v = load_packed(z, f"a{i}.prompt_k"), load_packed(z, f"a{i}.prompt_v")
        if f"a{i}.cold_k.meta" in z:
            kv.cold_k, kv.cold_v = load_packed(z, f"a{i}.cold_k"), load_packed(z, f"a{i}.cold_v")
        if f"a{i}.hot_k" in z:
            kv.hot_k, kv.hot_v = from_f16(z[f"a{i}.hot_k"]), from_f16(z[f"a{i}.hot_v"])
        q = from_f16(z[f"a{i}.q"])
        out = oracle.fused_decode_attention_reference(q, kv, q.shape[1])
        attention_close(out, from_f16(z[f"a{i}.out"]), atol=5e-4, rel=2e-3)


def test_cold_selection_matches_reference(golden, oracle):
    z = golden("cold_select.npz")
    for i in range(int(z["n_cases"][0])):
        window, keep, aged, bits, gs = (int(v) for v in z[f"k{i}.args"])
        hot_k, hot_v = from_f16(z[f"k{i}.hot_k"]), from_f16(z[f"k{i}.hot_v"])
        key, value = hot_k[:, :, :aged, :], hot_v[:, :, :aged, :]
        ref_idx = torch.from_numpy(z[f"k{i}.indices"])
        if keep < aged:
            idx, gap = oracle.value_norm_topk(value, keep)
            assert torch.equal(idx, ref_idx), f"case {i}: selection differs (min gap {gap.min():.2e})"
            gi = idx.unsqueeze(-1).expand(*idx.shape, key.shape[-1])
            key, value = key.gather(2, gi), value.gather(2, gi)
        else:
            assert ref_idx.numel() == 0
        for name, t, axis in (("key", key, -2), ("value", value, -1)):
            ref = load_packed(z, f"k{i}.{name}")
            got = oracle.quantize_pack(t.contiguous(), bits, axis, gs)
            assert torch.equal(got.packed, ref.packed), (i, name)
            assert torch.equal(got.scale.view(torch.int16), ref.scale.view(torch.int16)), (i, name)
            assert torch.equal(got.mins.view(torch.int16), ref.mins.view(torch.int16)), (i, name)


def test_known_answer_cold_selection(oracle):
    """tests/test_phasekv_cache.py:155-182 of the reference: V strengths (9,1) then (1,9) over two
    heads, keep 1 of 2 -> head 0 keeps token 0, head 1 keeps token 1, and cold V dequantises to 9."""
    toks = []
    for step, strengths in enumerate(((9, 1), (1, 9))):
        value = torch.tensor(strengths, dtype=torch.float16).view(1, 2, 1, 1).expand(1, 2, 1, 8)
        toks.append((torch.full_like(value, step + 1), value))
    key = torch.cat([t[0] for t in toks], dim=2).contiguous()
    value = torch.cat([t[1] for t in toks], dim=2).contiguous()
    idx, _ = oracle.value_norm_topk(value, 1)
    assert idx[0, :, 0].tolist() == [0, 1]
    gi = idx.unsqueeze(-1).expand(1, 2, 1, 8)
    ck = oracle.quantize_pack(key.gather(2, gi).contiguous(), 4, -2, 4)
    cv = oracle.quantize_pack(value.gather(2, gi).contiguous(), 4, -1, 4)
    cold_key = oracle.unpack_dequantize(ck)
    assert torch.equal(cold_key[0, :, 0, 0], torch.tensor([1., 2.], dtype=torch.float16))
    assert torch.equal(oracle.unpack_dequantize(cv), torch.full_like(cold_key, 9))
