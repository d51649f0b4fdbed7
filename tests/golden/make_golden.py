"""Regenerates the golden fixtures in this directory from the reference's own Python.

Run where a checkout of the reference is available (it is NOT needed to run the tests):

    python tests/golden/make_golden.py --reference /path/to/PhaseKV

It imports ``src/phasekv/kernels/{packing,reference,launch_config}.py`` by file path
(not ``import src.phasekv``, whose ``__init__`` pulls in transformers), runs them on
CPU, and stores inputs and outputs as small ``.npz``/``.json`` files:

  pack_cases.npz      quantize_pack / unpack_dequantize / pack_low_bits / unpack_low_bits
  attention_c1.npz    fused_decode_attention_reference on the Qwen2-0.5B plumbing case
                      (prompt 1024 @2-bit gsK 32 / gsV 64, cold 128 @4-bit, hot 64)
  attention_small.npz ragged multi-tier cases on small shapes
  cold_select.npz     value-norm top-k + pack of an aged hot batch
                      (the five tensor lines of phasekv_cache.py:328-334)
  planner.json        plan_kivi_decode over a grid of arguments
"""
from __future__ import annotations

import argparse
import importlib.util
import json
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.abspath(os.path.join(HERE, "..", "..")))

from phasekv_b200 import workloads  # noqa: E402


def load_reference(root: str):
    kdir = os.path.join(root, "src", "phasekv", "kernels")
    pkg = types.ModuleType("refkernels")
    pkg.__path__ = [kdir]
    sys.modules["refkernels"] = pkg
    mods = {}
    for name in ("packing", "launch_config", "reference"):
        spec = importlib.util.spec_from_file_location(f"refkernels.{name}", os.path.join(kdir, f"{name}.py"))
        mod = importlib.util.module_from_spec(spec)
        sys.modules[f"refkernels.{name}"] = mod
        spec.loader.exec_module(mod)
        mods[name] = mod
    return mods["packing"], mods["reference"], mods["launch_config"]


def f16(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().numpy().view(np.uint16)


def store_packed(out: dict, prefix: str, pt) -> None:
    out[f"{prefix}.packed"] = pt.packed.numpy()
    out[f"{prefix}.scale"] = f16(pt.scale)
    out[f"{prefix}.mins"] = f16(pt.mins)
    out[f"{prefix}.meta"] = np.array([pt.bits, pt.axis, pt.group_size, pt.axis_len, *pt.orig_shape],
                                     dtype=np.int64)


PACK_CASES = [
    # (shape, axis, bits, group_size, seed, kind)
    ((1, 2, 200, 64), -2, 2, 32, 1, "outlier"),
    ((1, 2, 200, 64), -1, 2, 64, 2, "randn"),
    ((1, 2, 200, 64), -2, 4, 32, 3, "outlier"),
    ((1, 2, 200, 64), -1, 4, 32, 4, "randn"),
    ((1, 2, 96, 128), -2, 8, 32, 5, "outlier"),
    ((1, 2, 96, 128), -1, 8, 32, 6, "randn"),
    ((1, 4, 129, 128), -2, 2, 32, 7, "outlier"),
    ((1, 4, 129, 128), -1, 2, 32, 8, "randn"),
    ((2, 3, 33, 8), -2, 4, 4, 9, "randn"),
    ((2, 3, 33, 8), -1, 2, 4, 10, "randn"),
    ((1, 1, 1, 8), -2, 2, 32, 11, "randn"),
    ((1, 1, 7, 256), -2, 2, 32, 12, "randn"),
    ((1, 1, 7, 256), -1, 4, 32, 13, "randn"),
    ((2, 31, 64), 1, 2, 32, 14, "randn"),
    ((2, 31, 64), 2, 8, 16, 15, "randn"),
    ((3, 50), 0, 4, 2, 16, "randn"),
    ((1, 2, 40, 64), -2, 2, 32, 17, "const"),
    ((1, 2, 40, 64), -1, 4, 32, 18, "halfgrid"),
    ((1, 2, 127, 64), -2, 2, 0, 19, "randn"),
]


def make_pack_input(shape, seed, kind):
    gen = torch.Generator().manual_seed(seed)
    if kind == "const":
        x = torch.full(shape, 0.75).half()
        x[..., 0] = 3.0
        return x
    if kind == "halfgrid":
        # values on a coarse grid: many quotients land exactly on .5, which makes
        # round-half-even observable
        return (torch.randint(-12, 13, shape, generator=gen).float() / 8.0).half()
    x = torch.randn(shape, generator=gen).half()
    if kind == "outlier" and shape[-1] in workloads.OUTLIER_CHANNELS:
        for c in workloads.OUTLIER_CHANNELS[shape[-1]]:
            x[..., c] = (x[..., c].float() * workloads.OUTLIER_GAIN).half()
    return x


def gen_pack(packing, out_dir):
    out = {}
    for i, (shape, axis, bits, gs, seed, kind) in enumerate(PACK_CASES):
        x = make_pack_input(shape, seed, kind)
        pt = packing.quantize_pack(x, bits, axis, gs)
        deq = packing.unpack_dequantize(pt)
        codes = packing.unpack_low_bits(pt.packed, bits, pt.axis_len)
        repacked = packing.pack_low_bits(codes, bits)
        assert torch.equal(repacked, pt.packed)
        out[f"c{i}.x"] = f16(x)
        out[f"c{i}.args"] = np.array([axis, bits, gs], dtype=np.int64)
        store_packed(out, f"c{i}.pt", pt)
        out[f"c{i}.deq"] = f16(deq)
        out[f"c{i}.codes"] = codes.numpy()
    out["n_cases"] = np.array([len(PACK_CASES)], dtype=np.int64)
    np.savez_compressed(os.path.join(out_dir, "pack_cases.npz"), **out)


def gen_attention_c1(packing, reference, out_dir):
    shape = workloads.QWEN2_0_5B
    (pk, pv), (ck, cv), (hk, hv), q = workloads.three_tier_dense(0, shape, 1024, 128, 64)
    kv = reference.ThreeTierKV(
        prompt_k=packing.quantize_pack(pk, 2, -2, 32), prompt_v=packing.quantize_pack(pv, 2, -1, 64),
        cold_k=packing.quantize_pack(ck, 4, -2, 32), cold_v=packing.quantize_pack(cv, 4, -1, 32),
        hot_k=hk, hot_v=hv)
    o = reference.fused_decode_attention_reference(q, kv, shape.num_q_heads)
    out = {"q": f16(q), "hot_k": f16(hk), "hot_v": f16(hv), "out": f16(o)}
    for name in ("prompt_k", "prompt_v", "cold_k", "cold_v"):
        store_packed(out, name, getattr(kv, name))
    np.savez_compressed(os.path.join(out_dir, "attention_c1.npz"), **out)


SMALL_ATTN = [
    # (Hq, Hkv, hd, prompt, pbits, cold, cbits, hot, gsK, gsV, seed)
    (4, 2, 8, 1, 2, 0, 4, 0, 32, 32, 21),
    (4, 2, 64, 10, 8, 0, 8, 3, 32, 32, 22),
    (12, 2, 128, 127, 4, 33, 4, 5, 32, 32, 23),
    (12, 2, 128, 513, 2, 64, 4, 17, 32, 32, 24),
    (4, 2, 256, 129, 8, 31, 4, 0, 32, 32, 25),
    (28, 4, 128, 300, 2, 96, 4, 40, 32, 32, 26),
    (14, 2, 64, 0, 2, 70, 2, 9, 32, 64, 27),
]


def gen_attention_small(packing, reference, out_dir):
    out = {}
    for i, (hq, hkv, hd, p, pb, c, cb, h, gsk, gsv, seed) in enumerate(SMALL_ATTN):
        shape = workloads.Shape("t", hq, hkv, hd, 1)
        (pk, pv), (ck, cv), (hk, hv), q = workloads.three_tier_dense(seed, shape, p, c, h)
        kv = reference.ThreeTierKV()
        if p:
            kv.prompt_k = packing.quantize_pack(pk, pb, -2, gsk)
            kv.prompt_v = packing.quantize_pack(pv, pb, -1, gsv)
            store_packed(out, f"a{i}.prompt_k", kv.prompt_k)
            store_packed(out, f"a{i}.prompt_v", kv.prompt_v)
        if c:
            kv.cold_k = packing.quantize_pack(ck, cb, -2, gsk)
            kv.cold_v = packing.quantize_pack(cv, cb, -1, gsv)
            store_packed(out, f"a{i}.cold_k", kv.cold_k)
            store_packed(out, f"a{i}.cold_v", kv.cold_v)
        if h:
            kv.hot_k, kv.hot_v = hk, hv
            out[f"a{i}.hot_k"] = f16(hk)
            out[f"a{i}.hot_v"] = f16(hv)
        o = reference.fused_decode_attention_reference(q, kv, hq)
        out[f"a{i}.q"] = f16(q)
        out[f"a{i}.out"] = f16(o)
        out[f"a{i}.dims"] = np.array([hq, hkv, hd], dtype=np.int64)
    out["n_cases"] = np.array([len(SMALL_ATTN)], dtype=np.int64)
    np.savez_compressed(os.path.join(out_dir, "attention_small.npz"), **out)


COLD_CASES = [
    # (B, Hkv, hot_len, hd, recent_window, keep_ratio, bits, gs, seed)
    (1, 4, 192, 128, 128, 0.5, 4, 32, 31),   # aged 64 -> keep 32 (the cold-batch config)
    (1, 2, 4, 8, 2, 0.5, 4, 4, 32),          # aged 2 -> keep 1
    (2, 2, 50, 64, 7, 0.3, 2, 32, 33),       # aged 43 -> keep round(12.9) = 13
    (1, 2, 40, 64, 8, 1.0, 8, 32, 34),       # keep everything: no selection
    (1, 3, 37, 64, 32, 0.5, 4, 32, 35),      # aged 5 -> round(2.5) = 2 (banker's rounding)
]


def gen_cold(packing, out_dir):
    out = {}
    for i, (b, hkv, hot_len, hd, window, ratio, bits, gs, seed) in enumerate(COLD_CASES):
        gen = torch.Generator().manual_seed(seed)
        hot_k, hot_v = workloads.make_kv(gen, hkv, hot_len, hd, batch=b)
        # phasekv_cache.py:324-334
        aged = hot_len - window
        key, value = hot_k[:, :, :aged, :], hot_v[:, :, :aged, :]
        keep_count = max(1, round(ratio * aged))
        indices = None
        if keep_count < aged:
            importance = torch.linalg.vector_norm(value.float(), dim=-1)
            indices = importance.topk(keep_count, dim=-1).indices.sort(dim=-1).values
            gi = indices.unsqueeze(-1).expand(*indices.shape, hd)
            key, value = key.gather(2, gi), value.gather(2, gi)
        kpt = packing.quantize_pack(key, bits, -2, gs)
        vpt = packing.quantize_pack(value, bits, -1, gs)
        out[f"k{i}.hot_k"] = f16(hot_k)
        out[f"k{i}.hot_v"] = f16(hot_v)
        out[f"k{i}.args"] = np.array([window, keep_count, aged, bits, gs], dtype=np.int64)
        out[f"k{i}.ratio"] = np.array([ratio], dtype=np.float64)
        out[f"k{i}.indices"] = (indices.numpy() if indices is not None
                                else np.zeros((0,), dtype=np.int64))
        store_packed(out, f"k{i}.key", kpt)
        store_packed(out, f"k{i}.value", vpt)
    out["n_cases"] = np.array([len(COLD_CASES)], dtype=np.int64)
    np.savez_compressed(os.path.join(out_dir, "cold_select.npz"), **out)


FAKE_QUANT_CASES = [
    # shape, axis, bits, group, dtype, seed, kind
    ((1, 2, 20, 8), -2, 2, 4, "f16", 31, "randn"),
    ((1, 2, 20, 8), -1, 2, 4, "f16", 32, "randn"),
    ((1, 4, 100, 128), -2, 2, 32, "f16", 33, "outlier"),
    ((1, 4, 100, 128), -1, 4, 32, "f16", 34, "outlier"),
    ((2, 2, 77, 64), -2, 3, 32, "bf16", 35, "randn"),
    ((2, 2, 77, 64), -1, 3, 32, "bf16", 36, "randn"),
    ((1, 2, 33, 64), -2, 8, 32, "f16", 37, "halfgrid"),
    ((1, 2, 64, 64), -1, 8, 64, "f32", 38, "randn"),
    ((1, 1, 5, 16), -2, 1, 32, "f16", 39, "randn"),
    ((1, 2, 40, 32), -2, 12, 0, "f32", 40, "randn"),
    ((1, 2, 16, 32), -1, 4, 8, "f16", 41, "const"),
]


def gen_fake_quant(root, out_dir):
    """Stage-A fake quantisation: the reference's quant.py executed as it is (it only needs torch)."""
    spec = importlib.util.spec_from_file_location("refquant", os.path.join(root, "src", "phasekv", "quant.py"))
    quant = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(quant)
    dt = {"f16": torch.float16, "bf16": torch.bfloat16, "f32": torch.float32}
    out = {}
    for i, (shape, axis, bits, gs, dtype, seed, kind) in enumerate(FAKE_QUANT_CASES):
        x = make_pack_input(shape, seed, kind).float()
        if dtype == "f32":
            x = x + torch.randn(shape, generator=torch.Generator().manual_seed(seed + 1000)) * 1e-3
        x = x.to(dt[dtype])
        y = quant._grouped_affine_quant_dequant(x, bits, axis, gs)
        assert y.dtype == x.dtype and y.shape == x.shape
        out[f"c{i}.x"] = x.float().numpy()
        out[f"c{i}.y"] = y.float().numpy()
        out[f"c{i}.args"] = np.array([axis, bits, gs, ["f16", "bf16", "f32"].index(dtype)], dtype=np.int64)
    # the two public wrappers on a cache-shaped tensor
    k = make_pack_input((1, 4, 96, 128), 50, "outlier")
    out["key.x"], out["key.y"] = f16(k), f16(quant.quantize_key(k, 2, 32))
    out["value.x"], out["value.y"] = f16(k), f16(quant.quantize_value(k, 4, 32))
    out["n_cases"] = np.array([len(FAKE_QUANT_CASES)], dtype=np.int64)
    out["bytes"] = np.array([quant.quantized_tier_bytes(1000, 28, 4, 128, 2, 2, 32, 1),
                             quant.quantized_tier_bytes(77, 2, 2, 64, 4, 16, 0, 3),
                             quant.fp16_tier_bytes(128, 28, 4, 128, 2),
                             *quant.kv_group_counts(1000, 128, 32), *quant.kv_group_counts(5, 8, 0)], dtype=np.int64)
    np.savez_compressed(os.path.join(out_dir, "fake_quant.npz"), **out)


PROMPT_SELECT_CASES = [
    # prompt_len, Hq, Hkv, layers, batch, keep_ratio, sink, obs_window, pool_kernel, pooling, seed
    (20, 4, 2, 2, 1, 0.5, 2, 4, 3, "maxpool", 61),
    (64, 14, 2, 1, 2, 0.25, 4, 8, 7, "maxpool", 62),
    (50, 8, 8, 1, 1, 0.6, 0, 16, 5, "avgpool", 63),
    (12, 4, 4, 1, 1, 1.0, 4, 32, 7, "maxpool", 64),
    (9, 2, 1, 1, 1, 0.1, 4, 2, 1, "maxpool", 65),
    (128, 28, 4, 1, 1, 0.3, 4, 32, 7, "maxpool", 66),
]


def gen_prompt_select(root, out_dir):
    """Stage-A prompt selection: the reference's prompt_tier.select_prompt_indices on seeded causal attention."""
    pkg = types.ModuleType("refphasekv")
    pkg.__path__ = [os.path.join(root, "src", "phasekv")]
    sys.modules["refphasekv"] = pkg
    mods = {}
    for name in ("quant", "hetero_cache", "prompt_tier"):
        spec = importlib.util.spec_from_file_location(f"refphasekv.{name}", os.path.join(root, "src", "phasekv", f"{name}.py"))
        mod = importlib.util.module_from_spec(spec)
        sys.modules[f"refphasekv.{name}"] = mod
        spec.loader.exec_module(mod)
        mods[name] = mod
    out = {}
    for i, (plen, hq, hkv, layers, batch, ratio, sink, obs, kernel, pooling, seed) in enumerate(PROMPT_SELECT_CASES):
        gen = torch.Generator().manual_seed(seed)
        cfg = types.SimpleNamespace(num_key_value_heads=hkv, num_attention_heads=hq)
        atts = []
        for _ in range(layers):
            logits = torch.randn(batch, hq, plen, plen, generator=gen) * 2.0
            mask = torch.ones(plen, plen, dtype=torch.bool).tril()
            atts.append(torch.softmax(logits.masked_fill(~mask, float("-inf")), dim=-1))
        keep = mods["prompt_tier"].select_prompt_indices(
            atts, prompt_len=plen, model_config=cfg, prefill_keep_ratio=ratio, sink_tokens=sink, obs_window=obs,
            pool_kernel=kernel, pooling=pooling)
        out[f"c{i}.att"] = torch.stack(atts).numpy()
        out[f"c{i}.keep"] = torch.stack(keep).numpy()
        out[f"c{i}.args"] = np.array([plen, hq, hkv, layers, batch, sink, obs, kernel, int(pooling == "avgpool")], dtype=np.int64)
        out[f"c{i}.ratio"] = np.array([ratio])
    out["n_cases"] = np.array([len(PROMPT_SELECT_CASES)], dtype=np.int64)
    np.savez_compressed(os.path.join(out_dir, "prompt_select.npz"), **out)


def gen_planner(launch_config, out_dir):
    rows = []
    for length in (1, 7, 31, 127, 128, 129, 511, 512, 4096, 8193, 28672, 32768, 131072, 262144):
        for heads, dim, sms in ((12, 128, 46), (4, 8, 1), (32, 256, 132), (28, 128, 148), (14, 64, 148)):
            for kw in ({}, {"num_splits": 8, "block_n": 64, "num_warps": 4}, {"num_splits": 3},
                       {"block_n": 16}, {"num_warps": 8}, {"num_splits": 100}):
                c = launch_config.plan_kivi_decode(length, heads, dim, sms, **kw)
                rows.append({"args": [length, heads, dim, sms], "kwargs": kw,
                             "plan": [c.num_splits, c.split_len, c.block_n, c.num_warps]})
    with open(os.path.join(out_dir, "planner.json"), "w") as f:
        json.dump(rows, f, separators=(",", ":"))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of a PhaseKV checkout")
    ap.add_argument("--out", default=HERE)
    args = ap.parse_args()
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    packing, reference, launch_config = load_reference(args.reference)
    gen_pack(packing, args.out)
    gen_attention_c1(packing, reference, args.out)
    gen_attention_small(packing, reference, args.out)
    gen_cold(packing, args.out)
    gen_planner(launch_config, args.out)
    gen_fake_quant(args.reference, args.out)
    gen_prompt_select(args.reference, args.out)
    for name in sorted(os.listdir(args.out)):
        if name.endswith((".npz", ".json")):
            print(name, os.path.getsize(os.path.join(args.out, name)))


if __name__ == "__main__":
    main()
