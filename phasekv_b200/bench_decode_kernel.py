"""Kernel-level decode-attention micro-benchmarks with the row keys of the reference's scripts.

``python -m phasekv_b200.bench_decode_kernel per-token`` follows ``scripts/bench_decode_kernel.py:66-118`` of the
reference: both K and V quantised along head_dim ("per-token layout"), one layer, one query step; FP16 SDPA over
GQA-expanded K/V, the single-pass entry point and the split-K entry point (best of a grid of ``num_splits``),
median of ``--iters`` CUDA-event timings after ``--warmup`` calls, errors against dequantise-then-attend in float32.
Rows carry the same keys (``seq_len, bits, sdpa_fp16_ms, packed_single_ms, packed_splitk_ms, best_num_splits,
speedup_*, kv_read_bytes_*, kv_bytes_saving_pct, max_abs_err_*``).

``python -m phasekv_b200.bench_decode_kernel kivi-launch`` follows ``scripts/bench_phasekv_launch.py:40-67``: the
production KIVI layout, 4-bit, Hq 12 / Hkv 2 / hd 128, lengths 128 / 512 / 8192 / 28672, CUDA-graph timing of
``_kivi_layer_partial`` with the old fixed launch parameters and with the automatic plan (``num_splits`` is
honoured as given; ``block_n`` and ``num_warps`` are Triton notions and only validated).

Inputs are ``torch.randn`` with the scripts' seeds and shapes; results go to stdout as JSON and, with ``--out``, to
a file.
"""
from __future__ import annotations

import argparse
import json
from dataclasses import asdict

import torch
import torch.nn.functional as F

from .kernels import packing as pk
from .kernels.attention_cuda import _kivi_layer_partial, decode_attention_packed, decode_attention_packed_splitk
from .kernels.launch_config import plan_kivi_decode


def _median_ms(fn, warmup: int, iters: int) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    times = []
    for _ in range(iters):
        start.record()
        fn()
        end.record()
        torch.cuda.synchronize()
        times.append(start.elapsed_time(end))
    times.sort()
    return times[len(times) // 2]


def _graph_ms(fn, reps: int = 100) -> float:
    """Mean milliseconds of fn() replayed from a CUDA graph (no Python launch overhead)."""
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        for _ in range(3):
            fn()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            fn()
        for _ in range(5):
            graph.replay()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(reps):
            graph.replay()
        end.record()
        end.synchronize()
    torch.cuda.current_stream().wait_stream(stream)
    return start.elapsed_time(end) / reps


def _dequantise_then_attend(q, key, value, group, hd):
    k = pk.unpack_dequantize(key).repeat_interleave(group, 0).float()
    v = pk.unpack_dequantize(value).repeat_interleave(group, 0).float()
    scores = (q.float().unsqueeze(1) @ k.transpose(-1, -2)).squeeze(1) * (1.0 / hd ** 0.5)
    return (scores.softmax(-1).unsqueeze(1) @ v).squeeze(1).half()


def per_token_rows(hkv, hq, hd, gs, seqs, bits_list, splits_grid, warmup, iters, seed):
    torch.manual_seed(seed)
    group = hq // hkv
    rows = []
    for length in seqs:
        k = torch.randn(hkv, length, hd, dtype=torch.float16, device="cuda")
        v = torch.randn(hkv, length, hd, dtype=torch.float16, device="cuda")
        q = torch.randn(hq, hd, dtype=torch.float16, device="cuda")
        qb = q.view(1, hq, 1, hd)
        kb = k.repeat_interleave(group, 0).view(1, hq, length, hd)
        vb = v.repeat_interleave(group, 0).view(1, hq, length, hd)
        t_sdpa = _median_ms(lambda: F.scaled_dot_product_attention(qb, kb, vb), warmup, iters)
        fp16_bytes = 2 * hkv * length * hd * 2
        for bits in bits_list:
            key, value = pk.quantize_pack(k, bits, -1, gs), pk.quantize_pack(v, bits, -1, gs)
            want = _dequantise_then_attend(q, key, value, group, hd).float()
            err_single = (decode_attention_packed(q, key, value, hq).float() - want).abs().max().item()
            t_single = _median_ms(lambda: decode_attention_packed(q, key, value, hq), warmup, iters)
            best_t, best_ns, best_err = float("inf"), 0, 0.0
            for ns in splits_grid:
                out = decode_attention_packed_splitk(q, key, value, hq, num_splits=ns)
                t = _median_ms(lambda: decode_attention_packed_splitk(q, key, value, hq, num_splits=ns), warmup, iters)
                if t < best_t:
                    best_t, best_ns, best_err = t, ns, (out.float() - want).abs().max().item()
            graph_ms = _graph_ms(lambda: decode_attention_packed_splitk(q, key, value, hq, num_splits=best_ns))
            auto_ms = _graph_ms(lambda: decode_attention_packed_splitk(q, key, value, hq, num_splits=None))
            packed_bytes = key.nbytes + value.nbytes
            rows.append({
                "seq_len": length, "bits": bits, "num_kv_heads": hkv, "num_q_heads": hq, "head_dim": hd, "group_size": gs,
                "sdpa_fp16_ms": round(t_sdpa, 5), "packed_single_ms": round(t_single, 5),
                "packed_splitk_ms": round(best_t, 5), "best_num_splits": best_ns,
                "speedup_splitk_vs_single": round(t_single / best_t, 3),
                "speedup_splitk_vs_sdpa": round(t_sdpa / best_t, 3),
                "kv_read_bytes_fp16": fp16_bytes, "kv_read_bytes_packed": packed_bytes,
                "kv_bytes_saving_pct": round(100.0 * (1 - packed_bytes / fp16_bytes), 2),
                "max_abs_err_single_vs_ref": round(err_single, 6), "max_abs_err_splitk_vs_ref": round(best_err, 6),
                "num_samples": iters,
                # beyond the reference's keys: the same call replayed from a CUDA graph (device time only), with the
                # best num_splits of the grid and with the library's own grid (num_splits=None)
                "packed_splitk_graph_ms": round(graph_ms, 5),
                "packed_auto_graph_ms": round(auto_ms, 5),
                "packed_GBps_auto_graph": round(packed_bytes / (auto_ms * 1e-3) / 1e9, 1),
            })
            print(json.dumps(rows[-1]), flush=True)
    return rows


@torch.inference_mode()
def kivi_launch_rows(lengths):
    torch.manual_seed(42)
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    rows = []
    for length in lengths:
        q = torch.randn(12, 128, device="cuda", dtype=torch.float16)
        k = pk.quantize_pack(torch.randn(2, length, 128, device="cuda", dtype=torch.float16), 4, 1, 32)
        v = pk.quantize_pack(torch.randn(2, length, 128, device="cuda", dtype=torch.float16), 4, 2, 32)
        for mode, options in (("old", dict(num_splits=8, block_n=64, num_warps=4)), ("auto", {})):
            config = plan_kivi_decode(length, 12, 128, sms, **options)
            ms = _graph_ms(lambda: _kivi_layer_partial(q, k, v, 12, **options))
            rows.append(dict(length=length, mode=mode, config=asdict(config), partial_with_reduce_ms=ms))
            print(json.dumps(rows[-1]), flush=True)
    return rows


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("which", choices=["per-token", "kivi-launch"])
    ap.add_argument("--num-kv-heads", type=int, default=4)
    ap.add_argument("--num-q-heads", type=int, default=28)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--group-size", type=int, default=32)
    ap.add_argument("--seqs", type=int, nargs="+", default=[4096, 8192, 16384, 32768])
    ap.add_argument("--bits", type=int, nargs="+", default=[2, 4])
    ap.add_argument("--splits", type=int, nargs="+", default=[8, 16, 32, 64, 128])
    ap.add_argument("--warmup", type=int, default=25)
    ap.add_argument("--iters", type=int, default=100)
    ap.add_argument("--seed", type=int, default=1234)
    ap.add_argument("--lengths", type=int, nargs="+", default=[128, 512, 8192, 28672])
    ap.add_argument("--out", type=str, default=None)
    args = ap.parse_args(argv)
    if not torch.cuda.is_available():
        raise SystemExit("a CUDA GPU is needed (需要 CUDA GPU 做真实测速)")
    props = torch.cuda.get_device_properties(0)
    meta = {"gpu": props.name, "sm_count": props.multi_processor_count, "torch": torch.__version__}
    if args.which == "per-token":
        meta.update(experiment="stage_b_decode_kernel_microbench", warmup=args.warmup, iters_median=args.iters)
        payload = {"meta": meta, "rows": per_token_rows(args.num_kv_heads, args.num_q_heads, args.head_dim, args.group_size,
                                                        args.seqs, args.bits, args.splits, args.warmup, args.iters, args.seed)}
    else:
        meta.update(measurement="CUDA graph, resident random 4-bit KV, single layer, Hq=12 Hkv=2 HD=128; excludes Python overhead")
        payload = {**meta, "results": kivi_launch_rows(args.lengths)}
    if args.out:
        with open(args.out, "w") as f:
            json.dump(payload, f, indent=2)
    return payload


if __name__ == "__main__":
    main()
