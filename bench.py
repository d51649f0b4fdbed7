"""Decode-attention benchmark of the three-tier packed KV path (Qwen2.5-7B attention shape).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--prompt S]

One *step* is one decode token's attention over all 28 layers of one sequence: per layer a 2-bit
packed prompt tier of ``--prompt`` tokens (default 32768), a 4-bit cold tier of 256 tokens and a
float16 hot tier of 128 tokens, batch 1, 28 query / 4 KV heads, head_dim 128.  The 28 layers own
distinct KV buffers (364 MB at 32768 tokens, larger than the 126 MB L2), so a step streams its
bytes from HBM.  ``value`` is algorithmic bytes per second with everything resident in HBM and
the step replayed as a CUDA graph; ``e2e`` is the same step through the public Python entry
point with q copied from pinned host memory and the output copied back, every step.

With more than one GPU (launched by torch.distributed.run) every rank decodes its own sequence
(batch sharding, no collective); the reported time is the maximum over ranks.

``--impl reference`` times the CPU restatement of the reference's dequantise-then-attend
(oracle/) on the host cores for the same layer shape, one layer per step.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

COLD_LEN, HOT_LEN, PROMPT_BITS, COLD_BITS, GROUP = 256, 128, 2, 4, 32
METRIC = "decode_attn_hbm_GBps"
UNIT = "GB/s"
FALLBACK_HBM_GBS = 6650.0
# dram__bytes_read.sum + dram__bytes_write.sum of one decode launch at 32768 prompt tokens,
# from the ncu capture summarised in profiles/decode_mma_kernel_qwen7b_32k.md.
NCU_TRAFFIC_BYTES_PER_LAUNCH = 13_630_000  # 13.12 MB split-K kernel + 0.51 MB merge, reads; writes 0


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=("ours", "reference"), default="ours")
    ap.add_argument("--prompt", type=int, default=32768, help="prompt-tier tokens per layer")
    ap.add_argument("--layers", type=int, default=28)
    ap.add_argument("--workload", choices=("decode", "pack", "serving", "longctx"), default="decode",
                    help="decode: the headline decode-attention step; pack: prefill quantise+pack and cold cooling; "
                         "serving: batch of 64 jittered sequences, batch-sharded over the GPUs; "
                         "longctx: 262144-token batch-1 decode, sequence-sharded over the GPUs")
    ap.add_argument("--batch", type=int, default=64, help="serving: sequences in the whole job")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the context sweep, the SDPA baselines and the CPU baseline")
    return ap.parse_args()


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            return float(json.load(open(path))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self._stop = index, [], threading.Event()
        self._thread = threading.Thread(target=self._run, daemon=True)

    def _run(self):
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}",
                                      "--format=csv,noheader,nounits"], capture_output=True, text=True,
                                     timeout=5).stdout.strip()
                if out:
                    self.rows.append([c.strip() for c in out.split(",")])
            except Exception:
                pass
            self._stop.wait(0.1)

    def __enter__(self):
        self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        self._thread.join(timeout=10)

    def summary(self):
        mhz = sorted(int(r[0]) for r in self.rows if r and r[0].isdigit())
        reasons = []
        for i, name in enumerate(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), 2):
            if any(len(r) > i and r[i].lower().startswith("active") for r in self.rows):
                reasons.append(name)
        mx = [int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()]
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(self.rows)}


# ----------------------------------------------------------------------------- workload
class LayerSet:
    """Packed three-tier KV of `layers` layers resident on one GPU, plus per-layer q and outputs."""

    def __init__(self, torch, device, prompt_len, layers, seed):
        from phasekv_b200 import workloads
        from phasekv_b200.kernels import packing
        from phasekv_b200.kernels.tiers import LayerTiers, PackedKVSegment
        self.shape = shape = workloads.QWEN2_5_7B
        self.prompt_len, self.layers = prompt_len, layers
        gen = torch.Generator(device=device).manual_seed(seed)

        def kv(length):
            k = torch.randn(1, shape.num_kv_heads, length, shape.head_dim, generator=gen, device=device).half()
            v = torch.randn(1, shape.num_kv_heads, length, shape.head_dim, generator=gen, device=device).half()
            for c in workloads.OUTLIER_CHANNELS[shape.head_dim]:
                k[..., c] *= workloads.OUTLIER_GAIN
            return k, v

        def pack(k, v, bits):
            return PackedKVSegment(packing.quantize_pack(k, bits, -2, GROUP), packing.quantize_pack(v, bits, -1, GROUP))

        self.tiers, self.q = [], []
        for _ in range(layers):
            pk, pv = kv(prompt_len)
            ck, cv = kv(COLD_LEN)
            hk, hv = kv(HOT_LEN)
            self.tiers.append(LayerTiers(prompt=pack(pk, pv, PROMPT_BITS), cold=[pack(ck, cv, COLD_BITS)],
                                         hot_k=hk, hot_v=hv, hot_len=HOT_LEN))
            self.q.append(torch.randn(shape.num_q_heads, shape.head_dim, generator=gen, device=device).half())
            del pk, pv
        self.bytes_per_layer = workloads.decode_algorithmic_bytes(shape, prompt_len, PROMPT_BITS, COLD_LEN,
                                                                 COLD_BITS, HOT_LEN, GROUP, GROUP)
        self.kv_bytes_resident = sum(t.prompt.nbytes + t.cold[0].nbytes + 2 * t.hot_k.numel() * 2 for t in self.tiers)


class NativeStep:
    """The step as direct C-ABI calls (descriptor arrays built once), for CUDA-graph capture."""

    def __init__(self, torch, ls: LayerSet, device):
        from phasekv_b200 import _native as nv
        from phasekv_b200.kernels.attention_cuda import layer_segments
        self.nv, self.torch, self.ls, self.device = nv, torch, ls, device
        self.L = nv.lib()
        self.sms = nv.sm_count(device)
        self.calls, self.keep = [], []
        need_max = 0
        for t in ls.tiers:
            segs, keep, hkv, hd = layer_segments(t)
            arr = (nv.Segment * len(segs))(*segs)
            need = ctypes.c_size_t(0)
            nv.check(self.L.pkv_decode_workspace_bytes(arr, len(segs), ls.shape.num_q_heads, hkv, hd, self.sms,
                                                       ctypes.byref(need)))
            need_max = max(need_max, need.value)
            self.calls.append((arr, len(segs)))
            self.keep.append(keep)
        self.ws = torch.empty(need_max, dtype=torch.uint8, device=device)
        self.out = [torch.empty_like(q) for q in ls.q]
        self.launches_per_step = 2 * ls.layers

    def run(self):
        s, ls = self.ls.shape, self.ls
        stream = self.nv.stream_of(self.device)
        for i, (arr, n) in enumerate(self.calls):
            self.nv.check(self.L.pkv_decode_attention(
                ls.q[i].data_ptr(), arr, n, s.num_q_heads, s.num_kv_heads, s.head_dim,
                1.0 / (s.head_dim ** 0.5), self.sms, self.ws.data_ptr(), self.ws.numel(),
                self.out[i].data_ptr(), None, None, None, stream))


def time_graph(torch, fn, steps, warmup, barrier=None, sampler=None, min_samples=5):
    """Capture fn() into a CUDA graph, replay it `warmup` untimed then `steps` timed times.
    Returns the mean milliseconds per step (CUDA events on the replay stream).  When a clock
    sampler is given it runs during the timed replays; if they end before it has `min_samples`
    readings, the same graph keeps replaying (untimed) until it has them, so the clocks are read
    under the load that was timed."""
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        fn()  # lazy initialisation outside the capture
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            fn()
        for _ in range(warmup):
            graph.replay()
        stream.synchronize()
        if barrier:
            barrier()
        if sampler is not None:
            sampler.__enter__()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(steps):
            graph.replay()
        e1.record(stream)
        e1.synchronize()
        torch.cuda.synchronize()
        if sampler is not None:
            t_end = time.time() + 3.0
            while len(sampler.rows) < min_samples and time.time() < t_end:
                for _ in range(50):
                    graph.replay()
                stream.synchronize()
            sampler.__exit__(None, None, None)
        if barrier:
            barrier()
    return e0.elapsed_time(e1) / steps


def time_e2e(torch, ls: LayerSet, device, steps, warmup):
    """Public API per layer with host buffers: q from pinned memory, output back to pinned memory."""
    from phasekv_b200.kernels.attention_triton import fused_phasekv_decode
    s = ls.shape
    q_host = [q.cpu().pin_memory() for q in ls.q]
    o_host = [torch.empty_like(q).pin_memory() for q in q_host]
    q_dev = [torch.empty_like(q) for q in ls.q]

    def step():
        for i in range(ls.layers):
            q_dev[i].copy_(q_host[i], non_blocking=True)
            o = fused_phasekv_decode(q_dev[i], ls.tiers[i], s.num_q_heads)
            o_host[i].copy_(o, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    e1.synchronize()
    per_step_bytes = ls.layers * s.num_q_heads * s.head_dim * 2
    return e0.elapsed_time(e1) / steps, per_step_bytes, per_step_bytes, o_host


def sdpa_baselines(torch, device, prompt_len, layers, steps, warmup):
    """FP16 scaled_dot_product_attention over the same logical context on the same GPU:
    (i) K/V expanded to the 28 query heads as the reference's micro-benchmark does
    (scripts/bench_decode_kernel.py:75-78) and (ii) GQA-aware, reading each KV head once."""
    import torch.nn.functional as F
    from phasekv_b200 import workloads
    s = workloads.QWEN2_5_7B
    S = prompt_len + COLD_LEN + HOT_LEN
    G = s.num_q_heads // s.num_kv_heads
    gen = torch.Generator(device=device).manual_seed(77)
    K = [torch.randn(1, s.num_kv_heads, S, s.head_dim, generator=gen, device=device).half() for _ in range(layers)]
    V = [torch.randn(1, s.num_kv_heads, S, s.head_dim, generator=gen, device=device).half() for _ in range(layers)]
    q = torch.randn(1, s.num_q_heads, 1, s.head_dim, generator=gen, device=device).half()
    qg = q.view(1, s.num_kv_heads, G, s.head_dim)

    def gqa():
        for k, v in zip(K, V):
            F.scaled_dot_product_attention(qg, k, v)
    res = {"gqa_aware_ms_per_step": time_graph(torch, gqa, steps, warmup)}
    if S * layers * s.num_q_heads * s.head_dim * 4 < 40e9:
        Ke = [k.repeat_interleave(G, 1) for k in K]
        Ve = [v.repeat_interleave(G, 1) for v in V]

        def expanded():
            for k, v in zip(Ke, Ve):
                F.scaled_dot_product_attention(q, k, v)
        res["expanded_ms_per_step"] = time_graph(torch, expanded, steps, warmup)
    res["fp16_kv_bytes_per_layer"] = S * s.num_kv_heads * s.head_dim * 4
    return res


# ----------------------------------------------------------------------------- CPU arm
def cpu_layer_inputs(prompt_len, seed=0):
    import torch
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import pkv_oracle as oracle
    from phasekv_b200 import workloads
    s = workloads.QWEN2_5_7B
    (pk, pv), (ck, cv), (hk, hv), q = workloads.three_tier_dense(seed, s, prompt_len, COLD_LEN, HOT_LEN)
    segs = [(oracle.quantize_pack(pk, PROMPT_BITS, -2, GROUP), oracle.quantize_pack(pv, PROMPT_BITS, -1, GROUP)),
            (oracle.quantize_pack(ck, COLD_BITS, -2, GROUP), oracle.quantize_pack(cv, COLD_BITS, -1, GROUP))]
    return oracle, s, segs, hk, hv, q[0, :, 0, :]


def time_cpu_layers(prompt_len, layers_per_step, steps, warmup):
    """Seconds per step of the CPU dequantise-then-attend for `layers_per_step` layers."""
    oracle, s, segs, hk, hv, q = cpu_layer_inputs(prompt_len)
    def step():
        for _ in range(layers_per_step):
            oracle.segments_decode_reference(q, segs, hk, hv, s.num_q_heads)
    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    return (time.perf_counter() - t0) / steps, oracle.num_threads()


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from phasekv_b200 import workloads
    bytes_per_layer = workloads.decode_algorithmic_bytes(workloads.QWEN2_5_7B, args.prompt, PROMPT_BITS, COLD_LEN,
                                                         COLD_BITS, HOT_LEN, GROUP, GROUP)
    steps, warmup = min(args.steps, 20), min(max(args.warmup, 1), 3)
    sec, cores = time_cpu_layers(args.prompt, 1, steps, warmup)
    value = bytes_per_layer / sec / 1e9
    sample = f"1 of {args.layers} layers per step (dequantise-then-attend of one layer at {args.prompt} prompt tokens)"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
        "warmup": warmup, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def workload_config(args):
    return {"workload": f"qwen2.5-7b decode attention, {args.layers} layers x ({args.prompt} prompt tok @2-bit KIVI + "
                        f"{COLD_LEN} cold tok @4-bit + {HOT_LEN} hot tok fp16), batch 1 per GPU, 28q/4kv heads, hd 128, gs 32",
            "prompt_tokens": args.prompt, "layers": args.layers, "l2_policy": "inputs larger than L2 (distinct KV per layer)",
            "parallelism": "batch-sharded, no collective"}


# ----------------------------------------------------------------------------- pack workload
def run_pack_workload(args):
    """Prefill quantise+pack of 32768 tokens x 4 KV heads x 128 dims (K along tokens, V along dims) at
    2/4/8 bits over rotating input buffers larger than L2, and the lazy cold-tier cooling step
    (64 aged tokens -> top 32 by value norm, 4-bit).  One JSON line; value = 2-bit K+V pack GB/s."""
    import torch
    from phasekv_b200 import workloads
    from phasekv_b200.cold_tier import select_and_pack_cold
    from phasekv_b200.kernels import packing
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    s = workloads.QWEN2_5_7B
    S, copies = 32768, 6  # 6 x (K + V) x 33.5 MB = 403 MB of input
    gen = torch.Generator(device=dev).manual_seed(5)
    ks = [torch.randn(1, s.num_kv_heads, S, s.head_dim, generator=gen, device=dev).half() for _ in range(copies)]
    vs = [torch.randn(1, s.num_kv_heads, S, s.head_dim, generator=gen, device=dev).half() for _ in range(copies)]
    peak, peak_kind = measured_peak()
    res = {}
    for bits in (2, 4, 8):
        def step():
            for k, v in zip(ks, vs):
                packing.quantize_pack(k, bits, -2, GROUP)
                packing.quantize_pack(v, bits, -1, GROUP)
        reps = args.steps // 10 + 1
        ms = time_graph(torch, step, reps, 3)  # graph replay: no Python between the launches
        us = ms * 1e3 / copies
        nbytes = 2 * (S * s.num_kv_heads * s.head_dim) * 2 + 2 * S * s.num_kv_heads * (s.head_dim * bits // 8 + 4 * s.head_dim // GROUP)
        res[str(bits)] = {"us_per_kv_pack": us, "GBps": nbytes / us / 1e3, "frac_of_peak": nbytes / us / 1e3 / peak,
                          "algorithmic_bytes": nbytes}
    hot_k = torch.randn(1, s.num_kv_heads, 192, s.head_dim, generator=gen, device=dev).half()
    hot_v = torch.randn(1, s.num_kv_heads, 192, s.head_dim, generator=gen, device=dev).half()
    for _ in range(3):
        select_and_pack_cold(hot_k.clone(), hot_v.clone(), 192, 64, 32, 4, GROUP)
    bufs = [(hot_k.clone(), hot_v.clone()) for _ in range(50)]
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for bk, bv in bufs:
        select_and_pack_cold(bk, bv, 192, 64, 32, 4, GROUP)
    e1.record()
    e1.synchronize()
    print(json.dumps({"metric": "quantize_pack_GBps", "value": res["2"]["GBps"], "unit": UNIT, "n_gpus": 1,
                      "steps": args.steps, "warmup": 3, "higher_is_better": True, "data": "synthetic",
                      "config": {"workload": "prefill quantise+pack, 32768 tok x 4 KV heads x 128 dims, K along tokens + V along dims, gs 32",
                                 "l2_policy": "rotating inputs larger than L2"},
                      "by_bits": res, "peak": peak, "peak_source": f"of {peak_kind}",
                      "cold_cooling_us": e0.elapsed_time(e1) * 1e3 / len(bufs),
                      "cold_config": "64 aged of 192 hot tokens -> keep 32, 4-bit, 4 KV heads, one launch (python call included)"}))


# ----------------------------------------------------------------------------- multi-GPU set-up shared by the sharded workloads
def dist_setup():
    import torch
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: phasekv_b200 has no CPU path")
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    barrier = None
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
        barrier = lambda: (dist.barrier(), torch.cuda.synchronize())  # noqa: E731
    return torch, dist, world, rank, local_rank, device, barrier


def max_over_ranks(torch, dist, world, device, values):
    if world == 1:
        return values
    t = torch.tensor(values, device=device, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return [float(x) for x in t]


# ----------------------------------------------------------------------------- batched serving workload
def run_serving_workload(args):
    """Batched serving decode: `--batch` sequences of 8192 prompt tokens @2-bit + 512 cold @4-bit + 128 hot
    (each length jittered by +-25 %), all layers, sharded by batch over the GPUs with no collective (strong
    scaling: the batch is fixed).  A step is one decode token: per layer ONE batched split-K launch + one merge
    launch over this rank's sequences.  Also timed: the same step as a loop of batch-1 calls over the sequences,
    which is how the reference's batch-1 entry point would be driven."""
    torch, dist, world, rank, local_rank, device, barrier = dist_setup()
    from phasekv_b200 import _native as nv
    from phasekv_b200 import sharding, workloads
    from phasekv_b200.kernels import attention_cuda as attn
    s = workloads.QWEN2_5_7B
    lengths = workloads.jittered_lengths(0, args.batch, 8192, 512, 128, hot_capacity=192)
    mine = sharding.batch_shard(args.batch, world, rank)
    plans, qs, tiers_all = [], [], []
    for layer in range(args.layers):
        tiers, q = [], []
        for i in mine:
            p, c, h = lengths[i]
            t, qq = workloads.gpu_three_tier(s, p, PROMPT_BITS, c, COLD_BITS, h, workloads.layer_seed(1, layer, i), device)
            tiers.append(t), q.append(qq)
        plans.append(attn.BatchDecodePlan(tiers, s.num_q_heads))
        qs.append(torch.stack(q))
        tiers_all.append(tiers)
    job_bytes = args.layers * sum(workloads.decode_algorithmic_bytes(s, p, PROMPT_BITS, c, COLD_BITS, h, GROUP, GROUP)
                                  for p, c, h in lengths)
    rank_layer_bytes = sum(workloads.decode_algorithmic_bytes(s, *_pch(lengths[i]), GROUP, GROUP) for i in mine)
    L = nv.lib()
    ws = torch.empty(max(p.workspace_bytes for p in plans), dtype=torch.uint8, device=device)
    outs = [torch.empty_like(q) for q in qs]

    def step():
        stream = nv.stream_of(device)
        for p, q, o in zip(plans, qs, outs):
            nv.check(L.pkv_decode_attention_batched(q.data_ptr(), p.table_host.data_ptr(), p.table_device.data_ptr(),
                                                    1.0 / (s.head_dim ** 0.5), ws.data_ptr(), ws.numel(), o.data_ptr(),
                                                    stream))
    torch.cuda.synchronize()
    clocks = ClockSampler(local_rank)
    ms = time_graph(torch, step, args.steps, max(args.warmup, 3), barrier, sampler=clocks)

    # end to end through the Python entry point: q from pinned host memory, outputs back to the host
    q_host = [q.cpu().pin_memory() for q in qs]
    o_host = [torch.empty_like(q) for q in q_host]
    o_host = [o.pin_memory() for o in o_host]
    q_dev = [torch.empty_like(q) for q in qs]

    def e2e_step():
        for i, p in enumerate(plans):
            q_dev[i].copy_(q_host[i], non_blocking=True)
            o_host[i].copy_(attn.fused_phasekv_decode_batched(q_dev[i], p, s.num_q_heads), non_blocking=True)
        torch.cuda.current_stream().synchronize()
    for _ in range(3):
        e2e_step()
    if barrier:
        barrier()
    n_e2e = max(3, min(args.steps, 20))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(n_e2e):
        e2e_step()
    e1.record()
    e1.synchronize()
    ms_e2e = e0.elapsed_time(e1) / n_e2e

    # the same step as a loop of batch-1 calls (2 layers, scaled)
    loop_layers = min(2, args.layers)

    def loop_step():
        for layer in range(loop_layers):
            for i, t in enumerate(tiers_all[layer]):
                attn.fused_phasekv_decode(qs[layer][i], t, s.num_q_heads)
    ms_loop = time_graph(torch, loop_step, 10, 3) * args.layers / loop_layers

    ms, ms_e2e, ms_loop = max_over_ranks(torch, dist, world, device, [ms, ms_e2e, ms_loop])
    peak, peak_kind = measured_peak()
    achieved = rank_layer_bytes / (ms / args.layers * 1e-3) / 1e9
    h2d = sum(q.numel() * 2 for q in qs) * world
    if rank == 0:
        print(json.dumps({
            "metric": METRIC, "value": job_bytes / (ms * 1e-3) / 1e9, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f16 codes x f16, f32 accumulate", "data": "synthetic",
            "config": {"workload": f"qwen2.5-7b batched serving decode, {args.layers} layers, batch {args.batch} "
                                   "(8192 prompt tok @2-bit KIVI + 512 cold @4-bit + 128 hot fp16 per sequence, lengths "
                                   "jittered +-25 %), 28q/4kv heads, hd 128, gs 32",
                       "batch": args.batch, "layers": args.layers, "sequences_per_gpu": len(mine),
                       "l2_policy": "inputs larger than L2 (distinct KV per layer and sequence)",
                       "parallelism": "batch-sharded, no collective"},
            "us_per_layer": ms / args.layers * 1e3, "tokens_per_s": args.batch / (ms * 1e-3),
            "e2e": {"value": job_bytes / (ms_e2e * 1e-3) / 1e9, "unit": UNIT, "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": h2d, "ms_per_step": ms_e2e},
            "gpu_launches": 2 * args.layers * args.steps,
            "per_sequence_loop": {"ms_per_step": ms_loop, "speedup_of_batched": ms_loop / ms,
                                  "sample": f"{loop_layers} of {args.layers} layers, scaled"},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": None, "peak_source": f"of {peak_kind}",
                         "kernel": "batched split-K decode + merge, per layer, rank 0's share",
                         "algorithmic_bytes_per_launch": rank_layer_bytes},
            "clocks": clocks.summary(),
        }))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def _pch(length):
    p, c, h = length
    return p, PROMPT_BITS, c, COLD_BITS, h


# ----------------------------------------------------------------------------- long-context workload
LONG_PROMPT, LONG_COLD = 262144, 1024


def run_longctx_workload(args):
    """Long-context batch-1 decode: 262144 prompt tokens @2-bit cut into one contiguous shard per GPU, 1024 cold
    tokens @4-bit and 128 hot tokens on rank 0.  Per layer every rank computes the un-normalised partial of its
    shard, the partials (Hq*(hd+2)*4 bytes per rank) are all-gathered over NVLink (NCCL) and merged on every
    rank.  Strong scaling: the context is fixed.  The layers are chained through the stream as they would be in
    a model (layer l+1 is launched behind layer l's exchange)."""
    torch, dist, world, rank, local_rank, device, barrier = dist_setup()
    from phasekv_b200 import sharding, workloads
    s = workloads.QWEN2_5_7B
    start, end = sharding.sequence_bounds(LONG_PROMPT, world)[rank]
    if world == 1:
        # one rank: the exchange is a loopback; a one-rank process group keeps the NCCL variant runnable
        dist.init_process_group("nccl", init_method="tcp://127.0.0.1:%d" % (29400 + os.getpid() % 500), rank=0,
                                world_size=1, device_id=device)
    exchange = sharding.PeerExchange(s.num_q_heads, s.head_dim, device, loopback=(world == 1),
                                     world=world, rank=rank)
    layers, layers_nccl, qs = [], [], []
    for layer in range(args.layers):
        t, q = workloads.gpu_three_tier(s, end - start, PROMPT_BITS, LONG_COLD if rank == 0 else 0, COLD_BITS,
                                        HOT_LEN if rank == 0 else 0, workloads.layer_seed(2, layer, rank), device)
        segs = [(t.prompt.key, t.prompt.value)] + [(c.key, c.value) for c in t.cold]
        layers.append(sharding.ShardedDecodeLayer(segs, t.hot_k, t.hot_v, s.num_q_heads, s.head_dim, device,
                                                  exchange=exchange))
        layers_nccl.append(sharding.ShardedDecodeLayer(segs, t.hot_k, t.hot_v, s.num_q_heads, s.head_dim, device))
        qs.append(q)
    layer_bytes = workloads.decode_algorithmic_bytes(s, LONG_PROMPT, PROMPT_BITS, LONG_COLD, COLD_BITS, HOT_LEN, GROUP, GROUP)
    rank_bytes = workloads.decode_algorithmic_bytes(s, end - start, PROMPT_BITS, LONG_COLD if rank == 0 else 0, COLD_BITS,
                                                    HOT_LEN if rank == 0 else 0, GROUP, GROUP)

    def step():
        for lay, q in zip(layers, qs):
            lay.run(q)

    def step_nccl():
        for lay, q in zip(layers_nccl, qs):
            lay.run(q)
    step(), step_nccl()
    torch.cuda.synchronize()
    same = all(bool(torch.equal(a.out, b.out)) for a, b in zip(layers, layers_nccl))
    clocks = ClockSampler(local_rank)
    ms = time_graph(torch, step, args.steps, max(args.warmup, 3), barrier, sampler=clocks)
    how = "cuda graph"
    try:
        ms_nccl = time_graph(torch, step_nccl, args.steps, max(args.warmup, 3), barrier)
    except Exception as exc:  # a collective that cannot be captured
        ms_nccl, how = None, how + f"; NCCL variant not captured ({type(exc).__name__})"
    timed_out = exchange.timed_out()
    # end to end: q from pinned host memory per layer, merged output back to the host
    q_host = [q.cpu().pin_memory() for q in qs]
    o_host = [torch.empty_like(q).pin_memory() for q in q_host]
    q_dev = [torch.empty_like(q) for q in qs]

    def e2e_step():
        for i, lay in enumerate(layers):
            q_dev[i].copy_(q_host[i], non_blocking=True)
            o_host[i].copy_(lay.run(q_dev[i]), non_blocking=True)
        torch.cuda.current_stream().synchronize()
    for _ in range(3):
        e2e_step()
    if barrier:
        barrier()
    n_e2e = max(3, min(args.steps, 20))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(n_e2e):
        e2e_step()
    e1.record()
    e1.synchronize()
    ms_e2e = e0.elapsed_time(e1) / n_e2e
    ms, ms_e2e, ms_nccl = max_over_ranks(torch, dist, world, device, [ms, ms_e2e, ms_nccl or 0.0])
    peak, peak_kind = measured_peak()
    achieved = rank_bytes / (ms / args.layers * 1e-3) / 1e9
    io = args.layers * s.num_q_heads * s.head_dim * 2
    if rank == 0:
        print(json.dumps({
            "metric": METRIC, "value": layer_bytes * args.layers / (ms * 1e-3) / 1e9, "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f16 codes x f16, f32 accumulate", "data": "synthetic",
            "config": {"workload": f"qwen2.5-7b long-context batch-1 decode, {args.layers} layers x ({LONG_PROMPT} prompt tok "
                                   f"@2-bit KIVI sequence-sharded + {LONG_COLD} cold @4-bit + {HOT_LEN} hot fp16 on rank 0), "
                                   "28q/4kv heads, hd 128, gs 32",
                       "layers": args.layers, "prompt_tokens_per_gpu": end - start,
                       "l2_policy": "inputs larger than L2 (distinct KV per layer)",
                       "parallelism": f"sequence-sharded x{world}; per layer every rank pushes its partial "
                                      f"({s.num_q_heads * (s.head_dim + 2) * 4} B) into the peers' memory over NVLink and "
                                      "merges what arrived, inside one kernel (no collective library)", "timed_as": how},
            "us_per_layer": ms / args.layers * 1e3,
            "nccl_all_gather_variant": {"ms_per_step": ms_nccl or None, "same_output_bits": same},
            "exchange_wait_timed_out": timed_out,
            "e2e": {"value": layer_bytes * args.layers / (ms_e2e * 1e-3) / 1e9, "unit": UNIT, "h2d_bytes_per_step": io,
                    "d2h_bytes_per_step": io, "ms_per_step": ms_e2e},
            "gpu_launches": 2 * args.layers * args.steps,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": None, "peak_source": f"of {peak_kind}",
                         "kernel": "split-K decode of rank 0's shard + exchange/merge kernel, per layer",
                         "algorithmic_bytes_per_launch": rank_bytes},
            "clocks": clocks.summary(),
        }))
    dist.barrier()
    exchange.close()
    dist.destroy_process_group()


# ----------------------------------------------------------------------------- main arm
def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
        return
    if args.workload == "pack":
        run_pack_workload(args)
        return
    if args.workload == "serving":
        run_serving_workload(args)
        return
    if args.workload == "longctx":
        run_longctx_workload(args)
        return
    import torch
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: phasekv_b200 has no CPU path")
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    barrier = None
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
        barrier = lambda: (dist.barrier(), torch.cuda.synchronize())  # noqa: E731

    ls = LayerSet(torch, device, args.prompt, args.layers, seed=1234 + rank)
    native = NativeStep(torch, ls, device)
    torch.cuda.synchronize()

    clocks = ClockSampler(local_rank)
    ms = time_graph(torch, native.run, args.steps, max(args.warmup, 3), barrier, sampler=clocks)
    ms_e2e, h2d, d2h, o_host = time_e2e(torch, ls, device, max(3, min(args.steps, 20)), 3)

    if world > 1:
        t = torch.tensor([ms, ms_e2e], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, ms_e2e = float(t[0]), float(t[1])

    step_bytes = ls.bytes_per_layer * ls.layers * world
    value = step_bytes / (ms * 1e-3) / 1e9
    e2e_value = step_bytes / (ms_e2e * 1e-3) / 1e9
    peak, peak_kind = measured_peak()
    per_launch_ms = ms / ls.layers
    achieved = ls.bytes_per_layer / (per_launch_ms * 1e-3) / 1e9
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16 codes x f16, f32 accumulate", "data": "synthetic",
        "config": workload_config(args),
        "us_per_layer": per_launch_ms * 1e3,
        "pct_of_8TBps": 100.0 * achieved / 8000.0,
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": ms_e2e},
        "gpu_launches": native.launches_per_step * args.steps,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": NCU_TRAFFIC_BYTES_PER_LAUNCH, "peak_source": f"of {peak_kind}",
                     "kernel": "split-K decode + merge, per layer", "algorithmic_bytes_per_launch": ls.bytes_per_layer},
        "clocks": clocks.summary(),
    }

    if rank == 0 and world == 1 and not args.no_extras:
        # parity spot check of the timed configuration against the CPU oracle (layer built from CPU bits)
        oracle, s, segs, hk, hv, q = cpu_layer_inputs(args.prompt)
        from phasekv_b200.kernels.attention_triton import fused_phasekv_decode
        from phasekv_b200.kernels.packing import PackedTensor
        from phasekv_b200.kernels.tiers import LayerTiers, PackedKVSegment

        def gpu(pt):
            return PackedTensor(pt.packed.to(device), pt.scale.to(device), pt.mins.to(device), pt.bits, pt.axis,
                                pt.group_size, pt.orig_shape, pt.axis_len)
        tiers = LayerTiers(prompt=PackedKVSegment(gpu(segs[0][0]), gpu(segs[0][1])),
                           cold=[PackedKVSegment(gpu(segs[1][0]), gpu(segs[1][1]))],
                           hot_k=hk.to(device), hot_v=hv.to(device), hot_len=HOT_LEN)
        out = fused_phasekv_decode(q.to(device), tiers, s.num_q_heads).float().cpu()
        t0 = time.perf_counter()
        ref = oracle.segments_decode_reference(q, segs, hk, hv, s.num_q_heads).float()
        line["parity"] = {"max_abs_err_vs_oracle": float((out - ref).abs().max()), "max_abs_ref": float(ref.abs().max())}
        # CPU baseline on a bounded sample
        n_cpu = 8
        sec, cores = time_cpu_layers(args.prompt, 1, n_cpu, 1)
        line["cpu_baseline"] = {"value": ls.bytes_per_layer / sec / 1e9, "unit": UNIT, "cores": cores, "kind": "port",
                                "sample": f"{n_cpu} single-layer calls of the CPU dequantise-then-attend at {args.prompt} prompt tokens",
                                "ms_per_layer": sec * 1e3}
        # FP16 SDPA on the same GPU
        del native, ls
        torch.cuda.empty_cache()
        sd = sdpa_baselines(torch, device, args.prompt, args.layers, 20, 3)
        sd["speedup_vs_gqa_aware"] = sd["gqa_aware_ms_per_step"] / ms
        if "expanded_ms_per_step" in sd:
            sd["speedup_vs_expanded"] = sd["expanded_ms_per_step"] / ms
        line["sdpa_fp16"] = sd
        # context sweep 4K .. 128K
        sweep = {}
        for S in (4096, 8192, 16384, 32768, 131072):
            if S == args.prompt:
                sweep[str(S)] = {"us_per_layer": per_launch_ms * 1e3, "GBps": achieved, "frac_of_peak": achieved / peak}
                continue
            l2 = LayerSet(torch, device, S, args.layers, seed=99 + S)
            n2 = NativeStep(torch, l2, device)
            m2 = time_graph(torch, n2.run, 20, 3)
            a2 = l2.bytes_per_layer / (m2 / l2.layers * 1e-3) / 1e9
            sweep[str(S)] = {"us_per_layer": m2 / l2.layers * 1e3, "GBps": a2, "frac_of_peak": a2 / peak,
                             "kv_bytes_resident": l2.kv_bytes_resident}
            del l2, n2
            torch.cuda.empty_cache()
        line["contexts"] = sweep
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
