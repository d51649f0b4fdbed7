"""Decode-attention benchmark of the three-tier packed KV path (Qwen2.5-7B attention shape).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--prompt S]

One *step* is one decode token's attention over all 28 layers of one sequence: per layer a 2-bit
packed prompt tier of ``--prompt`` tokens (default 32768), a 4-bit cold tier of 256 tokens and a
float16 hot tier of 128 tokens, batch 1, 28 query / 4 KV heads, head_dim 128.  The 28 layers own
distinct KV buffers (364 MB at 32768 tokens, larger than the 126 MB L2), so a step streams its
bytes from HBM.  ``value`` is algorithmic bytes per second with everything resident in HBM and
the step replayed as a CUDA graph; ``e2e`` is the same step with host buffers: every step the queries are copied
from pinned host memory, ``pkv_decode_attention`` is called once per layer through the C ABI (no graph), the outputs
are copied back and the host waits for them (``e2e.python_entry_*``: the same through the reference-facing Python
function ``fused_phasekv_decode`` with per-layer copies).

With more than one GPU (launched by torch.distributed.run) every rank decodes its own sequence
(batch sharding, no collective); the reported time is the maximum over ranks.

After the headline the same process measures, and adds to the JSON line under ``sharded``, the two configurations
that shard over GPUs (``longctx``: 262144 prompt tokens sequence-sharded with one exchange of partials per layer;
``serving``: 64 sequences batch-sharded) and, on one GPU, the quantise+pack kernels (``pack``), the one-launch
attention of a chunk of new prompt tokens against the token-by-token order (``prompt_chunk``), decode over a
cold tier kept in arenas after 1000 generated tokens (``cold_arena``), one attention layer through the model adapter
(``adapter_layer``) and a whole decode step of the attention path replayed from one CUDA graph (``graphed_step``).

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
# dram__bytes_read.sum + dram__bytes_write.sum of the kernels of one layer (split-K + merge), per prompt length, from
# ncu captures of this workload with a few layers (traffic per launch does not depend on the layer count).
# A prompt length without a capture reports null.  At 32768 tokens: split-K launch 13 140 736 + merge launch 508 160.
NCU_TRAFFIC_BYTES_PER_LAUNCH = {32768: 13648896}
NCU_TRAFFIC_SOURCE = "ncu dram__bytes_read.sum + dram__bytes_write.sum, split-K + merge kernels of one layer"


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
    ap.add_argument("--no-sharded", action="store_true",
                    help="decode workload: skip the `sharded` block (long-context, serving and pack measurements)")
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
        need_max, launches = 0, 0
        for t in ls.tiers:
            segs, keep, hkv, hd = layer_segments(t)
            arr = (nv.Segment * len(segs))(*segs)
            need = ctypes.c_size_t(0)
            nv.check(self.L.pkv_decode_workspace_bytes(arr, len(segs), ls.shape.num_q_heads, hkv, hd, self.sms,
                                                       ctypes.byref(need)))
            need_max = max(need_max, need.value)
            count = ctypes.c_int(0)
            nv.check(self.L.pkv_decode_launches(arr, len(segs), ls.shape.num_q_heads, hkv, hd, self.sms,
                                                ctypes.byref(count)))
            launches += count.value
            self.calls.append((arr, len(segs)))
            self.keep.append(keep)
        self.ws = torch.empty(need_max, dtype=torch.uint8, device=device)
        self.out = [torch.empty_like(q) for q in ls.q]
        self.launches_per_step = launches

    def run(self):
        s, ls = self.ls.shape, self.ls
        stream = self.nv.stream_of(self.device)
        for i, (arr, n) in enumerate(self.calls):
            self.nv.check(self.L.pkv_decode_attention(
                ls.q[i].data_ptr(), arr, n, s.num_q_heads, s.num_kv_heads, s.head_dim,
                1.0 / (s.head_dim ** 0.5), self.sms, self.ws.data_ptr(), self.ws.numel(),
                self.out[i].data_ptr(), None, None, None, stream))


def time_graph(torch, fn, steps, warmup, barrier=None, sampler=None, agree_max=None):
    """Capture fn() into a CUDA graph, replay it `warmup` untimed then `steps` timed times.
    Returns the mean milliseconds per step (CUDA events on the replay stream).  When a clock
    sampler is given it runs during the timed replays and during a top-up of further untimed
    replays (about 1.5 s of the same load), so that it reads the clocks under the load that was
    timed.  The number of top-up replays is computed from the measured step time and, when the
    step contains an exchange between ranks, agreed on across the ranks first (`agree_max`, a
    function that returns the maximum of an int over all ranks): every rank must replay a graph
    that holds a peer exchange exactly as often as its peers do."""
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
        ms = e0.elapsed_time(e1) / steps
        if sampler is not None:
            extra = max(0, min(40000, int(1500.0 / max(ms, 1e-3)) - steps))
            if agree_max is not None:
                extra = agree_max(extra)
            for _ in range(extra):
                graph.replay()
            stream.synchronize()
            sampler.__exit__(None, None, None)
        if barrier:
            barrier()
    return ms


def _timed_steps(torch, step, steps, warmup):
    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    e1.synchronize()
    return e0.elapsed_time(e1) / steps


def time_e2e(torch, ls: LayerSet, native: "NativeStep", device, steps, warmup):
    """The step with HOST buffers, copies inside the timed region.  Two ways to call:

    * `c_abi`: what a serving runtime does: every step the queries of all layers are copied from pinned host memory,
      `pkv_decode_attention` is called once per layer (plain calls, no graph: the cache may have changed since the
      last step), the outputs are copied back to pinned host memory, and the host waits for them;
    * `python_entry`: the reference-facing Python function `fused_phasekv_decode(q, tiers, Hq)` per layer with a
      host-to-device and a device-to-host copy per layer, as a caller of the reference's module would write it.

    Returns (c_abi ms, python_entry ms, bytes in per step, bytes out per step, host outputs of the c_abi way)."""
    from phasekv_b200.kernels.attention_triton import fused_phasekv_decode
    s = ls.shape
    nv, L = native.nv, native.L
    q_host = torch.stack([q.cpu() for q in ls.q]).pin_memory()           # [layers, Hq, hd]
    o_host = torch.empty_like(q_host).pin_memory()
    q_dev, o_dev = torch.empty_like(q_host, device=device), torch.empty_like(q_host, device=device)
    scale = 1.0 / (s.head_dim ** 0.5)

    def step_c_abi():
        q_dev.copy_(q_host, non_blocking=True)
        stream = nv.stream_of(device)
        for i, (arr, n) in enumerate(native.calls):
            nv.check(L.pkv_decode_attention(q_dev[i].data_ptr(), arr, n, s.num_q_heads, s.num_kv_heads, s.head_dim, scale,
                                            native.sms, native.ws.data_ptr(), native.ws.numel(), o_dev[i].data_ptr(),
                                            None, None, None, stream))
        o_host.copy_(o_dev, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    q_dev_l = [torch.empty_like(q) for q in ls.q]
    o_host_l = [torch.empty_like(q).cpu().pin_memory() for q in ls.q]

    def step_python():
        for i in range(ls.layers):
            q_dev_l[i].copy_(q_host[i], non_blocking=True)
            o = fused_phasekv_decode(q_dev_l[i], ls.tiers[i], s.num_q_heads)
            o_host_l[i].copy_(o, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    ms_c = _timed_steps(torch, step_c_abi, steps, warmup)
    ms_py = _timed_steps(torch, step_python, steps, warmup)
    per_step_bytes = ls.layers * s.num_q_heads * s.head_dim * 2
    return ms_c, ms_py, per_step_bytes, per_step_bytes, o_host


def sdpa_baselines(torch, device, prompt_len, layers, steps, warmup):
    """FP16 attention over the same logical context on the same GPU, every variant a CUDA-graph replay over
    `layers` distinct K/V buffers:
    (i)   K/V expanded to the 28 query heads as the reference's micro-benchmark does
          (scripts/bench_decode_kernel.py:75-78);
    (ii)  GQA-aware calls that read each KV head once: scaled_dot_product_attention with enable_gqa under the
          flash and the memory-efficient backends, the same with q viewed as [1, Hkv, G, hd], and
          flash_attn_with_kvcache where that library runs;
    (iii) this library's own float16 tile path over the whole context (one PKV_SEG_FP16 segment).
    The fastest GQA-aware time is what "x times faster than FP16" is quoted against; the bound of an ideal
    FP16 kernel (K/V bytes at the measured HBM peak) is printed beside it."""
    import torch.nn.functional as F
    from torch.nn.attention import SDPBackend, sdpa_kernel
    from phasekv_b200 import _native as nv
    from phasekv_b200 import workloads
    from phasekv_b200.kernels import attention_cuda as attn
    s = workloads.QWEN2_5_7B
    S = prompt_len + COLD_LEN + HOT_LEN
    G = s.num_q_heads // s.num_kv_heads
    gen = torch.Generator(device=device).manual_seed(77)
    K = [torch.randn(1, s.num_kv_heads, S, s.head_dim, generator=gen, device=device).half() for _ in range(layers)]
    V = [torch.randn(1, s.num_kv_heads, S, s.head_dim, generator=gen, device=device).half() for _ in range(layers)]
    q = torch.randn(1, s.num_q_heads, 1, s.head_dim, generator=gen, device=device).half()
    qg = q.view(1, s.num_kv_heads, G, s.head_dim)
    res, gqa = {}, {}

    def attempt(name, fn):
        try:
            gqa[name] = time_graph(torch, fn, steps, warmup)
        except Exception as exc:  # a backend that does not take the call
            gqa[name] = f"unavailable: {type(exc).__name__}"

    for tag, backend in (("flash", SDPBackend.FLASH_ATTENTION), ("efficient", SDPBackend.EFFICIENT_ATTENTION)):
        def gqa_flag(backend=backend):
            with sdpa_kernel([backend]):
                for k, v in zip(K, V):
                    F.scaled_dot_product_attention(q, k, v, enable_gqa=True)

        def gqa_view(backend=backend):
            with sdpa_kernel([backend]):
                for k, v in zip(K, V):
                    F.scaled_dot_product_attention(qg, k, v)
        attempt(f"sdpa_enable_gqa_{tag}_ms_per_step", gqa_flag)
        attempt(f"sdpa_q_as_group_rows_{tag}_ms_per_step", gqa_view)

    def gqa_default():
        for k, v in zip(K, V):
            F.scaled_dot_product_attention(qg, k, v)
    attempt("sdpa_q_as_group_rows_default_ms_per_step", gqa_default)
    try:
        from flash_attn import flash_attn_with_kvcache
        Kt = [k.transpose(1, 2).contiguous() for k in K]  # [1, S, Hkv, hd]
        Vt = [v.transpose(1, 2).contiguous() for v in V]
        qt = q.transpose(1, 2).contiguous()

        def fa():
            for k, v in zip(Kt, Vt):
                flash_attn_with_kvcache(qt, k, v)
        attempt("flash_attn_with_kvcache_ms_per_step", fa)
        del Kt, Vt
    except Exception as exc:
        gqa["flash_attn_with_kvcache_ms_per_step"] = f"unavailable: {type(exc).__name__}"

    # this library's float16 tiles over the whole context
    L, sms = nv.lib(), nv.sm_count(device)
    calls, keep, need_max = [], [], 0
    for k, v in zip(K, V):
        seg, kp = attn._fp16_segment(k[0], v[0])
        arr = (nv.Segment * 1)(seg)
        need = ctypes.c_size_t(0)
        nv.check(L.pkv_decode_workspace_bytes(arr, 1, s.num_q_heads, s.num_kv_heads, s.head_dim, sms, ctypes.byref(need)))
        need_max = max(need_max, need.value)
        calls.append(arr), keep.append(kp)
    ws = torch.empty(need_max, dtype=torch.uint8, device=device)
    out = torch.empty(s.num_q_heads, s.head_dim, dtype=torch.float16, device=device)
    q2 = q[0, :, 0, :].contiguous()

    def own():
        stream = nv.stream_of(device)
        for arr in calls:
            nv.check(L.pkv_decode_attention(q2.data_ptr(), arr, 1, s.num_q_heads, s.num_kv_heads, s.head_dim,
                                            1.0 / (s.head_dim ** 0.5), sms, ws.data_ptr(), ws.numel(), out.data_ptr(),
                                            None, None, None, stream))
    attempt("own_fp16_kernel_ms_per_step", own)
    res["gqa_aware"] = gqa
    timed = {k: v for k, v in gqa.items() if isinstance(v, float)}
    if timed:
        best = min(timed, key=timed.get)
        res["gqa_aware_best"] = best
        res["gqa_aware_ms_per_step"] = timed[best]
    if S * layers * s.num_q_heads * s.head_dim * 4 < 40e9:
        Ke = [k.repeat_interleave(G, 1) for k in K]
        Ve = [v.repeat_interleave(G, 1) for v in V]

        def expanded():
            for k, v in zip(Ke, Ve):
                F.scaled_dot_product_attention(q, k, v)
        res["expanded_ms_per_step"] = time_graph(torch, expanded, steps, warmup)
    res["fp16_kv_bytes_per_layer"] = S * s.num_kv_heads * s.head_dim * 4
    peak, _ = measured_peak()
    res["ideal_fp16_ms_per_step"] = layers * res["fp16_kv_bytes_per_layer"] / (peak * 1e9) * 1e3
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
    # torch.distributed.run exports OMP_NUM_THREADS=1 to its workers: this arm runs on rank 0 alone and takes
    # every host core it is allowed to use
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import pkv_oracle
    try:
        avail = len(os.sched_getaffinity(0))
    except AttributeError:
        avail = os.cpu_count() or 1
    pkv_oracle.set_num_threads(avail)
    steps, warmup = min(args.steps, 20), max(args.warmup, 1)
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


# ----------------------------------------------------------------------------- process group and helpers
class Ctx:
    """One process per GPU: device, process group (NCCL; a one-rank group at N = 1 so that the all-gather variant
    of the sequence-sharded decode can run), a barrier and a maximum-over-ranks of small host values."""

    def __init__(self):
        import torch
        import torch.distributed as dist
        self.torch, self.dist = torch, dist
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        if not torch.cuda.is_available():
            raise SystemExit("bench.py needs a CUDA device: phasekv_b200 has no CPU path")
        self.device = torch.device("cuda", self.local_rank)
        torch.cuda.set_device(self.device)
        self.group_ok = False
        self.barrier = None

    def init_group(self):
        """NCCL process group; at N = 1 a one-rank group on the loopback address."""
        if self.group_ok:
            return True
        torch, dist = self.torch, self.dist
        try:
            if self.world > 1:
                dist.init_process_group("nccl", device_id=self.device)
                self.barrier = lambda: (dist.barrier(), torch.cuda.synchronize())
            else:
                dist.init_process_group("nccl", init_method="tcp://127.0.0.1:%d" % (29400 + os.getpid() % 500), rank=0,
                                        world_size=1, device_id=self.device)
            self.group_ok = True
        except Exception as exc:  # no NCCL on this box: the all-gather variant is skipped
            self.group_error = f"{type(exc).__name__}: {exc}"
        return self.group_ok

    def max_over_ranks(self, values):
        if self.world == 1:
            return list(values)
        t = self.torch.tensor(list(values), device=self.device, dtype=self.torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return [float(x) for x in t]

    def agree_max(self, n: int) -> int:
        return int(self.max_over_ranks([float(n)])[0])

    def close(self):
        if self.group_ok:
            if self.world > 1:
                self.dist.barrier()
            self.dist.destroy_process_group()
            self.group_ok = False


def _timed_eager(torch, fn, n, barrier):
    """Mean milliseconds of `fn` over n calls (CUDA events on the current stream); fn synchronises itself."""
    for _ in range(3):
        fn()
    if barrier:
        barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(n):
        fn()
    e1.record()
    e1.synchronize()
    return e0.elapsed_time(e1) / n


def _roofline(achieved, nbytes, kernel):
    peak, peak_kind = measured_peak()
    return {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
            "traffic": None, "peak_source": f"of {peak_kind}", "kernel": kernel, "algorithmic_bytes_per_launch": nbytes}


def _parity_verdict(err, ref_max):
    return {"max_abs_err": err, "max_abs_ref": ref_max, "within_2e-3_and_1e-2_rel": bool(err <= 2e-3 and err <= 1e-2 * ref_max)}


# ----------------------------------------------------------------------------- pack workload
def measure_pack(ctx, steps):
    """Prefill quantise+pack of 32768 tokens x 4 KV heads x 128 dims (K along tokens, V along dims) at
    2/4/8 bits over rotating input buffers larger than L2, and the lazy cold-tier cooling step
    (64 aged tokens -> top 32 by value norm, 4-bit).  value = 2-bit K+V pack GB/s."""
    torch, dev = ctx.torch, ctx.device
    from phasekv_b200 import workloads
    from phasekv_b200.cold_tier import select_and_pack_cold
    from phasekv_b200.kernels import packing
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
        ms = time_graph(torch, step, steps // 10 + 1, 3)  # graph replay: no Python between the launches
        us = ms * 1e3 / copies
        nbytes = 2 * (S * s.num_kv_heads * s.head_dim) * 2 + 2 * S * s.num_kv_heads * (s.head_dim * bits // 8 + 4 * s.head_dim // GROUP)
        res[str(bits)] = {"us_per_kv_pack": us, "GBps": nbytes / us / 1e3, "frac_of_peak": nbytes / us / 1e3 / peak,
                          "algorithmic_bytes": nbytes}
    del ks, vs
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
    torch.cuda.empty_cache()
    return {"metric": "quantize_pack_GBps", "value": res["2"]["GBps"], "unit": UNIT, "n_gpus": 1, "steps": steps,
            "warmup": 3, "higher_is_better": True, "data": "synthetic",
            "config": {"workload": "prefill quantise+pack, 32768 tok x 4 KV heads x 128 dims, K along tokens + V along dims, gs 32",
                       "l2_policy": "rotating inputs larger than L2"},
            "by_bits": res, "peak": peak, "peak_source": f"of {peak_kind}",
            "cold_cooling_us": e0.elapsed_time(e1) * 1e3 / len(bufs),
            "cold_config": "64 aged of 192 hot tokens -> keep 32, 4-bit, 4 KV heads, one launch (python call included)"}


# ----------------------------------------------------------------------------- batched serving workload
def _pch(length):
    p, c, h = length
    return p, PROMPT_BITS, c, COLD_BITS, h


def measure_serving(ctx, steps, warmup, layers, batch):
    """Batched serving decode: `batch` sequences of 8192 prompt tokens @2-bit + 512 cold @4-bit + 128 hot
    (each length jittered by +-25 %), all layers, sharded by batch over the GPUs with no collective (strong
    scaling: the batch is fixed).  A step is one decode token: per layer ONE batched split-K launch + one merge
    launch over this rank's sequences.  Also timed: the same step as a loop of batch-1 calls over the sequences,
    which is how the reference's batch-1 entry point would be driven.  Parity inside the run: rows of the batched
    output of layer 0 (first, shortest and longest sequence of this rank) against the batch-1 entry point."""
    torch, device, world, rank = ctx.torch, ctx.device, ctx.world, ctx.rank
    from phasekv_b200 import _native as nv
    from phasekv_b200 import sharding, workloads
    from phasekv_b200.kernels import attention_cuda as attn
    s = workloads.QWEN2_5_7B
    lengths = workloads.jittered_lengths(0, batch, 8192, 512, 128, hot_capacity=192)
    mine = sharding.batch_shard(batch, world, rank)
    plans, qs, tiers_all = [], [], []
    for layer in range(layers):
        tiers, q = [], []
        for i in mine:
            p, c, h = lengths[i]
            t, qq = workloads.gpu_three_tier(s, p, PROMPT_BITS, c, COLD_BITS, h, workloads.layer_seed(1, layer, i), device)
            tiers.append(t), q.append(qq)
        plans.append(attn.BatchDecodePlan(tiers, s.num_q_heads))
        qs.append(torch.stack(q))
        tiers_all.append(tiers if layer < 2 else None)  # the per-sequence loop and the parity check use two layers
    job_bytes = layers * sum(workloads.decode_algorithmic_bytes(s, p, PROMPT_BITS, c, COLD_BITS, h, GROUP, GROUP)
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
    clocks = ClockSampler(ctx.local_rank)
    ms = time_graph(torch, step, steps, max(warmup, 3), ctx.barrier, sampler=clocks)

    # parity inside the run: batched rows against the batch-1 entry point on the same tensors
    order = sorted(range(len(mine)), key=lambda j: lengths[mine[j]][0])
    err, ref_max = 0.0, 0.0
    for j in sorted({0, order[0], order[-1]}):
        single = attn.fused_phasekv_decode(qs[0][j], tiers_all[0][j], s.num_q_heads).float()
        err = max(err, float((outs[0][j].float() - single).abs().max()))
        ref_max = max(ref_max, float(single.abs().max()))

    # end to end through the Python entry point: q from pinned host memory, outputs back to the host
    q_host = [q.cpu().pin_memory() for q in qs]
    o_host = [torch.empty_like(q).pin_memory() for q in q_host]
    q_dev = [torch.empty_like(q) for q in qs]

    def e2e_step():
        for i, p in enumerate(plans):
            q_dev[i].copy_(q_host[i], non_blocking=True)
            o_host[i].copy_(attn.fused_phasekv_decode_batched(q_dev[i], p, s.num_q_heads), non_blocking=True)
        torch.cuda.current_stream().synchronize()
    ms_e2e = _timed_eager(torch, e2e_step, max(3, min(steps, 20)), ctx.barrier)

    # the same step as a loop of batch-1 calls (2 layers, scaled)
    loop_layers = min(2, layers)

    def loop_step():
        for layer in range(loop_layers):
            for i, t in enumerate(tiers_all[layer]):
                attn.fused_phasekv_decode(qs[layer][i], t, s.num_q_heads)
    ms_loop = time_graph(torch, loop_step, 10, 3) * layers / loop_layers

    ms, ms_e2e, ms_loop, err, ref_max = ctx.max_over_ranks([ms, ms_e2e, ms_loop, err, ref_max])
    achieved = rank_layer_bytes / (ms / layers * 1e-3) / 1e9
    h2d = sum(q.numel() * 2 for q in qs) * world
    del plans, qs, tiers_all, outs, ws
    torch.cuda.empty_cache()
    return {
        "metric": METRIC, "value": job_bytes / (ms * 1e-3) / 1e9, "unit": UNIT, "n_gpus": world, "steps": steps,
        "warmup": max(warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f16 codes x f16, f32 accumulate", "data": "synthetic",
        "config": {"workload": f"qwen2.5-7b batched serving decode, {layers} layers, batch {batch} "
                               "(8192 prompt tok @2-bit KIVI + 512 cold @4-bit + 128 hot fp16 per sequence, lengths "
                               "jittered +-25 %), 28q/4kv heads, hd 128, gs 32",
                   "batch": batch, "layers": layers, "sequences_per_gpu": len(mine),
                   "l2_policy": "inputs larger than L2 (distinct KV per layer and sequence)",
                   "parallelism": "batch-sharded, no collective"},
        "us_per_layer": ms / layers * 1e3, "tokens_per_s": batch / (ms * 1e-3),
        "e2e": {"value": job_bytes / (ms_e2e * 1e-3) / 1e9, "unit": UNIT, "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": h2d, "ms_per_step": ms_e2e},
        "gpu_launches": 2 * layers * steps,
        "per_sequence_loop": {"ms_per_step": ms_loop, "speedup_of_batched": ms_loop / ms,
                              "sample": f"{loop_layers} of {layers} layers, scaled"},
        "parity_vs_batch1_entry": _parity_verdict(err, ref_max),
        "roofline": _roofline(achieved, rank_layer_bytes, "batched split-K decode + merge, per layer, rank 0's share"),
        "clocks": clocks.summary(),
    }


# ----------------------------------------------------------------------------- long-context workload
LONG_PROMPT, LONG_COLD = 262144, 1024


def measure_longctx(ctx, steps, warmup, layers):
    """Long-context batch-1 decode: 262144 prompt tokens @2-bit cut into one contiguous shard per GPU, 1024 cold
    tokens @4-bit and 128 hot tokens on rank 0.  Per layer every rank computes the un-normalised partial of its
    shard and one kernel pushes it into every peer's memory over NVLink, waits for the peers' partials and merges
    them (no collective library); the NCCL all-gather variant is timed beside it.  Strong scaling: the context
    is fixed.  The layers are chained through the stream as they would be in a model.  Layer 0 is cut out of one
    global packed tensor that every rank builds from the same seed, so that the sharded output of that layer can
    be checked, inside the run, against the unsharded entry point on rank 0."""
    torch, dist, device, world, rank = ctx.torch, ctx.dist, ctx.device, ctx.world, ctx.rank
    from phasekv_b200 import sharding, workloads
    from phasekv_b200.kernels import attention_cuda as attn
    from phasekv_b200.kernels.tiers import LayerTiers
    s = workloads.QWEN2_5_7B
    if not ctx.init_group():
        return {"error": "no process group: " + getattr(ctx, "group_error", "?")}
    start, end = sharding.sequence_bounds(LONG_PROMPT, world)[rank]
    exchange = sharding.PeerExchange(s.num_q_heads, s.head_dim, device, loopback=(world == 1), world=world, rank=rank)
    try:
        # layer 0: the same global tensors on every rank, this rank keeps its shard (and rank 0 the whole for the check)
        full, q0 = workloads.gpu_three_tier(s, LONG_PROMPT, PROMPT_BITS, LONG_COLD, COLD_BITS, HOT_LEN,
                                            workloads.layer_seed(2, 0, 0), device)
        shard0 = sharding.shard_kivi_segment(full.prompt.key, full.prompt.value, start, end)
        layer_inputs = [([shard0] + ([(c.key, c.value) for c in full.cold] if rank == 0 else []),
                         full.hot_k if rank == 0 else None, full.hot_v if rank == 0 else None, q0)]
        if rank != 0:
            full = None
        for layer in range(1, layers):
            t, q = workloads.gpu_three_tier(s, end - start, PROMPT_BITS, LONG_COLD if rank == 0 else 0, COLD_BITS,
                                            HOT_LEN if rank == 0 else 0, workloads.layer_seed(2, layer, rank), device)
            layer_inputs.append(([(t.prompt.key, t.prompt.value)] + [(c.key, c.value) for c in t.cold], t.hot_k, t.hot_v, q))
        p2p = [sharding.ShardedDecodeLayer(segs, hk, hv, s.num_q_heads, s.head_dim, device, exchange=exchange)
               for segs, hk, hv, _ in layer_inputs]
        nccl = [sharding.ShardedDecodeLayer(segs, hk, hv, s.num_q_heads, s.head_dim, device)
                for segs, hk, hv, _ in layer_inputs]
        qs = [x[3] for x in layer_inputs]
        layer_bytes = workloads.decode_algorithmic_bytes(s, LONG_PROMPT, PROMPT_BITS, LONG_COLD, COLD_BITS, HOT_LEN, GROUP, GROUP)
        rank_bytes = workloads.decode_algorithmic_bytes(s, end - start, PROMPT_BITS, LONG_COLD if rank == 0 else 0, COLD_BITS,
                                                        HOT_LEN if rank == 0 else 0, GROUP, GROUP)

        def step():
            for lay, q in zip(p2p, qs):
                lay.run(q)

        def step_nccl():
            for lay, q in zip(nccl, qs):
                lay.run(q)
        # every rank makes the same sequence of exchange calls; a rank that fell out of step shows up here
        def check_all_ranks(where):
            # the verdict is shared, so that every rank leaves (or stays) together
            if ctx.max_over_ranks([1.0 if exchange.timed_out() else 0.0])[0]:
                raise RuntimeError(f"a peer's partial did not arrive in time ({where}); the ranks are out of step")
        if ctx.barrier:
            ctx.barrier()  # building the layers takes the ranks different times; the exchange waits 250 ms at most
        step(), step_nccl()
        torch.cuda.synchronize()
        check_all_ranks("first eager step")
        diff = max(float((a.out.float() - b.out.float()).abs().max()) for a, b in zip(p2p, nccl))
        err, ref_max = 0.0, 0.0
        if rank == 0:
            want = attn.fused_phasekv_decode(q0, full, s.num_q_heads).float()
            err, ref_max = float((p2p[0].out.float() - want).abs().max()), float(want.abs().max())
        clocks = ClockSampler(ctx.local_rank)
        ms = time_graph(torch, step, steps, max(warmup, 3), ctx.barrier, sampler=clocks, agree_max=ctx.agree_max)
        torch.cuda.synchronize()
        check_all_ranks("graph replays")
        how = "cuda graph"
        try:
            ms_nccl = time_graph(torch, step_nccl, steps, max(warmup, 3), ctx.barrier)
        except Exception as exc:  # a collective that cannot be captured
            ms_nccl, how = 0.0, how + f"; NCCL variant not captured ({type(exc).__name__})"
        # end to end: q from pinned host memory per layer, merged output back to the host
        q_host = [q.cpu().pin_memory() for q in qs]
        o_host = [torch.empty_like(q).pin_memory() for q in q_host]
        q_dev = [torch.empty_like(q) for q in qs]

        def e2e_step():
            for i, lay in enumerate(p2p):
                q_dev[i].copy_(q_host[i], non_blocking=True)
                o_host[i].copy_(lay.run(q_dev[i]), non_blocking=True)
            torch.cuda.current_stream().synchronize()
        ms_e2e = _timed_eager(torch, e2e_step, max(3, min(steps, 20)), ctx.barrier)
        timed_out = exchange.timed_out()
        ms, ms_e2e, ms_nccl, err, ref_max, diff = ctx.max_over_ranks([ms, ms_e2e, ms_nccl, err, ref_max, diff])
        achieved = rank_bytes / (ms / layers * 1e-3) / 1e9
        io = layers * s.num_q_heads * s.head_dim * 2
        return {
            "metric": METRIC, "value": layer_bytes * layers / (ms * 1e-3) / 1e9, "unit": UNIT, "n_gpus": world,
            "steps": steps, "warmup": max(warmup, 3), "ms_per_step": ms, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f16 codes x f16, f32 accumulate", "data": "synthetic",
            "config": {"workload": f"qwen2.5-7b long-context batch-1 decode, {layers} layers x ({LONG_PROMPT} prompt tok "
                                   f"@2-bit KIVI sequence-sharded + {LONG_COLD} cold @4-bit + {HOT_LEN} hot fp16 on rank 0), "
                                   "28q/4kv heads, hd 128, gs 32",
                       "layers": layers, "prompt_tokens_per_gpu": end - start,
                       "l2_policy": "inputs larger than L2 (distinct KV per layer)",
                       "parallelism": f"sequence-sharded x{world}; per layer every rank pushes its partial "
                                      f"({s.num_q_heads * (s.head_dim + 2) * 4} B) into the peers' memory over NVLink and "
                                      "merges what arrived, inside one kernel (no collective library)", "timed_as": how},
            "us_per_layer": ms / layers * 1e3,
            "nccl_all_gather_variant": {"ms_per_step": ms_nccl or None, "max_abs_diff_of_outputs": diff},
            "exchange_wait_timed_out": timed_out,
            "parity_vs_unsharded_entry": _parity_verdict(err, ref_max),
            "e2e": {"value": layer_bytes * layers / (ms_e2e * 1e-3) / 1e9, "unit": UNIT, "h2d_bytes_per_step": io,
                    "d2h_bytes_per_step": io, "ms_per_step": ms_e2e},
            "gpu_launches": 2 * layers * steps,
            "roofline": _roofline(achieved, rank_bytes, "split-K decode of rank 0's shard + exchange/merge kernel, per layer"),
            "clocks": clocks.summary(),
        }
    finally:
        if ctx.barrier:
            try:
                ctx.barrier()
            except Exception:
                pass
        exchange.close()
        torch.cuda.empty_cache()


def _random_prefill(torch, device, layers, tokens, seed):
    import types
    g = torch.Generator().manual_seed(seed)
    dense = types.SimpleNamespace(key_cache=[], value_cache=[])
    for _ in range(layers):
        dense.key_cache.append(torch.randn(1, 4, tokens, 128, generator=g, dtype=torch.float16).to(device))
        dense.value_cache.append(torch.randn(1, 4, tokens, 128, generator=g, dtype=torch.float16).to(device))
    return dense


def measure_prompt_chunk(ctx, prompt_len=4096, chunk=64):
    """A chunk of new input tokens against one layer (7B geometry): all queries in one split-K + merge launch pair
    versus the reference's order, one append and one single-query call per token (qwen2_attention.py:99-106).
    Device time of ten rounds each, host work included (both are what a caller pays per layer)."""
    torch, device = ctx.torch, ctx.device
    from phasekv_b200.kernels.attention_cuda import fused_phasekv_chunk_decode, fused_phasekv_decode
    from phasekv_b200.phasekv_cache import PhaseKVCache
    cache = PhaseKVCache.from_dense_prefill(_random_prefill(torch, device, 1, prompt_len, 5), prompt_len=prompt_len)
    for _ in range(100):
        k = torch.randn(1, 4, 1, 128, device=device, dtype=torch.float16)
        cache.append_hot(0, k, k)
        cache.finish_decode_step()
    cache.begin_prompt_chunk(chunk)
    ks = torch.randn(1, 4, chunk, 128, device=device, dtype=torch.float16)
    q = torch.randn(chunk, 28, 128, device=device, dtype=torch.float16)
    tiers = cache.layer_tiers(0)
    start = tiers.hot_len

    def token_loop():
        tiers.hot_len = start
        outs = []
        for i in range(chunk):
            cache.append_prompt_token(0, ks[:, :, i:i + 1], ks[:, :, i:i + 1])
            outs.append(fused_phasekv_decode(q[i], tiers, 28))
        return torch.stack(outs)

    def one_launch_pair():
        tiers.hot_len = start + chunk
        return fused_phasekv_chunk_decode(q, tiers, 28)
    res = {"config": {"workload": "prompt chunk attention, one layer", "prompt_tokens": prompt_len, "chunk_tokens": chunk,
                      "cold_steps": len(tiers.cold)}}
    for name, fn in (("token_loop_us", token_loop), ("one_launch_pair_us", one_launch_pair)):
        res[name] = _timed_eager(torch, fn, 10, ctx.barrier) * 1e3
    res["max_abs_diff"] = float((token_loop().float() - one_launch_pair().float()).abs().max())
    res["speedup"] = res["token_loop_us"] / res["one_launch_pair_us"]
    return res


def measure_cold_arena(ctx, prompt_len, layers, generated=1000):
    """Decode over a cache that has generated `generated` tokens with the reference's defaults (window 32, batch 16,
    half kept: a cooling step of 8 tokens every 16 tokens).  `arena`: the steps of a layer are slots of one arena and
    are read as ONE masked segment; `per_step`: the same steps as tensors of their own, one descriptor each (what a
    list of segments costs); `single_segment`: as many cold tokens in one ordinary segment (the lower bound)."""
    torch, device = ctx.torch, ctx.device
    from dataclasses import replace

    from phasekv_b200.kernels import packing
    from phasekv_b200.kernels.attention_cuda import fused_phasekv_decode
    from phasekv_b200.kernels.tiers import LayerTiers, PackedKVSegment
    from phasekv_b200.phasekv_cache import PhaseKVCache
    cache = PhaseKVCache.from_dense_prefill(_random_prefill(torch, device, layers, prompt_len, 6), prompt_len=prompt_len)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(generated):
        k = torch.randn(1, 4, 1, 128, device=device, dtype=torch.float16)
        for l in range(layers):
            cache.append_hot(l, k, k)
        cache.finish_decode_step()
    torch.cuda.synchronize()
    host_ms = (time.perf_counter() - t0) / generated * 1e3
    q = torch.randn(28, 128, device=device, dtype=torch.float16)

    def own(pt):
        return replace(pt, packed=pt.packed.clone(), scale=pt.scale.clone(), mins=pt.mins.clone())

    def per_step(t):
        return LayerTiers(prompt=t.prompt, cold=[PackedKVSegment(own(s.key), own(s.value)) for s in t.cold],
                          hot_k=t.hot_k, hot_v=t.hot_v, hot_len=t.hot_len)

    def single(t):
        k = torch.randn(1, 4, sum(s.length for s in t.cold), 128, device=device, dtype=torch.float16)
        seg = PackedKVSegment(packing.quantize_pack(k, COLD_BITS, -2, GROUP), packing.quantize_pack(k, COLD_BITS, -1, GROUP))
        return LayerTiers(prompt=t.prompt, cold=[seg], hot_k=t.hot_k, hot_v=t.hot_v, hot_len=t.hot_len)
    first = cache.layer_tiers(0)
    res = {"config": {"workload": "decode after generation, cold tier in arenas", "prompt_tokens": prompt_len,
                      "layers": layers, "generated_tokens": generated, "cold_steps": len(first.cold),
                      "cold_tokens": first.cold_len, "hot_tokens": first.hot_len},
           "cache_update_host_ms_per_token": host_ms}
    for name, view in (("arena", lambda t: t), ("per_step", per_step), ("single_segment", single)):
        tl = [view(cache.layer_tiers(l)) for l in range(layers)]

        def run():
            for t in tl:
                fused_phasekv_decode(q, t, 28)
        run()  # settles the descriptors (the first launch over a segment is flagged fresh)
        res[name + "_us_per_layer"] = time_graph(torch, run, 20, 3) / layers * 1e3
    res["arena_over_single_segment"] = res["arena_us_per_layer"] / res["single_segment_us_per_layer"]
    return res


def measure_adapter_layer(ctx, prompt_len=32768, chunk=64):
    """One attention layer of Qwen2.5-7B geometry (hidden 3584, 28 query / 4 KV heads, random weights) over a PhaseKVCache,
    through the adapter: projections, rotary embedding, append and attention.  `fused` is this package's adapter
    (one rotary+convert+append launch, one launch pair of attention, also for a chunk of new prompt tokens);
    `reference_order` performs the same layer the way the reference's adapter does (qwen2_attention.py:79-109):
    torch rotary embedding, three conversions, then per token an append and a single-query attention call.
    Wall-clock microseconds per layer call, host work included (the reference reports a 22 ms/token launch floor
    for a whole model; this is the per-layer share of that floor)."""
    torch, device = ctx.torch, ctx.device
    try:
        from transformers import Qwen2Config
        from transformers.models.qwen2.modeling_qwen2 import Qwen2Attention, Qwen2RotaryEmbedding, apply_rotary_pos_emb
    except Exception as exc:  # transformers is optional
        return {"unavailable": f"transformers: {exc}"}
    from phasekv_b200.kernels.attention_cuda import fused_phasekv_decode
    from phasekv_b200.phasekv_cache import PhaseKVCache
    from phasekv_b200.qwen2_attention import PhaseKVQwen2Attention
    cfg = Qwen2Config(vocab_size=128, hidden_size=3584, intermediate_size=64, num_hidden_layers=1, num_attention_heads=28,
                      num_key_value_heads=4, max_position_embeddings=prompt_len + 4096, attention_dropout=0.0,
                      attn_implementation="eager")
    torch.manual_seed(0)
    attn = PhaseKVQwen2Attention(Qwen2Attention(cfg, 0).to(device, torch.float16).eval()).eval()
    rotary = Qwen2RotaryEmbedding(cfg).to(device)

    def fresh_cache():
        cache = PhaseKVCache.from_dense_prefill(_random_prefill(torch, device, 1, prompt_len, 9), prompt_len=prompt_len)
        g = torch.Generator(device=device).manual_seed(11)   # both variants see the same cache and inputs
        for _ in range(40):
            k = torch.randn(1, 4, 1, 128, device=device, dtype=torch.float16, generator=g)
            cache.append_hot(0, k, k)
            cache.finish_decode_step()
        return cache, g

    def fused(cache, hidden, positions):
        pe = rotary(hidden, positions)
        return attn(hidden, position_embeddings=pe, past_key_values=cache, use_cache=True)[0]

    def reference_order(cache, hidden, positions):
        base = attn.original
        n = hidden.shape[1]
        q = base.q_proj(hidden).view(1, n, 28, 128).transpose(1, 2)
        k = base.k_proj(hidden).view(1, n, 4, 128).transpose(1, 2)
        v = base.v_proj(hidden).view(1, n, 4, 128).transpose(1, 2)
        cos, sin = rotary(hidden, positions)
        q, k = apply_rotary_pos_emb(q, k, cos, sin)
        q, k, v = q.to(torch.float16), k.to(torch.float16), v.to(torch.float16)
        append = cache.append_prompt_token if cache.prompt_chunk_len else cache.append_hot
        tiers = cache.layer_tiers(0)
        outs = []
        for i in range(n):
            append(0, k[:, :, i:i + 1, :], v[:, :, i:i + 1, :])
            outs.append(fused_phasekv_decode(q[0, :, i, :], tiers, 28))
        return base.o_proj(torch.stack(outs, 0).reshape(1, n, 3584))
    res = {"config": {"workload": "one attention layer through the model adapter, Qwen2.5-7B geometry", "prompt_tokens": prompt_len,
                      "chunk_tokens": chunk, "timed_as": "wall clock per call incl. host work: best of three blocks of 20 decode steps; mean of 5 chunks"}}
    with torch.inference_mode():
        for name, fn in (("fused", fused), ("reference_order", reference_order)):
            cache, g = fresh_cache()
            hidden = torch.randn(1, 1, 3584, device=device, dtype=torch.float16, generator=g)
            blocks = []
            for block in range(4):      # the first block warms up (lazy initialisation, the first cooling step's arena)
                torch.cuda.synchronize()
                t0 = time.perf_counter()
                for rep in range(20):
                    pos = torch.tensor([[cache.true_seq_length]], device=device)
                    last = fn(cache, hidden, pos)
                    cache.finish_decode_step()
                torch.cuda.synchronize()
                blocks.append((time.perf_counter() - t0) / 20 * 1e6)
            res[f"decode_{name}_us"] = min(blocks[1:])
            last_decode = last.float()
            hidden = torch.randn(1, chunk, 3584, device=device, dtype=torch.float16, generator=g)
            for rep in range(7):
                pos = torch.arange(cache.true_seq_length, cache.true_seq_length + chunk, device=device).unsqueeze(0)
                if rep == 2:
                    torch.cuda.synchronize()
                    t0 = time.perf_counter()
                cache.begin_prompt_chunk(chunk)
                out = fn(cache, hidden, pos)
                cache.finish_prompt_chunk()
            torch.cuda.synchronize()
            res[f"chunk_{name}_us"] = (time.perf_counter() - t0) / 5 * 1e6
            res[f"_{name}"] = (last_decode, out.float())
        res["max_abs_diff_decode"] = float((res["_fused"][0] - res["_reference_order"][0]).abs().max())
        res["max_abs_diff_chunk"] = float((res["_fused"][1] - res["_reference_order"][1]).abs().max())
        del res["_fused"], res["_reference_order"]
    res["decode_speedup"] = res["decode_reference_order_us"] / res["decode_fused_us"]
    res["chunk_speedup"] = res["chunk_reference_order_us"] / res["chunk_fused_us"]
    return res


def measure_graphed_step(ctx, prompt_len, layers, tokens=200):
    """A whole decode step of the attention path (per layer: rotary embedding + float16 conversion + append, then
    attention over all tiers; at the end of the step the reference's lazy cooling) for `tokens` generated tokens:
    `graphed`: the step's launches captured once with device-resident lengths and replayed per token
    (phasekv_b200.graph_step); `eager`: the same through append_rotated + fused_phasekv_decode per layer.
    Wall clock per token, host work and cooling steps included; q, k, v of the token are already on the device."""
    torch, device = ctx.torch, ctx.device
    from phasekv_b200.graph_step import GraphedDecodeStep
    from phasekv_b200.kernels.attention_cuda import fused_phasekv_decode
    from phasekv_b200.phasekv_cache import PhaseKVCache
    g = torch.Generator(device=device).manual_seed(3)
    q = torch.randn(layers, 28, 128, device=device, dtype=torch.float16, generator=g)
    k = torch.randn(layers, 4, 128, device=device, dtype=torch.float16, generator=g)
    v = torch.randn(layers, 4, 128, device=device, dtype=torch.float16, generator=g)
    cos = torch.ones(128, device=device)
    sin = torch.zeros(128, device=device)
    res = {"config": {"workload": "decode step of the attention path incl. KV append and lazy cooling, all layers",
                      "prompt_tokens": prompt_len, "layers": layers, "generated_tokens": tokens,
                      "timed_as": "wall clock per token incl. host work"}}
    outs = {}
    for name in ("graphed", "eager"):
        cache = PhaseKVCache.from_dense_prefill(_random_prefill(torch, device, layers, prompt_len, 4), prompt_len=prompt_len)
        runner = GraphedDecodeStep(cache, 28) if name == "graphed" else None

        def token():
            if runner is not None:
                return runner.step(q, k, v, cos, sin)
            out = [fused_phasekv_decode(cache.append_rotated(l, q[l:l + 1], k[l:l + 1], v[l:l + 1], cos[None], sin[None])[0],
                                        cache.layer_tiers(l), 28) for l in range(layers)]
            cache.finish_decode_step()
            return torch.stack(out)
        for _ in range(20):
            token()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(tokens):
            last = token()
        torch.cuda.synchronize()
        res[f"{name}_us_per_token"] = (time.perf_counter() - t0) / tokens * 1e6
        outs[name] = last.float().clone()
        if runner is not None:
            res["graph_captures"] = runner.captures
        res["cold_steps"] = len(cache.layer_tiers(0).cold)
        del cache, runner
        torch.cuda.empty_cache()
    res["max_abs_diff"] = float((outs["graphed"] - outs["eager"]).abs().max())
    res["speedup"] = res["eager_us_per_token"] / res["graphed_us_per_token"]
    return res


def measure_per_token_layout(ctx, layers):
    """The per-token layout of the reference's published micro-benchmark (K and V both quantised along head_dim,
    4 KV heads x S x 128, 28 query heads) on its own tensor-core kernel: distinct layers (more than the L2 holds)
    replayed from a CUDA graph, library-sized grid.  Bytes = packed K + V."""
    torch, device = ctx.torch, ctx.device
    from phasekv_b200.kernels import packing as pk
    from phasekv_b200.kernels.attention_cuda import decode_attention_packed_splitk
    peak, _ = measured_peak()
    res = {"config": {"workload": "per-token layout decode attention, 28q/4kv heads, hd 128, gs 32", "timed_as": "cuda graph",
                      "l2_policy": "distinct KV per layer, at least 300 MB resident"}}
    q = torch.randn(28, 128, device=device, dtype=torch.float16)
    for bits in (2, 4):
        for S in (4096, 32768, 131072):
            per_layer = 2 * 4 * S * (128 * bits // 8 + 16)
            n_layers = max(layers, int(3e8 // per_layer) + 1)
            g = torch.Generator(device=device).manual_seed(S + bits)
            kv = []
            for _ in range(n_layers):
                x = torch.randn(4, S, 128, device=device, dtype=torch.float16, generator=g)
                kv.append((pk.quantize_pack(x, bits, -1, 32), pk.quantize_pack(x.flip(1).contiguous(), bits, -1, 32)))
                del x

            def run():
                for a, b in kv:
                    decode_attention_packed_splitk(q, a, b, 28, num_splits=None)
            ms = time_graph(torch, run, 20, 3)
            us = ms / n_layers * 1e3
            res[f"{bits}bit_{S}"] = {"us_per_layer": us, "GBps": per_layer / us / 1e3, "frac_of_peak": per_layer / us / 1e3 / peak,
                                     "layers_resident": n_layers}
            del kv
            torch.cuda.empty_cache()
    return res


def measure_general_kernel(ctx):
    """Shapes the tensor-core kernels do not take run on the general kernel: the Qwen2-0.5B attention shape of the
    CPU-plumbing configuration (14 query / 2 KV heads, head_dim 64; prompt 2-bit with value groups of 64, 128 cold
    tokens at 4 bits, 64 float16 tokens) at its own 1024 prompt tokens and at 32768.  Distinct layers replayed from a
    CUDA graph (the parity of this configuration is a test, tests/test_decode_gpu.py)."""
    torch, device = ctx.torch, ctx.device
    from phasekv_b200 import workloads
    from phasekv_b200.kernels import packing as pk
    from phasekv_b200.kernels.attention_cuda import fused_phasekv_decode
    from phasekv_b200.kernels.tiers import LayerTiers, PackedKVSegment
    shape = workloads.QWEN2_0_5B
    peak, _ = measured_peak()
    res = {"config": {"workload": "qwen2-0.5b attention shape on the general kernel (hd 64, gsK 32 / gsV 64)",
                      "timed_as": "cuda graph", "l2_policy": "distinct KV per layer, at least 300 MB resident at 32768"}}
    for S in (1024, 32768):
        nbytes = workloads.decode_algorithmic_bytes(shape, S, 2, 128, 4, 64, 32, 64)
        n_layers = 24 if S == 1024 else max(24, int(3e8 // nbytes) + 1)
        gen = torch.Generator(device=device).manual_seed(S)
        tiers = []
        for _ in range(n_layers):
            def packed(tokens, bits):
                k = torch.randn(1, 2, tokens, 64, device=device, dtype=torch.float16, generator=gen)
                return PackedKVSegment(pk.quantize_pack(k, bits, -2, 32), pk.quantize_pack(k.flip(2).contiguous(), bits, -1, 64))
            hot = torch.randn(1, 2, 64, 64, device=device, dtype=torch.float16, generator=gen)
            tiers.append(LayerTiers(prompt=packed(S, 2), cold=[packed(128, 4)], hot_k=hot, hot_v=hot.flip(2).contiguous(), hot_len=64))
        q = torch.randn(14, 64, device=device, dtype=torch.float16, generator=gen)

        def run():
            for t in tiers:
                fused_phasekv_decode(q, t, 14)
        run()
        us = time_graph(torch, run, 20, 3) / n_layers * 1e3
        res[str(S)] = {"us_per_layer": us, "GBps": nbytes / us / 1e3, "frac_of_peak": nbytes / us / 1e3 / peak,
                       "algorithmic_bytes": nbytes, "layers_resident": n_layers}
        del tiers
        torch.cuda.empty_cache()
    return res


def sharded_block(ctx, args):
    """The two configurations that shard over GPUs (sequence-sharded long context, batch-sharded serving) and, on
    one GPU, the pack kernels, measured in the same process group after the headline.  A workload that fails
    reports its error instead of taking the headline down with it."""
    steps = max(3, min(args.steps, 20))
    block = {}
    for name, fn in (("longctx", lambda: measure_longctx(ctx, steps, args.warmup, args.layers)),
                     ("serving", lambda: measure_serving(ctx, steps, args.warmup, args.layers, args.batch))):
        try:
            res = fn()
        except Exception as exc:
            res = {"error": f"{type(exc).__name__}: {exc}"}
        keep = ("ms_per_step", "us_per_layer", "value", "unit", "scaling", "e2e", "clocks", "config", "roofline",
                "exchange_wait_timed_out", "nccl_all_gather_variant", "parity_vs_unsharded_entry",
                "parity_vs_batch1_entry", "per_sequence_loop", "tokens_per_s", "gpu_launches", "error")
        block[name] = {k: v for k, v in res.items() if k in keep}
    if ctx.world == 1:
        try:
            res = measure_pack(ctx, steps)
            block["pack"] = {k: res[k] for k in ("by_bits", "cold_cooling_us", "cold_config", "config")}
        except Exception as exc:
            block["pack"] = {"error": f"{type(exc).__name__}: {exc}"}
        for name, fn in (("prompt_chunk", lambda: [measure_prompt_chunk(ctx, 4096, 64), measure_prompt_chunk(ctx, args.prompt, 64)]),
                         ("cold_arena", lambda: measure_cold_arena(ctx, args.prompt, args.layers)),
                         ("adapter_layer", lambda: measure_adapter_layer(ctx, args.prompt, 64)),
                         ("graphed_step", lambda: measure_graphed_step(ctx, args.prompt, args.layers)),
                         ("per_token_layout", lambda: measure_per_token_layout(ctx, args.layers)),
                         ("general_kernel", lambda: measure_general_kernel(ctx))):
            try:
                block[name] = fn()
            except Exception as exc:
                block[name] = {"error": f"{type(exc).__name__}: {exc}"}
            ctx.torch.cuda.empty_cache()
    return block


# ----------------------------------------------------------------------------- main arm
def measure_decode(ctx, args):
    torch, dist, device, world, rank = ctx.torch, ctx.dist, ctx.device, ctx.world, ctx.rank
    ls = LayerSet(torch, device, args.prompt, args.layers, seed=1234 + rank)
    native = NativeStep(torch, ls, device)
    torch.cuda.synchronize()
    clocks = ClockSampler(ctx.local_rank)
    ms = time_graph(torch, native.run, args.steps, max(args.warmup, 3), ctx.barrier, sampler=clocks)
    ms_e2e, ms_e2e_py, h2d, d2h, o_host = time_e2e(torch, ls, native, device, max(3, min(args.steps, 20)), 3)
    ms, ms_e2e, ms_e2e_py = ctx.max_over_ranks([ms, ms_e2e, ms_e2e_py])
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
                "ms_per_step": ms_e2e,
                "called_as": "pkv_decode_attention per layer (C ABI, no graph), q of the step copied from pinned host "
                             "memory, outputs copied back, host waits",
                "python_entry_ms_per_step": ms_e2e_py,
                "python_entry_value": step_bytes / (ms_e2e_py * 1e-3) / 1e9},
        "gpu_launches": native.launches_per_step * args.steps,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": NCU_TRAFFIC_BYTES_PER_LAUNCH.get(args.prompt), "traffic_source": NCU_TRAFFIC_SOURCE,
                     "peak_source": f"of {peak_kind}",
                     "kernel": "split-K decode + merge, per layer", "algorithmic_bytes_per_launch": ls.bytes_per_layer},
        "clocks": clocks.summary(),
    }
    if rank == 0 and world == 1 and not args.no_extras:
        # latency of ONE call issued on an idle GPU and waited for (not a replay): launch, two kernels, host wake-up
        one = []
        for i in range(25):
            arr, n = native.calls[i % len(native.calls)]
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            native.nv.check(native.L.pkv_decode_attention(
                ls.q[0].data_ptr(), arr, n, ls.shape.num_q_heads, ls.shape.num_kv_heads, ls.shape.head_dim,
                1.0 / (ls.shape.head_dim ** 0.5), native.sms, native.ws.data_ptr(), native.ws.numel(),
                native.out[0].data_ptr(), None, None, None, native.nv.stream_of(device)))
            torch.cuda.synchronize()
            one.append((time.perf_counter() - t0) * 1e6)
        line["single_call_latency_us"] = sorted(one[5:])[len(one[5:]) // 2]
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
        ref = oracle.segments_decode_reference(q, segs, hk, hv, s.num_q_heads).float()
        err = float((out - ref).abs().max())
        line["parity"] = {"max_abs_err_vs_oracle": err, "max_abs_ref": float(ref.abs().max()),
                          "within_2e-3_and_1e-2_of_max_ref": err <= 2e-3 and err <= 1e-2 * float(ref.abs().max()),
                          "elementwise_atol_2e-3_rtol_1e-2": bool(torch.allclose(out, ref, atol=2e-3, rtol=1e-2)),
                          "elementwise_atol_3e-4_rtol_1e-3": bool(torch.allclose(out, ref, atol=3e-4, rtol=1e-3))}
        # CPU baseline on a bounded sample
        n_cpu = 8
        sec, cores = time_cpu_layers(args.prompt, 1, n_cpu, 1)
        line["cpu_baseline"] = {"value": ls.bytes_per_layer / sec / 1e9, "unit": UNIT, "cores": cores, "kind": "port",
                                "sample": f"{n_cpu} single-layer calls of the CPU dequantise-then-attend at {args.prompt} prompt tokens",
                                "ms_per_layer": sec * 1e3}
        # FP16 attention on the same GPU
        del native, ls, tiers
        torch.cuda.empty_cache()
        sd = sdpa_baselines(torch, device, args.prompt, args.layers, 20, 3)
        if "gqa_aware_ms_per_step" in sd:
            sd["speedup_vs_gqa_aware"] = sd["gqa_aware_ms_per_step"] / ms
        sd["speedup_vs_ideal_fp16"] = sd["ideal_fp16_ms_per_step"] / ms
        if "expanded_ms_per_step" in sd:
            sd["speedup_vs_expanded"] = sd["expanded_ms_per_step"] / ms
        line["sdpa_fp16"] = sd
        torch.cuda.empty_cache()
        # context sweep 4K .. 128K
        from phasekv_b200 import workloads as _w
        sweep = {}
        for S in (4096, 8192, 16384, 32768, 131072):
            if S == args.prompt:
                sweep[str(S)] = {"us_per_layer": per_launch_ms * 1e3, "GBps": achieved, "frac_of_peak": achieved / peak}
                continue
            # as many distinct layers as it takes to keep more than the 126 MB L2 resident (at least 300 MB)
            per_layer = _w.decode_algorithmic_bytes(_w.QWEN2_5_7B, S, PROMPT_BITS, COLD_LEN, COLD_BITS, HOT_LEN, GROUP, GROUP)
            n_layers = max(args.layers, int(3e8 // per_layer) + 1)
            l2 = LayerSet(torch, device, S, n_layers, seed=99 + S)
            n2 = NativeStep(torch, l2, device)
            m2 = time_graph(torch, n2.run, 20, 3)
            a2 = l2.bytes_per_layer / (m2 / l2.layers * 1e-3) / 1e9
            sweep[str(S)] = {"us_per_layer": m2 / l2.layers * 1e3, "GBps": a2, "frac_of_peak": a2 / peak,
                             "layers_resident": n_layers, "kv_bytes_resident": l2.kv_bytes_resident}
            del l2, n2
            torch.cuda.empty_cache()
        line["contexts"] = sweep
    else:
        del native, ls
        torch.cuda.empty_cache()
    return line


def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
        return
    ctx = Ctx()
    try:
        if args.workload == "decode":
            if ctx.world > 1:
                ctx.init_group()
            line = measure_decode(ctx, args)
            if not args.no_sharded:
                line["sharded"] = sharded_block(ctx, args)
        elif args.workload == "pack":
            line = measure_pack(ctx, args.steps)
        elif args.workload == "serving":
            if ctx.world > 1:
                ctx.init_group()
            line = measure_serving(ctx, args.steps, args.warmup, args.layers, args.batch)
        else:
            line = measure_longctx(ctx, args.steps, args.warmup, args.layers)
        if ctx.rank == 0:
            print(json.dumps(line))
    finally:
        ctx.close()


if __name__ == "__main__":
    main()
