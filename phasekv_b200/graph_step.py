"""One decode step of a whole model's attention (KV write + attention of every layer) as a CUDA graph that stays
valid while the cache grows.

The reference's adapter pays its launch overhead per layer and per token (``results/phasekv_auto_decode.json``: about
22 ms per token on its GPU, most of it host time); its cache lives in Python lists and plain integers, so nothing it
launches can be replayed.  Here the two numbers that change from token to token — how many tokens the float16 tier
holds and how many cold slots are filled — are kept in device memory as well (``pkv_segment_t.seq_len_dev``, the
``slot_dev`` argument of ``pkv_rope_append``), so the launches of a step are captured ONCE:

    hot_len += 1
    for every layer:  rotary embedding + float16 conversion + append at slot hot_len - 1     (pkv_rope_append)
                      attention over prompt, extensions, the cold arena and the float16 tier   (pkv_decode_attention)

and every later token is one graph replay plus host bookkeeping.  The lazy cooling of aged tokens stays where the
reference has it, on the host's schedule between steps (``PhaseKVCache.finish_decode_step``): when it runs, it
rewrites the hot buffers and an arena slot in place and the two device-resident lengths are updated; the graph is
captured again only when a buffer it points at is replaced (a prompt chunk, an arena that had to grow).

Layouts: those the tensor-core kernel takes (head_dim 128, groups of 32, GQA group <= 8), batch 1, a cold tier that
lives in one arena per layer (what ``PhaseKVCache`` builds for these layouts).
"""
from __future__ import annotations

import ctypes
from typing import List

import torch

from . import _native as nv
from .cold_arena import ColdArena
from .kernels.attention_cuda import _cached_packed_segment, _device_sm_count
from .phasekv_cache import _ROPE_DTYPES, PhaseKVCache, _Phase


class GraphedDecodeStep:
    """``step(q, k, v, cos, sin)``: ``q [L, Hq, hd]``, ``k / v [L, Hkv, hd]`` (the projections of one token for all
    ``L`` layers, float16 or bfloat16), ``cos / sin [hd]`` of the token's position -> attention outputs float16
    ``[L, Hq, hd]``.  Equivalent to ``append_rotated`` + ``fused_phasekv_decode`` per layer followed by
    ``finish_decode_step()``.

    The attention of layer ``l`` does not depend on layer ``l - 1`` here: in a real model the projections of layer
    ``l`` need the output of layer ``l - 1``, so a model runner captures its own graph around ``capture_layer``-style
    calls; this class is the attention-only form (what a benchmark of the path, or a runner that batches the
    projections, uses) and the reference for how the pieces are wired."""

    def __init__(self, cache: PhaseKVCache, num_attention_heads: int, dtype: torch.dtype = torch.float16,
                 rope_dtype: torch.dtype = torch.float32):
        if dtype not in (torch.float16, torch.bfloat16) or rope_dtype not in _ROPE_DTYPES:
            raise ValueError("q/k/v must be float16 or bfloat16, cos/sin float16, bfloat16 or float32")
        first = cache.layers[0]
        if first.hot_k.shape[0] != 1:
            raise ValueError("a graphed decode step serves batch 1")
        self.cache, self.heads = cache, num_attention_heads
        self.hkv, self.hd = first.hot_k.shape[1], first.hot_k.shape[3]
        self.device = first.hot_k.device
        layers = len(cache.layers)
        dev = self.device
        self.q = torch.zeros(layers, num_attention_heads, self.hd, dtype=dtype, device=dev)
        self.k = torch.zeros(layers, self.hkv, self.hd, dtype=dtype, device=dev)
        self.v = torch.zeros_like(self.k)
        self.cos = torch.zeros(1, self.hd, dtype=rope_dtype, device=dev)
        self.sin = torch.zeros_like(self.cos)
        self.q_rot = torch.empty(layers, num_attention_heads, self.hd, dtype=torch.float16, device=dev)
        self.out = torch.empty_like(self.q_rot)
        self.lengths = torch.zeros(2, dtype=torch.int32, device=dev)   # [float16 tokens, cold tokens incl. slot padding]
        self._graph = None
        self._signature = None
        self.captures = 0

    # ------------------------------------------------------------------ what the captured launches point at
    def _ensure_arenas(self) -> List[ColdArena]:
        """Every layer gets the arena its next cooling step would create, so that the graph can point at it."""
        c = self.cache
        keep = max(1, round(c.decode_keep_ratio * c.lazy_g))
        arenas = []
        for layer in c.layers:
            runs = layer._cold_runs
            if not runs and not layer.cold:
                runs.append(ColdArena(layer.hot_k, c.cold_bits, c.group_size, keep))
            if len(runs) != 1 or runs[0].events != len(layer.cold) or not runs[0].decode_ready:
                raise ValueError("a graphed decode step needs the cold tier of every layer in one arena the tensor-core "
                                 "kernel can read (head_dim 128, groups of 32, cooling steps of one size)")
            arenas.append(runs[0])
        return arenas

    def _structure(self, arenas: List[ColdArena]):
        """Everything a captured pointer or capacity depends on."""
        return tuple((id(l.prompt), len(l.prompt_extensions), l.hot_k.data_ptr(), l.hot_v.data_ptr(), l.hot_k.shape[2],
                      a.k_packed.data_ptr(), a.max_events) for l, a in zip(self.cache.layers, arenas))

    def _host_lengths(self, arenas: List[ColdArena]):
        return self.cache.layers[0].hot_len, arenas[0].events * arenas[0].slot_tokens

    def _sync_lengths(self, arenas: List[ColdArena]) -> None:
        hot, cold = self._host_lengths(arenas)
        self.lengths.copy_(torch.tensor([hot, cold], dtype=torch.int32))

    def _capture(self, arenas: List[ColdArena]) -> None:
        c, dev, L = self.cache, self.device, nv.lib()
        sms = _device_sm_count(dev)
        hot_len_ptr = self.lengths.data_ptr()
        cold_len_ptr = hot_len_ptr + 4
        calls, keep_alive, need = [], [], 0
        for layer, arena in zip(c.layers, arenas):
            segs = []
            for segment in (layer.prompt, *layer.prompt_extensions):
                s, kp, _ = _cached_packed_segment(segment, None)
                segs.append(s), keep_alive.append(kp)
            cold = arena.descriptor()
            cold.seq_len = arena.max_events * arena.slot_tokens      # the capacity; what counts is read from the device
            cold.seq_len_dev = cold_len_ptr
            segs.append(cold)
            capacity = layer.hot_k.shape[2]
            segs.append(nv.Segment(layer.hot_k.data_ptr(), None, None, layer.hot_v.data_ptr(), None, None, capacity,
                                   capacity * self.hd, nv.PKV_SEG_FP16, 8, 8, 1, 1, 0, 0, 0, 0, 0, 0, hot_len_ptr))
            arr = (nv.Segment * len(segs))(*segs)
            size = ctypes.c_size_t(0)
            nv.check(L.pkv_decode_workspace_bytes(arr, len(segs), self.heads, self.hkv, self.hd, sms, ctypes.byref(size)))
            need = max(need, int(size.value))
            calls.append((arr, len(segs), layer))
        self._workspace = torch.empty(need, dtype=torch.uint8, device=dev)
        self._keep_alive = keep_alive
        self._sync_lengths(arenas)
        scale = 1.0 / (self.hd ** 0.5)

        def launches():
            self.lengths[0:1].add_(1)
            stream = nv.stream_of(dev)
            for l, (arr, n, layer) in enumerate(calls):
                nv.check(L.pkv_rope_append(
                    self.q[l].data_ptr(), self.k[l].data_ptr(), self.v[l].data_ptr(), _ROPE_DTYPES[self.q.dtype],
                    self.heads * self.hd, self.hkv * self.hd, self.hkv * self.hd,
                    self.cos.data_ptr(), self.sin.data_ptr(), _ROPE_DTYPES[self.cos.dtype], self.hd, 1, self.heads,
                    self.hkv, self.hd, self.q_rot[l].data_ptr(), layer.hot_k.data_ptr(), layer.hot_v.data_ptr(),
                    layer.hot_k.shape[2], -1, hot_len_ptr, stream))
                nv.check(L.pkv_decode_attention(self.q_rot[l].data_ptr(), arr, n, self.heads, self.hkv, self.hd, scale, sms,
                                                self._workspace.data_ptr(), self._workspace.numel(),
                                                self.out[l].data_ptr(), None, None, None, stream))

        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            launches()                       # lazy initialisation outside the capture (it appends a token: undone below)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                launches()
        torch.cuda.current_stream(dev).wait_stream(side)
        self._sync_lengths(arenas)           # the warm-up run counted a token that the cache does not hold
        self._graph, self._signature = graph, self._structure(arenas)
        self.captures += 1

    # ------------------------------------------------------------------ one token
    @torch.no_grad()
    def step(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
        c = self.cache
        if c._phase is not _Phase.IDLE:
            raise RuntimeError("a graphed decode step starts between steps: finish the decode step or the prompt chunk first")
        if c.layers[0].hot_len + 1 > c.layers[0].hot_k.shape[2]:
            raise RuntimeError("the hot tier is full")
        arenas = self._ensure_arenas()
        with torch.cuda.device(self.device):
            if self._graph is None or self._signature != self._structure(arenas):
                self._capture(arenas)
            self.q.copy_(q.reshape(self.q.shape)), self.k.copy_(k.reshape(self.k.shape)), self.v.copy_(v.reshape(self.v.shape))
            self.cos.copy_(cos.reshape(self.cos.shape)), self.sin.copy_(sin.reshape(self.sin.shape))
            self._graph.replay()
        # the host's view of what the replay did, then the reference's end of step (cooling when a batch has aged)
        for layer_idx, layer in enumerate(c.layers):
            layer.hot_len += 1
            c._written.add(layer_idx)
        c._phase = _Phase.DECODE_STEP
        events = arenas[0].events
        c.finish_decode_step()
        if arenas[0].events != events:   # a cooling step moved tokens from the float16 tier into the next cold slot
            with torch.cuda.device(self.device):
                self._sync_lengths(arenas)
        for arena in arenas:
            arena.launched_events = arena.events
        return self.out
