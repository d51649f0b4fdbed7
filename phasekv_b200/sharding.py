"""Multi-GPU partitioning of the decode path (one process per GPU, torch.distributed).

The reference is single-GPU.  Three partitions are offered:

* batch: sequences are independent, rank r owns sequences ``r, r + R, ...``; no collective;
* KV head: the GQA groups are independent, a rank owns a contiguous range of KV heads and writes a
  disjoint slice of the output heads; no collective;
* sequence (long context, batch 1): the read-only prompt tier is cut into R contiguous shards at
  multiples of 64 tokens, so that every shard is a self-contained ``PackedTensor`` whose bytes equal
  slices of the global one (group boundaries and byte boundaries are multiples of 32 and 4 tokens).
  Each rank computes the un-normalised partial ``(m, l, acc)`` of its shard (plus, on rank 0, the
  cold and hot tiers); the partials (``Hq * (hd + 2) * 4`` bytes per rank) are all-gathered and
  merged with the same log-sum-exp algebra as the split-K merge
  (attention_triton.py:257-266, 300-307 of the reference).
"""
from __future__ import annotations

from dataclasses import replace
from typing import List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

SHARD_ALIGN = 64  # tokens; multiple of the quantisation group (32) and of the codes per byte (4)


def batch_shard(num_sequences: int, world_size: int, rank: int) -> List[int]:
    """Indices of the sequences owned by ``rank``."""
    return list(range(rank, num_sequences, world_size))


def head_shard(num_kv_heads: int, world_size: int, rank: int) -> Tuple[int, int]:
    """[begin, end) KV heads of ``rank``; needs ``num_kv_heads % world_size == 0``."""
    if num_kv_heads % world_size:
        raise ValueError("KV heads must divide evenly over the ranks")
    per = num_kv_heads // world_size
    return rank * per, (rank + 1) * per


def sequence_bounds(seq_len: int, world_size: int, align: int = SHARD_ALIGN) -> List[Tuple[int, int]]:
    """Contiguous token ranges, one per rank, every boundary a multiple of ``align`` (the last range
    takes the ragged remainder; a rank may get an empty range when the sequence is short)."""
    if seq_len <= 0 or world_size <= 0:
        raise ValueError("sequence length and world size must be positive")
    units = -(-seq_len // align)
    per, extra = divmod(units, world_size)
    bounds, start = [], 0
    for r in range(world_size):
        n = (per + (1 if r < extra else 0)) * align
        end = min(seq_len, start + n)
        bounds.append((start, end))
        start = end
    return bounds


def shard_kivi_segment(key, value, start: int, end: int):
    """Token range ``[start, end)`` of a KIVI-packed pair (originals ``[B, Hkv, S, hd]``, K packed along
    tokens, V along head_dim) as a new self-contained pair.  ``start`` must be a multiple of 64."""
    if start % SHARD_ALIGN or not (0 <= start < end <= key.orig_shape[-2]):
        raise ValueError("shard must start on a multiple of 64 tokens and lie inside the segment")
    if key.axis != len(key.orig_shape) - 2 or value.axis != len(value.orig_shape) - 1:
        raise ValueError("K must be packed along tokens and V along head_dim")
    vpb, n = 8 // key.bits, end - start
    kgs = key.group_size
    if kgs <= 0 or SHARD_ALIGN % kgs:
        raise ValueError("the key group size must divide 64")
    shape = tuple(key.orig_shape[:-2]) + (n, key.orig_shape[-1])
    k = replace(key,
                packed=key.packed[..., start // vpb:-(-end // vpb)].contiguous(),
                scale=key.scale[..., start // kgs:-(-end // kgs)].contiguous(),
                mins=key.mins[..., start // kgs:-(-end // kgs)].contiguous(),
                orig_shape=shape, axis_len=n, group_size=min(kgs, n))
    v = replace(value,
                packed=value.packed[..., start:end, :].contiguous(),
                scale=value.scale[..., start:end, :].contiguous(),
                mins=value.mins[..., start:end, :].contiguous(),
                orig_shape=shape)
    return k, v


def gather_partials(m: torch.Tensor, l: torch.Tensor, acc: torch.Tensor,
                    group: Optional[dist.ProcessGroup] = None):
    """All-gather one partial per rank into stacked ``m, l [R, Hq]`` and ``acc [R, Hq, hd]``.

    One message per rank: the three tensors travel packed as ``[Hq, hd + 2]`` float32."""
    world = dist.get_world_size(group)
    packed = torch.cat([acc.float(), m.float().unsqueeze(-1), l.float().unsqueeze(-1)], dim=-1).contiguous()
    out = torch.empty((world,) + tuple(packed.shape), dtype=torch.float32, device=packed.device)
    dist.all_gather(list(out.unbind(0)), packed, group=group)  # supported by both nccl and gloo
    hd = acc.shape[-1]
    return out[..., hd].contiguous(), out[..., hd + 1].contiguous(), out[..., :hd].contiguous()


def empty_partial(num_q_heads: int, head_dim: int, device) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """The neutral element of the merge (a rank whose shard is empty contributes this)."""
    return (torch.full((num_q_heads,), float("-inf"), dtype=torch.float32, device=device),
            torch.zeros((num_q_heads,), dtype=torch.float32, device=device),
            torch.zeros((num_q_heads, head_dim), dtype=torch.float32, device=device))


class PeerExchange:
    """This rank's end of the peer-to-peer exchange used by the sequence-sharded decode: a buffer in this
    GPU's memory that every other rank of the node maps through CUDA IPC and writes its partial into.  One
    exchange serves all layers of a model (its calls are ordered by the stream).  With ``loopback=True`` no
    other process is involved: every peer slot is the local buffer (``world == 1`` is then a complete
    exchange; a larger ``world`` only exercises the bounded wait)."""

    def __init__(self, num_q_heads: int, head_dim: int, device, group: Optional[dist.ProcessGroup] = None,
                 loopback: bool = False, world: Optional[int] = None, rank: Optional[int] = None):
        import ctypes
        from . import _native as nv
        self.nv, self.device = nv, device
        self.world = world if world is not None else dist.get_world_size(group)
        self.rank = rank if rank is not None else dist.get_rank(group)
        self.handle = ctypes.c_void_p()
        mine = ctypes.create_string_buffer(64)
        with torch.cuda.device(device):
            nv.check(nv.lib().pkv_exchange_create(self.world, self.rank, num_q_heads, head_dim,
                                                  ctypes.byref(self.handle), mine))
            if loopback:
                nv.check(nv.lib().pkv_exchange_connect_loopback(self.handle))
            else:
                handles: List[Optional[bytes]] = [None] * self.world
                dist.all_gather_object(handles, mine.raw, group=group)
                nv.check(nv.lib().pkv_exchange_connect(self.handle, b"".join(handles)))
                dist.barrier(group=group)  # every rank has mapped every buffer before anyone pushes

    def set_spin_limit(self, polls: int) -> None:
        self.nv.check(self.nv.lib().pkv_exchange_set_spin_limit(self.handle, polls))

    def set_wait_us(self, microseconds: int) -> None:
        """Most microseconds a rank waits for its peers in one call (default 250 000).  Ranks that prepare their
        layers at different speeds should meet at a host barrier before the first call."""
        self.nv.check(self.nv.lib().pkv_exchange_set_wait_us(self.handle, microseconds))

    def check(self) -> None:
        """Raise if a wait of this rank has run out (synchronises the device).  After that the exchange
        answers every call with NaN rows at once; it has to be closed and rebuilt."""
        if self.timed_out():
            raise RuntimeError("phasekv_b200: a peer's partial did not arrive in time; the ranks of this exchange "
                               "are out of step (did every rank make the same sequence of calls?)")

    def timed_out(self) -> bool:
        """True once any wait of this rank has run out (synchronises the device)."""
        import ctypes
        flag = ctypes.c_int(0)
        with torch.cuda.device(self.device):
            self.nv.check(self.nv.lib().pkv_exchange_status(self.handle, ctypes.byref(flag)))
        return bool(flag.value)

    def close(self) -> None:
        if self.handle:
            with torch.cuda.device(self.device):
                torch.cuda.synchronize(self.device)
                self.nv.check(self.nv.lib().pkv_exchange_destroy(self.handle))
            self.handle = None


class ShardedDecodeLayer:
    """One layer of the sequence-sharded decode on this rank, with every buffer allocated up front so that
    a step is three launches: split-K decode of the local shard into a flat partial ``[acc Hq*hd | m Hq | l Hq]``
    (float32), one all-gather of that message (``Hq * (hd + 2) * 4`` bytes per rank), and one merge that
    reads the gathered partials in place (``pkv_merge_partials_strided``).

    ``segments``: this rank's ``(key, value)`` pairs with batch dim 1 (its shard of the prompt tier and, on
    one rank, the cold segments); ``hot_k``/``hot_v``: ``[1, Hkv, hot, hd]`` on the rank that owns the hot
    tier, else ``None``.  A rank without any tokens contributes the neutral partial.

    With ``exchange`` (a :class:`PeerExchange`) the all-gather and the merge become part of ONE kernel that
    pushes the partial into the peers' memory over NVLink and merges what the peers pushed here: two launches
    per step, no collective library on the path."""

    def __init__(self, segments: Sequence, hot_k, hot_v, num_attention_heads: int, head_dim: int, device,
                 group: Optional[dist.ProcessGroup] = None, exchange: Optional[PeerExchange] = None):
        from . import _native as nv
        from .kernels import attention_cuda as ac
        from .kernels.tiers import LayerTiers, PackedKVSegment
        import ctypes
        self.nv, self.group, self.device, self.exchange = nv, group, device, exchange
        self.hq, self.hd = num_attention_heads, head_dim
        self.world = exchange.world if exchange is not None else dist.get_world_size(group)
        n = self.hq * (self.hd + 2)
        self.part = torch.zeros(n, dtype=torch.float32, device=device)
        self.part[self.hq * self.hd:self.hq * self.hd + self.hq] = float("-inf")  # neutral element
        self.gathered = torch.empty(self.world * n, dtype=torch.float32, device=device)
        self.out = torch.empty((self.hq, self.hd), dtype=torch.float16, device=device)
        segs = [PackedKVSegment(k, v) for k, v in segments]
        hot_len = 0 if hot_k is None else hot_k.shape[-2]
        self.segs, self.hkv, self.sms = None, 1, nv.sm_count(device)
        self.ws = torch.empty(16, dtype=torch.uint8, device=device)
        if segs or hot_len:
            if segs:
                tiers = LayerTiers(prompt=segs[0], cold=segs[1:], hot_k=hot_k, hot_v=hot_v, hot_len=hot_len)
                seg_list, self._keep, self.hkv, _ = ac.layer_segments(tiers)
            else:
                s, self._keep = ac._fp16_segment(hot_k[0], hot_v[0])
                seg_list, self.hkv = [s], hot_k.shape[1]
            self.segs = (nv.Segment * len(seg_list))(*seg_list)
            self.sms = nv.sm_count(device)
            need = ctypes.c_size_t(0)
            nv.check(nv.lib().pkv_decode_workspace_bytes(self.segs, len(seg_list), self.hq, self.hkv, self.hd, self.sms,
                                                         ctypes.byref(need)))
            self.ws = torch.empty(max(need.value, 16), dtype=torch.uint8, device=device)

    def run(self, q: torch.Tensor) -> torch.Tensor:
        nv, L = self.nv, self.nv.lib()
        stream = nv.stream_of(self.device)
        if self.exchange is not None:
            n_segs = 0 if self.segs is None else len(self.segs)
            nv.check(L.pkv_decode_attention_sharded(q.data_ptr(), self.segs, n_segs, self.hq, self.hkv, self.hd,
                                                    1.0 / (self.hd ** 0.5), self.sms, self.ws.data_ptr(),
                                                    self.ws.numel(), self.exchange.handle, self.out.data_ptr(), stream))
            return self.out
        base, f = self.part.data_ptr(), 4
        if self.segs is not None:
            nv.check(L.pkv_decode_attention(q.data_ptr(), self.segs, len(self.segs), self.hq, self.hkv, self.hd,
                                            1.0 / (self.hd ** 0.5), self.sms, self.ws.data_ptr(), self.ws.numel(),
                                            None, base + f * self.hq * self.hd, base + f * (self.hq * self.hd + self.hq),
                                            base, stream))
        dist.all_gather_into_tensor(self.gathered, self.part, group=self.group)
        n = self.hq * (self.hd + 2)
        g = self.gathered.data_ptr()
        nv.check(L.pkv_merge_partials_strided(g + f * self.hq * self.hd, g + f * (self.hq * self.hd + self.hq), g,
                                              self.world, n, n, self.hq, self.hd, self.out.data_ptr(), None, None,
                                              None, stream))
        return self.out


def sequence_sharded_decode(q: torch.Tensor, segments: Sequence, hot_k, hot_v, num_attention_heads: int,
                            group: Optional[dist.ProcessGroup] = None,
                            exchange: Optional[PeerExchange] = None) -> torch.Tensor:
    """Decode attention of ``q [Hq, hd]`` where this rank holds ``segments`` (its shard of the prompt
    tier and, on one rank, the cold segments; each a ``(key, value)`` pair with batch dim 1) and
    optionally the hot tier ``[1, Hkv, hot, hd]``.  Returns the merged ``[Hq, hd]`` float16 on every rank."""
    layer = ShardedDecodeLayer(segments, hot_k, hot_v, num_attention_heads, q.shape[-1], q.device, group, exchange)
    with torch.cuda.device(q.device):
        return layer.run(q.contiguous()).clone()
