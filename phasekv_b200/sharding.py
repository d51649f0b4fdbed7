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


def sequence_sharded_decode(q: torch.Tensor, segments: Sequence, hot_k, hot_v, num_attention_heads: int,
                            group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """Decode attention of ``q [Hq, hd]`` where this rank holds ``segments`` (its shard of the prompt
    tier and, on one rank, the cold segments; each a ``(key, value)`` pair with batch dim 1) and
    optionally the hot tier ``[1, Hkv, hot, hd]``.  Returns the merged ``[Hq, hd]`` float16 on every rank."""
    from .kernels import attention_cuda as ac
    from .kernels.tiers import LayerTiers, PackedKVSegment
    hq, hd = q.shape
    segs = [PackedKVSegment(k, v) for k, v in segments]
    hot_len = 0 if hot_k is None else hot_k.shape[-2]
    if segs or hot_len:
        if segs:
            tiers = LayerTiers(prompt=segs[0], cold=segs[1:], hot_k=hot_k, hot_v=hot_v, hot_len=hot_len)
            seg_list, keep, hkv, _ = ac.layer_segments(tiers)
        else:
            s, keep = ac._fp16_segment(hot_k[0], hot_v[0])
            seg_list, hkv = [s], hot_k.shape[1]
        _, (m, l, acc) = ac._run_decode(q.contiguous(), seg_list, keep, num_attention_heads, hkv, False, True)
    else:
        m, l, acc = empty_partial(hq, hd, q.device)
    gm, gl, gacc = gather_partials(m, l, acc, group)
    return ac._merge_stacked(gm, gl, gacc, want_out=True)[0]
