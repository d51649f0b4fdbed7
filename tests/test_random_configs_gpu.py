"""Seeded random layer configurations through the decode entry points, against the oracle.

Every draw mixes what the fixed-shape tests vary one at a time: the attention shape (both kernels: head_dim 128 on the
tensor-core kernel, head_dim 64 / 256 and value groups of 64 on the general one), prompt length and width, zero to
three cold segments of their own widths and lengths (down to one token), a float16 tier of any length including none.
Keys are plain N(0, 1) here (no outlier channels), and contexts hold at least 256 tokens, so the output is an
average of many value rows and the parity bar applies without the single-row float16-step effect of tiny contexts."""
import random

import pytest
import torch

from conftest import attention_close
from util import make_tiers

pytestmark = pytest.mark.gpu


def _draw(rng):
    hq, hkv, hd, gsv = rng.choice([(28, 4, 128, 32), (32, 4, 128, 32), (8, 8, 128, 32), (12, 2, 128, 32), (14, 2, 64, 64),
                                   (14, 2, 64, 32), (8, 2, 256, 32)])
    prompt = rng.choice([256, 300, 777, 1024, 2049, 4096, 5000])
    cold = [rng.choice([1, 7, 32, 64, 100, 255]) for _ in range(rng.randrange(4))]
    hot = rng.choice([0, 1, 31, 32, 33, 64, 130])
    return hq, hkv, hd, gsv, prompt, rng.choice([2, 4, 8]), cold, rng.choice([2, 4, 8]), hot


@pytest.mark.parametrize("seed", range(24))
def test_random_layer_against_the_oracle(oracle, seed):
    from phasekv_b200.kernels import attention_triton as attn
    rng = random.Random(seed)
    hq, hkv, hd, gsv, prompt, pbits, cold, cbits, hot = _draw(rng)
    gen = torch.Generator().manual_seed(1000 + seed)

    def kv(length):
        return (torch.randn(1, hkv, length, hd, generator=gen).half(), torch.randn(1, hkv, length, hd, generator=gen).half())
    segs = []
    for length, bits in [(prompt, pbits)] + [(c, cbits) for c in cold]:
        k, v = kv(length)
        segs.append((oracle.quantize_pack(k, bits, -2, 32), oracle.quantize_pack(v, bits, -1, gsv)))
    hk, hv = kv(hot) if hot else (None, None)
    q = torch.randn(hq, hd, generator=gen).half()
    ref = oracle.segments_decode_reference(q, segs, hk, hv, hq)
    tiers = make_tiers(segs, hk, hv, hot_len=hot)
    out = attn.fused_phasekv_decode(q.cuda(), tiers, hq)
    assert out.shape == (hq, hd) and torch.isfinite(out).all()
    attention_close(out, ref)
    if hd == 128 and hq // hkv <= 8:
        # the same layer as one sequence of a batch, and as a one-token "chunk" (its query sees the whole float16 tier)
        from phasekv_b200.kernels.attention_cuda import BatchDecodePlan, fused_phasekv_chunk_decode
        batched = BatchDecodePlan([tiers, tiers], hq).run(torch.stack([q, q]).cuda())
        attention_close(batched[0], ref), attention_close(batched[1], ref)
        if hot:
            attention_close(fused_phasekv_chunk_decode(q[None].cuda(), tiers, hq)[0], ref)
