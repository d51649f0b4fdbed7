"""The peer-to-peer exchange + merge kernel of the sequence-sharded decode, on ONE GPU (loopback)."""
import pytest
import torch

from tests.test_decode_gpu import _pack_tiers
from tests.util import make_tiers

pytestmark = pytest.mark.gpu


def _layer(oracle, exchange, seed=11, prompt=3000):
    from phasekv_b200 import workloads
    from phasekv_b200.sharding import ShardedDecodeLayer
    shape = workloads.QWEN2_5_7B
    segs, hk, hv, q = _pack_tiers(oracle, shape, prompt, 2, [256], 4, 100, seed=seed)
    tiers = make_tiers(segs, hk, hv, hot_len=100)
    pairs = [(tiers.prompt.key, tiers.prompt.value)] + [(c.key, c.value) for c in tiers.cold]
    layer = ShardedDecodeLayer(pairs, tiers.hot_k, tiers.hot_v, shape.num_q_heads, shape.head_dim,
                               torch.device("cuda", 0), exchange=exchange)
    return shape, tiers, q[0, :, 0, :].cuda(), layer


def test_world_of_one_is_a_complete_exchange(oracle):
    """Push to self, wait on own flag, merge one row: must agree with the ordinary entry point to within the
    rounding of a different summation order (that one merges its partials inside the split-K launch, this one in
    the exchange kernel), call after call (the epoch and the slot parity advance in device memory), also when
    replayed as a CUDA graph."""
    from phasekv_b200.kernels import attention_cuda as attn
    from phasekv_b200.sharding import PeerExchange
    ex = PeerExchange(28, 128, torch.device("cuda", 0), loopback=True, world=1, rank=0)
    try:
        shape, tiers, q, layer = _layer(oracle, ex)
        for k in range(5):
            qk = torch.roll(q, k, dims=0).contiguous()
            want = attn.fused_phasekv_decode(qk, tiers, shape.num_q_heads)
            got = layer.run(qk).clone()
            assert (got.float() - want.float()).abs().max().item() <= 5e-4, k
        stream = torch.cuda.Stream()
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream):
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                layer.run(q)
            for _ in range(3):
                layer.out.zero_()
                graph.replay()
                stream.synchronize()
                want = attn.fused_phasekv_decode(q, tiers, shape.num_q_heads)
                assert (layer.out.float() - want.float()).abs().max().item() <= 5e-4
        torch.cuda.current_stream().wait_stream(stream)
        assert not ex.timed_out()
    finally:
        ex.close()


def test_a_peer_that_never_arrives_runs_the_wait_out(oracle):
    """world 2 in loopback: nobody ever writes rank 1's row, so the bounded wait gives up.  The kernel must
    return (NaN rows, status word set) and leave the context usable."""
    from phasekv_b200.kernels import attention_cuda as attn
    from phasekv_b200.sharding import PeerExchange
    ex = PeerExchange(28, 128, torch.device("cuda", 0), loopback=True, world=2, rank=0)
    try:
        ex.set_spin_limit(2000)  # a few hundred microseconds
        shape, tiers, q, layer = _layer(oracle, ex, seed=12, prompt=512)
        assert not ex.timed_out()
        out = layer.run(q).clone()
        torch.cuda.synchronize()
        assert ex.timed_out()
        assert torch.isnan(out).all()
        again = attn.fused_phasekv_decode(q, tiers, shape.num_q_heads)
        assert torch.isfinite(again).all()
        # the failure is sticky: with the budget set back to its large default, later calls still return at once
        ex.set_spin_limit(1 << 21)
        import time
        t0 = time.perf_counter()
        for _ in range(28):
            out = layer.run(q)
        torch.cuda.synchronize()
        assert time.perf_counter() - t0 < 0.25, "calls after a timed-out wait must not wait again"
        assert torch.isnan(out).all()
        with pytest.raises(RuntimeError):
            ex.check()
    finally:
        ex.close()


def test_the_clock_bounds_the_wait_too(oracle):
    """A huge pass budget, a 2 ms clock budget: the wait ends by the clock."""
    import time
    from phasekv_b200.sharding import PeerExchange
    ex = PeerExchange(28, 128, torch.device("cuda", 0), loopback=True, world=2, rank=0)
    try:
        ex.set_spin_limit(0x7fffffff)
        ex.set_wait_us(2000)
        shape, tiers, q, layer = _layer(oracle, ex, seed=13, prompt=512)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        out = layer.run(q).clone()
        torch.cuda.synchronize()
        assert time.perf_counter() - t0 < 0.5
        assert ex.timed_out() and torch.isnan(out).all()
    finally:
        ex.close()


def test_exchange_argument_checks():
    import ctypes
    from phasekv_b200 import _native as nv
    L = nv.lib()
    h, buf = ctypes.c_void_p(), ctypes.create_string_buffer(64)
    assert L.pkv_exchange_create(0, 0, 28, 128, ctypes.byref(h), buf) == nv.PKV_E_SHAPE
    assert L.pkv_exchange_create(2, 2, 28, 128, ctypes.byref(h), buf) == nv.PKV_E_SHAPE
    assert L.pkv_exchange_create(17, 0, 28, 128, ctypes.byref(h), buf) == nv.PKV_E_LIMIT
    assert L.pkv_exchange_create(1, 0, 28, 128, None, buf) == nv.PKV_E_NULL
    nv.check(L.pkv_exchange_create(1, 0, 28, 128, ctypes.byref(h), buf))
    out = torch.empty(28, 128, dtype=torch.float16, device="cuda")
    # not connected yet / wrong shape
    assert L.pkv_decode_attention_sharded(None, None, 0, 28, 4, 128, 0.1, 148, None, 0, h, out.data_ptr(), None) == nv.PKV_E_SHAPE
    nv.check(L.pkv_exchange_connect_loopback(h))
    assert L.pkv_decode_attention_sharded(None, None, 0, 14, 2, 64, 0.1, 148, None, 0, h, out.data_ptr(), None) == nv.PKV_E_SHAPE
    # a rank without tokens: the neutral partial alone merges to 0/0
    nv.check(L.pkv_decode_attention_sharded(None, None, 0, 28, 4, 128, 0.1, 148, None, 0, h, out.data_ptr(), None))
    torch.cuda.synchronize()
    assert torch.isnan(out).all()
    nv.check(L.pkv_exchange_destroy(h))
