"""Host-side logic of the multi-GPU partitions, on CPU ranks (gloo, world size 2 and 3)."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))


def test_bounds_and_shards_are_aligned_and_cover():
    from phasekv_b200.sharding import batch_shard, head_shard, sequence_bounds
    for S in (1, 63, 64, 65, 1000, 32768, 262144, 262144 + 17):
        for R in (1, 2, 3, 4, 8):
            b = sequence_bounds(S, R)
            assert len(b) == R and b[0][0] == 0 and b[-1][1] == S
            for (s0, e0), (s1, e1) in zip(b, b[1:]):
                assert e0 == s1 and s1 % 64 == 0 or s1 == S
            sizes = [e - s for s, e in b]
            assert max(sizes) - min(s for s in sizes) <= 64 + 63
    assert sorted(sum((batch_shard(10, 4, r) for r in range(4)), [])) == list(range(10))
    assert [head_shard(4, 2, r) for r in range(2)] == [(0, 2), (2, 4)]
    with pytest.raises(ValueError):
        head_shard(4, 3, 0)


def test_sharded_packed_tensors_equal_slices_of_the_global_one(oracle):
    """Quantising a 64-aligned token shard on its own gives exactly the bytes of the global tensor's slice."""
    from phasekv_b200 import workloads
    from phasekv_b200.sharding import sequence_bounds, shard_kivi_segment
    gen = torch.Generator().manual_seed(3)
    k, v = workloads.make_kv(gen, 2, 1000, 64)
    for bits in (2, 4, 8):
        gk, gv = oracle.quantize_pack(k, bits, -2, 32), oracle.quantize_pack(v, bits, -1, 32)
        for start, end in sequence_bounds(1000, 3):
            sk, sv = shard_kivi_segment(gk, gv, start, end)
            lk = oracle.quantize_pack(k[:, :, start:end].contiguous(), bits, -2, 32)
            lv = oracle.quantize_pack(v[:, :, start:end].contiguous(), bits, -1, 32)
            for a, b in ((sk, lk), (sv, lv)):
                assert tuple(a.orig_shape) == tuple(b.orig_shape) and a.axis_len == b.axis_len
                assert torch.equal(a.packed, b.packed)
                assert torch.equal(a.scale.view(torch.int16), b.scale.view(torch.int16))
                assert torch.equal(a.mins.view(torch.int16), b.mins.view(torch.int16))


def _rank_main(rank, world, port, seed, tmp):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import pkv_oracle as oracle
        from phasekv_b200 import workloads
        from phasekv_b200.sharding import empty_partial, gather_partials, sequence_bounds, shard_kivi_segment
        shape = workloads.Shape("t", 8, 2, 64, 1)
        (pk, pv), (ck, cv), (hk, hv), q = workloads.three_tier_dense(seed, shape, 700, 64, 20)
        q = q[0, :, 0, :]
        gk, gv = oracle.quantize_pack(pk, 2, -2, 32), oracle.quantize_pack(pv, 2, -1, 32)
        cold = (oracle.quantize_pack(ck, 4, -2, 32), oracle.quantize_pack(cv, 4, -1, 32))
        start, end = sequence_bounds(700, world)[rank]
        segs = [shard_kivi_segment(gk, gv, start, end)] if end > start else []
        if rank == 0:
            segs.append(cold)
        if segs or rank == 0:
            _, _, (m, l, acc) = oracle.segments_decode_reference(q, segs, hk if rank == 0 else None,
                                                                 hv if rank == 0 else None, 8, want_partial=True)
        else:
            m, l, acc = empty_partial(8, 64, "cpu")
        gm, gl, gacc = gather_partials(m, l, acc)
        assert gm.shape == (world, 8) and gacc.shape == (world, 8, 64)
        # the merge algebra, in plain torch (the product merge is the CUDA kernel; this is the checker)
        M = gm.max(dim=0).values
        w = torch.exp(gm - M)
        out = ((w[..., None] * gacc).sum(0) / (w * gl).sum(0)[:, None])
        full = oracle.segments_decode_reference(q, [(gk, gv), cold], hk, hv, 8).float()
        err = (out - full).abs().max().item()
        torch.save({"err": err}, os.path.join(tmp, f"r{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_sequence_sharded_partials_merge_to_the_unsharded_result(tmp_path, world):
    port = 29000 + (os.getpid() + world) % 2000
    mp.spawn(_rank_main, args=(world, port, 11, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert torch.load(os.path.join(tmp_path, f"r{r}.pt"))["err"] < 1e-3
