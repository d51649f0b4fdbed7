"""Sequence-sharded decode on real GPUs (one process per GPU, NCCL); skipped with fewer than two GPUs."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))


def _rank_main(rank, world, port, tmp):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        import pkv_oracle as oracle
        from phasekv_b200 import workloads
        from phasekv_b200.sharding import sequence_bounds, sequence_sharded_decode, shard_kivi_segment
        from util import to_gpu_packed
        shape = workloads.QWEN2_5_7B
        (pk, pv), (ck, cv), (hk, hv), q = workloads.three_tier_dense(5, shape, 8192 + 640, 256, 100)
        q = q[0, :, 0, :]
        gk, gv = oracle.quantize_pack(pk, 2, -2, 32), oracle.quantize_pack(pv, 2, -1, 32)
        cold = (oracle.quantize_pack(ck, 4, -2, 32), oracle.quantize_pack(cv, 4, -1, 32))
        start, end = sequence_bounds(pk.shape[2], world)[rank]
        dev = torch.device("cuda", rank)
        segs = [tuple(to_gpu_packed(t, dev) for t in shard_kivi_segment(gk, gv, start, end))]
        if rank == 0:
            segs.append(tuple(to_gpu_packed(t, dev) for t in cold))
        out = sequence_sharded_decode(q.to(dev), segs, hk.to(dev) if rank == 0 else None,
                                      hv.to(dev) if rank == 0 else None, shape.num_q_heads)
        full = oracle.segments_decode_reference(q, [(gk, gv), cold], hk, hv, shape.num_q_heads).float()
        err = (out.float().cpu() - full).abs().max().item()
        # the same through the peer-to-peer exchange kernel (plain peer stores, no NVLS, no collective library)
        from phasekv_b200.sharding import PeerExchange, ShardedDecodeLayer
        ex = PeerExchange(shape.num_q_heads, shape.head_dim, dev)
        try:
            layer = ShardedDecodeLayer(segs, hk.to(dev) if rank == 0 else None, hv.to(dev) if rank == 0 else None,
                                       shape.num_q_heads, shape.head_dim, dev, exchange=ex)
            err_p2p = 0.0
            for _ in range(4):  # slots alternate with the call parity
                got = layer.run(q.to(dev)).float().cpu()
                err_p2p = max(err_p2p, (got - full).abs().max().item())
            same = (layer.out.float() - out.float()).abs().max().item() <= 5e-4  # two merge orders of the same partials
            timed_out = ex.timed_out()
        finally:
            dist.barrier()
            ex.close()
        torch.save({"err": err, "err_p2p": err_p2p, "same": same, "timed_out": timed_out,
                    "ref": full.abs().max().item()}, os.path.join(tmp, f"r{rank}.pt"))
    finally:
        dist.destroy_process_group()


def test_sequence_sharded_decode_over_nccl(tmp_path):
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    port = 29500 + os.getpid() % 1000
    mp.spawn(_rank_main, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        res = torch.load(os.path.join(tmp_path, f"r{r}.pt"))
        assert res["err"] <= 2e-3 and res["err"] <= 1e-2 * res["ref"], res
        assert not res["timed_out"] and res["err_p2p"] <= 2e-3 and res["same"], res
