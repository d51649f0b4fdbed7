"""Helpers shared by the GPU parity tests."""
from dataclasses import replace

import torch

from phasekv_b200.kernels.packing import PackedTensor
from phasekv_b200.kernels.tiers import LayerTiers, PackedKVSegment


def to_gpu_packed(pt, device="cuda") -> PackedTensor:
    """Any PackedTensor-shaped object (oracle result, golden fixture) -> PackedTensor on the GPU."""
    return PackedTensor(packed=pt.packed.to(device), scale=pt.scale.to(device), mins=pt.mins.to(device),
                        bits=int(pt.bits), axis=int(pt.axis), group_size=int(pt.group_size),
                        orig_shape=tuple(int(s) for s in pt.orig_shape), axis_len=int(pt.axis_len))


def to_cpu_packed(pt) -> PackedTensor:
    return to_gpu_packed(pt, "cpu")


def remove_batch(pt: PackedTensor) -> PackedTensor:
    return replace(pt, packed=pt.packed[0], scale=pt.scale[0], mins=pt.mins[0],
                   orig_shape=tuple(pt.orig_shape[1:]), axis=pt.axis - 1)


def assert_packed_equal(got, ref, what=""):
    g, r = to_cpu_packed(got), to_cpu_packed(ref)
    assert (g.bits, g.axis, g.group_size, g.axis_len, g.orig_shape) == \
        (r.bits, r.axis, r.group_size, r.axis_len, r.orig_shape), what
    assert g.packed.shape == r.packed.shape and g.scale.shape == r.scale.shape, what
    assert torch.equal(g.packed, r.packed), f"{what}: packed codes differ " \
        f"({(g.packed != r.packed).sum().item()} of {g.packed.numel()} bytes)"
    assert torch.equal(g.scale.view(torch.int16), r.scale.view(torch.int16)), f"{what}: scales differ"
    assert torch.equal(g.mins.view(torch.int16), r.mins.view(torch.int16)), f"{what}: zeros differ"


def make_tiers(segments, hot_k=None, hot_v=None, hot_len=0, device="cuda") -> LayerTiers:
    """segments: list of (key_pt, value_pt) with batch dim 1; first is the prompt, the rest cold."""
    segs = [PackedKVSegment(to_gpu_packed(k, device), to_gpu_packed(v, device)) for k, v in segments]
    return LayerTiers(prompt=segs[0], cold=segs[1:],
                      hot_k=None if hot_k is None else hot_k.to(device),
                      hot_v=None if hot_v is None else hot_v.to(device), hot_len=hot_len)
