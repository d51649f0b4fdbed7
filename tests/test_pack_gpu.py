"""Bit-exact parity of the CUDA quantise+pack kernels (through the C ABI) with the oracle and with
fixtures produced by the reference's packing.py on CPU."""
import pytest
import torch

from conftest import from_f16, load_packed
from util import assert_packed_equal, to_gpu_packed

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def pk():
    from phasekv_b200.kernels import packing
    return packing


def test_golden_pack_cases(golden, pk):
    z = golden("pack_cases.npz")
    for i in range(int(z["n_cases"][0])):
        x = from_f16(z[f"c{i}.x"]).cuda()
        axis, bits, gs = (int(v) for v in z[f"c{i}.args"])
        ref = load_packed(z, f"c{i}.pt")
        got = pk.quantize_pack(x, bits, axis, gs)
        assert_packed_equal(got, ref, f"golden case {i}")
        deq = pk.unpack_dequantize(to_gpu_packed(ref)).cpu()
        assert torch.equal(deq.view(torch.int16), from_f16(z[f"c{i}.deq"]).view(torch.int16)), i
        codes = pk.unpack_low_bits(ref.packed.cuda(), ref.bits, ref.axis_len)
        assert torch.equal(codes.cpu(), torch.from_numpy(z[f"c{i}.codes"])), i
        assert torch.equal(pk.pack_low_bits(codes, ref.bits).cpu(), ref.packed), i


@pytest.mark.parametrize("bits", [2, 4, 8])
def test_prefill_pack_32768_tokens(oracle, pk, bits):
    """The prefill pack configuration: K/V of 32768 tokens x 4 KV heads x 128 dims."""
    from phasekv_b200 import workloads
    gen = torch.Generator().manual_seed(3)
    k, v = workloads.make_kv(gen, 4, 32768, 128)
    for x, axis in ((k, -2), (v, -1)):
        ref = oracle.quantize_pack(x, bits, axis, 32)
        got = pk.quantize_pack(x.cuda(), bits, axis, 32)
        assert_packed_equal(got, ref, f"bits {bits} axis {axis}")
        # size-independent property: dequantisation error is bounded by half a step
        deq = pk.unpack_dequantize(got).float().cpu()
        step = ref.scale.float()
        step = step.repeat_interleave(32, dim=-1)
        step = step.movedim(-1, axis) if axis == -2 else step
        err = (deq - x.float()).abs()
        qmax = (1 << bits) - 1  # the stored scale is float16: up to qmax * 2^-11 steps of extra error
        assert bool((err <= (0.5 + qmax / 1024) * step * 1.01 + 2e-3 * x.float().abs() + 1e-6).all())


@pytest.mark.parametrize("hd", [8, 64, 128, 256])
@pytest.mark.parametrize("S", [1, 7, 31, 33, 127, 129])
def test_ragged_shapes(oracle, pk, S, hd):
    gen = torch.Generator().manual_seed(S * 1000 + hd)
    x = torch.randn(2, 2, S, hd, generator=gen).half()
    for bits in (2, 4, 8):
        for axis, gs in ((-2, 32), (-1, 32), (-2, 5), (-1, 0), (1, 3)):
            ref = oracle.quantize_pack(x, bits, axis, gs)
            got = pk.quantize_pack(x.cuda(), bits, axis, gs)
            assert_packed_equal(got, ref, f"S {S} hd {hd} bits {bits} axis {axis} gs {gs}")
            deq_ref = oracle.unpack_dequantize(ref)
            deq = pk.unpack_dequantize(got).cpu()
            assert torch.equal(deq.view(torch.int16), deq_ref.view(torch.int16))


def test_constant_and_half_way_groups(oracle, pk):
    # constant groups give scale 1e-8/qmax -> float16 zero; a coarse grid makes exact .5 quotients
    gen = torch.Generator().manual_seed(5)
    const = torch.full((1, 2, 64, 64), -1.25).half()
    grid = (torch.randint(-12, 13, (1, 2, 256, 128), generator=gen).float() / 8).half()
    for x in (const, grid):
        for bits in (2, 4, 8):
            for axis in (-2, -1):
                assert_packed_equal(pk.quantize_pack(x.cuda(), bits, axis, 32),
                                    oracle.quantize_pack(x, bits, axis, 32), f"{bits} {axis}")


def test_low_bits_round_trip(pk):
    gen = torch.Generator().manual_seed(11)
    for bits in (2, 4, 8):
        for length in (1, 3, 4, 5, 64, 129):
            codes = torch.randint(0, 1 << bits, (3, 5, length), generator=gen, dtype=torch.uint8).cuda()
            packed = pk.pack_low_bits(codes, bits)
            assert packed.shape[-1] == -(-length // (8 // bits))
            assert torch.equal(pk.unpack_low_bits(packed, bits, length), codes)


def test_argument_errors(pk):
    x = torch.zeros(2, 4, 8, dtype=torch.float16, device="cuda")
    with pytest.raises(ValueError):
        pk.quantize_pack(x, 3, -1, 4)
    with pytest.raises(ValueError):
        pk.pack_low_bits(torch.zeros(4, dtype=torch.int32, device="cuda"), 2)
    with pytest.raises(ValueError):
        pk.unpack_low_bits(torch.zeros(4, dtype=torch.uint8, device="cuda"), 5, 4)
    with pytest.raises(RuntimeError):
        pk.quantize_pack(x.cpu(), 2, -1, 4)  # no CPU path
