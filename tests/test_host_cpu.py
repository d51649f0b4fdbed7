"""Host-side logic that needs no GPU: the planner, the C-ABI library's exports, argument checks."""
import ctypes
import json
import os
import re

import pytest
import torch

from conftest import GOLDEN, ROOT


def test_planner_matches_reference_outputs():
    from phasekv_b200.kernels.launch_config import plan_kivi_decode
    rows = json.load(open(os.path.join(GOLDEN, "planner.json")))
    assert len(rows) > 100
    for r in rows:
        c = plan_kivi_decode(*r["args"], **r["kwargs"])
        assert [c.num_splits, c.split_len, c.block_n, c.num_warps] == r["plan"], r


def test_planner_invariants_and_errors():
    """tests/test_phasekv_launch_config.py:9-47 of the reference."""
    from phasekv_b200.kernels.launch_config import plan_kivi_decode
    for length in (1, 7, 31, 127, 128, 129, 511, 512, 8193, 28672):
        for heads, dim, sms in ((12, 128, 46), (4, 8, 1), (32, 256, 132), (28, 128, 148)):
            c = plan_kivi_decode(length, heads, dim, sms)
            assert 1 <= c.num_splits <= 128
            assert (c.num_splits - 1) * c.split_len < length <= c.num_splits * c.split_len
            assert c.split_len % c.block_n == 0 and c.block_n * dim <= 1024
    old = plan_kivi_decode(8192, 12, 128, 46, 8, 64, 4)
    assert (old.num_splits, old.split_len, old.block_n, old.num_warps) == (8, 1024, 64, 4)
    uneven = plan_kivi_decode(10, 12, 128, 46, num_splits=8)
    assert (uneven.num_splits, uneven.split_len) == (5, 2)
    assert plan_kivi_decode(1, 12, 128, 46, num_splits=100).num_splits == 1
    assert plan_kivi_decode(32768, 28, 128, 148) == plan_kivi_decode(32768, 28, 128, 148)
    for kwargs in ({"num_splits": 0}, {"block_n": 0}, {"block_n": 3}, {"num_warps": 3}):
        with pytest.raises(ValueError):
            plan_kivi_decode(128, 12, 128, 46, **kwargs)
    with pytest.raises(ValueError):
        plan_kivi_decode(0, 12, 128, 46)
    with pytest.raises(ValueError):
        plan_kivi_decode(16, 12, 96, 46)


def test_library_exports_every_declared_symbol():
    from phasekv_b200 import _native, build
    build.build()
    header = open(os.path.join(ROOT, "include", "phasekv_b200.h")).read()
    declared = set(re.findall(r"\b(pkv_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations parsed"
    lib = ctypes.CDLL(_native.LIB_PATH)
    for name in sorted(declared):
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"
    assert declared == set(_native.EXPORTED_SYMBOLS), declared ^ set(_native.EXPORTED_SYMBOLS)
    L = _native.lib()
    assert L.pkv_abi_version() >= 1
    assert L.pkv_strerror(0) == b"ok" and b"bit width" in L.pkv_strerror(-1)


def _c_layout_of_segment(tmp_path):
    """sizeof and field offsets of pkv_segment_t as the C compiler lays the header's struct out."""
    import subprocess
    fields = [name for name, _ in __import__("phasekv_b200")._native.Segment._fields_]
    src = tmp_path / "layout.c"
    src.write_text('#include <stdio.h>\n#include <stddef.h>\n#include "phasekv_b200.h"\nint main(void) {\n'
                   '  printf("%zu", sizeof(pkv_segment_t));\n'
                   + "".join(f'  printf(" %zu", offsetof(pkv_segment_t, {f}));\n' for f in fields)
                   + "  return 0;\n}\n")
    exe = tmp_path / "layout"
    subprocess.run(["gcc", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe)], check=True)
    nums = [int(v) for v in subprocess.run([str(exe)], capture_output=True, text=True, check=True).stdout.split()]
    return nums[0], dict(zip(fields, nums[1:]))


def test_segment_struct_layout_matches_the_header(tmp_path):
    """The ctypes mirror in _native.py and the stub printed in INTEGRATION.md both describe the C struct."""
    from phasekv_b200 import _native
    size, offsets = _c_layout_of_segment(tmp_path)
    assert ctypes.sizeof(_native.Segment) == size
    for name, _ in _native.Segment._fields_:
        assert getattr(_native.Segment, name).offset == offsets[name], name
    # the stub a maintainer would copy out of INTEGRATION.md
    text = open(os.path.join(ROOT, "INTEGRATION.md")).read()
    block = text[text.index("class Segment(ctypes.Structure)"):]
    block = block[:block.index("\n\n")]
    scope = {"ctypes": ctypes}
    exec(block, scope)
    stub = scope["Segment"]
    assert ctypes.sizeof(stub) == size
    assert [n for n, _ in stub._fields_] == [n for n, _ in _native.Segment._fields_]


def test_abi_rejects_bad_arguments_without_touching_a_gpu():
    from phasekv_b200 import _native
    L = _native.lib()
    assert L.pkv_pack_low_bits(None, 4, 4, 3, None, None) == _native.PKV_E_BITS
    assert L.pkv_pack_low_bits(None, 4, 4, 2, None, None) == _native.PKV_E_NULL
    assert L.pkv_quantize_pack(None, 1, 0, 1, 2, 1, None, None, None, None) == _native.PKV_E_SHAPE
    assert L.pkv_quantize_pack(None, 1, 8, 1, 2, 9, None, None, None, None) == _native.PKV_E_SHAPE
    assert L.pkv_merge_partials(None, None, None, 1, 1, 8, None, None, None, None, None) == _native.PKV_E_NULL
    need = ctypes.c_size_t(0)
    seg = _native.Segment(1, 1, 1, 1, 1, 1, 4096, 0, _native.PKV_SEG_KIVI, 2, 2, 32, 32, 0)
    arr = (_native.Segment * 1)(seg)
    assert L.pkv_decode_workspace_bytes(arr, 1, 28, 4, 128, 148, ctypes.byref(need)) == 0
    assert need.value > 0 and need.value % (28 * 130 * 4) == 0
    assert L.pkv_decode_workspace_bytes(arr, 1, 28, 5, 128, 148, ctypes.byref(need)) == _native.PKV_E_SHAPE
    seg.k_bits = 3
    arr = (_native.Segment * 1)(seg)
    assert L.pkv_decode_workspace_bytes(arr, 1, 28, 4, 128, 148, ctypes.byref(need)) == _native.PKV_E_BITS


def test_cpu_tensors_are_refused():
    from phasekv_b200.kernels import packing
    with pytest.raises(RuntimeError, match="no CPU path"):
        packing.quantize_pack(torch.zeros(2, 8, dtype=torch.float16), 2, -1, 4)
    with pytest.raises(ValueError):
        packing.quantize_pack(torch.zeros(2, 8, dtype=torch.float16), 3, -1, 4)
    with pytest.raises(ValueError):
        packing._vals_per_byte(16)


def test_algorithmic_bytes_table():
    from phasekv_b200 import workloads as w
    s = w.QWEN2_5_7B
    assert w.decode_algorithmic_bytes(s, 4096, 2, 256, 4, 128) == 2_013_184
    assert w.decode_algorithmic_bytes(s, 32768, 2, 256, 4, 128) == 13_023_232
    assert w.decode_algorithmic_bytes(s, 131072, 2, 256, 4, 128) == 50_771_968


def test_batch_plan_covers_every_tile_once():
    """pkv_decode_batch_plan is host-only: with made-up (aligned) device addresses it must produce a table
    whose work items cover every tile of every segment exactly once, longest first, with the partials of a
    sequence contiguous."""
    import ctypes
    import struct

    from phasekv_b200 import _native as nv
    L = nv.lib()
    lengths = [(8192, 512, 128), (6150, 384, 97), (64, 0, 0), (12288, 640, 192), (1, 0, 1)]
    segs, offsets, base = [], [0], 0x10000000
    for p, c, h in lengths:
        for n, bits in ((p, 2), (c, 4)):
            if n:
                ptrs = [base + 0x100000 * k for k in range(6)]
                base += 0x1000000
                segs.append(nv.Segment(*ptrs, n, 0, nv.PKV_SEG_KIVI, bits, bits, 32, 32, 0))
        if h:
            segs.append(nv.Segment(base, None, None, base + 0x100000, None, None, h, 192 * 128, nv.PKV_SEG_FP16,
                                   8, 8, 1, 1, 0))
            base += 0x1000000
        offsets.append(len(segs))
    arr = (nv.Segment * len(segs))(*segs)
    off = (ctypes.c_int32 * len(offsets))(*offsets)
    tb, wb = ctypes.c_size_t(0), ctypes.c_size_t(0)
    nv.check(L.pkv_decode_batch_plan(arr, off, len(lengths), 28, 4, 128, 148, None, 0, ctypes.byref(tb), ctypes.byref(wb)))
    buf = ctypes.create_string_buffer(tb.value + 16)
    addr = (ctypes.addressof(buf) + 15) & ~15
    assert L.pkv_decode_batch_plan(arr, off, len(lengths), 28, 4, 128, 148, addr, tb.value - 16, ctypes.byref(tb),
                                   ctypes.byref(wb)) == nv.PKV_E_WORKSPACE
    nv.check(L.pkv_decode_batch_plan(arr, off, len(lengths), 28, 4, 128, 148, addr, tb.value, ctypes.byref(tb), ctypes.byref(wb)))
    raw = ctypes.string_at(addr, tb.value)
    magic, batch, n_segs, n_work, n_parts, hq, hkv, hd, o_segs, o_work, o_ranges, nbytes = struct.unpack_from("<I7i4I", raw)
    assert (magic, batch, n_segs, hq, hkv, hd, nbytes) == (0x42564B50, len(lengths), len(segs), 28, 4, 128, tb.value)
    assert n_work == n_parts and wb.value == n_parts * 28 * 130 * 4
    covered = [set() for _ in segs]
    parts, prev = set(), None
    seq_of_seg = [b for b in range(len(lengths)) for _ in range(offsets[b], offsets[b + 1])]
    ranges = [struct.unpack_from("<2i", raw, o_ranges + 8 * b) for b in range(batch)]
    for w in range(n_work):
        seg, seq, t0, nt, part = struct.unpack_from("<5i", raw, o_work + 32 * w)
        assert seq == seq_of_seg[seg] and nt > 0 and (prev is None or nt <= prev)
        prev = nt
        tiles = set(range(t0, t0 + nt))
        assert not (tiles & covered[seg])
        covered[seg] |= tiles
        assert part not in parts and ranges[seq][0] <= part < ranges[seq][0] + ranges[seq][1]
        parts.add(part)
        if segs[seg].kind == nv.PKV_SEG_KIVI and nt > 4:
            assert t0 % 4 == 0
    for s, got in zip(segs, covered):
        per = 32 if s.kind == nv.PKV_SEG_FP16 else 64
        assert got == set(range((s.seq_len + per - 1) // per))
    assert sorted(parts) == list(range(n_parts)) and sum(r[1] for r in ranges) == n_parts
    # a per-token-layout segment is not a batched shape
    bad = (nv.Segment * 1)(nv.Segment(*[0x1000 * (k + 1) for k in range(6)], 64, 0, nv.PKV_SEG_PER_TOKEN, 4, 4, 32, 32, 0))
    one = (ctypes.c_int32 * 2)(0, 1)
    assert L.pkv_decode_batch_plan(bad, one, 1, 28, 4, 128, 148, None, 0, ctypes.byref(tb), ctypes.byref(wb)) == nv.PKV_E_LAYOUT


def test_chunk_plan_applies_the_causal_rule_by_length():
    """pkv_decode_chunk_plan is host-only: query i of a chunk of N new tokens must see every packed segment in full
    and the float16 tier up to and including its own token (seq_len - (N - 1 - i) tokens)."""
    import struct

    from phasekv_b200 import _native as nv
    L = nv.lib()
    base = 0x20000000
    prompt = nv.Segment(*(base + 0x100000 * k for k in range(6)), 4096, 0, nv.PKV_SEG_KIVI, 2, 2, 32, 32, 0)
    arena = nv.Segment(*(base + 0x1000000 + 0x100000 * k for k in range(6)), 5 * 32, 64 * 32, nv.PKV_SEG_KIVI, 4, 4, 32, 32, 0,
                       64 * 16, 64, 0, 32, 8)
    hot = nv.Segment(base + 0x2000000, None, None, base + 0x2100000, None, None, 45, 96 * 128, nv.PKV_SEG_FP16, 8, 8, 1, 1, 0)
    arr = (nv.Segment * 3)(prompt, arena, hot)
    n = 7
    tb, wb = ctypes.c_size_t(0), ctypes.c_size_t(0)
    nv.check(L.pkv_decode_chunk_plan(arr, 3, n, 28, 4, 128, 148, None, 0, ctypes.byref(tb), ctypes.byref(wb)))
    buf = ctypes.create_string_buffer(tb.value + 16)
    addr = (ctypes.addressof(buf) + 15) & ~15
    nv.check(L.pkv_decode_chunk_plan(arr, 3, n, 28, 4, 128, 148, addr, tb.value, ctypes.byref(tb), ctypes.byref(wb)))
    raw = ctypes.string_at(addr, tb.value)
    magic, batch, n_segs, n_work, n_parts, hq, hkv, hd, o_segs, o_work, o_ranges, nbytes = struct.unpack_from("<I7i4I", raw)
    assert (magic, batch, n_segs) == (0x42564B50, n, 3 * n) and wb.value == n_parts * 28 * 130 * 4
    seg_bytes = (o_work - o_segs) // n_segs
    assert seg_bytes * n_segs <= o_work - o_segs and seg_bytes >= 7 * 8
    lengths = [struct.unpack_from("<q", raw, o_segs + seg_bytes * i + 6 * 8)[0] for i in range(n_segs)]  # after six pointers
    for i in range(n):
        assert lengths[3 * i:3 * i + 3] == [4096, 5 * 32, 45 - (n - 1 - i)], i
    # every query owns a contiguous range of partials, and all work items point at its own three segments
    for w in range(n_work):
        seg, seq, t0, nt, part = struct.unpack_from("<5i", raw, o_work + 32 * w)
        assert seg // 3 == seq and nt > 0
    # the chunk cannot be longer than the float16 tier, and the last segment must be that tier
    assert L.pkv_decode_chunk_plan(arr, 3, 46, 28, 4, 128, 148, None, 0, ctypes.byref(tb), ctypes.byref(wb)) == nv.PKV_E_SHAPE
    assert L.pkv_decode_chunk_plan(arr, 2, 1, 28, 4, 128, 148, None, 0, ctypes.byref(tb), ctypes.byref(wb)) == nv.PKV_E_SHAPE
    assert L.pkv_decode_chunk_plan(None, 3, 1, 28, 4, 128, 148, None, 0, ctypes.byref(tb), ctypes.byref(wb)) == nv.PKV_E_NULL
    # a layout the tensor-core kernel does not take: the caller serves the chunk query by query
    hot64 = nv.Segment(base, None, None, base + 0x100000, None, None, 9, 96 * 64, nv.PKV_SEG_FP16, 8, 8, 1, 1, 0)
    assert L.pkv_decode_chunk_plan((nv.Segment * 1)(hot64), 1, 3, 14, 2, 64, 148, None, 0, ctypes.byref(tb),
                                   ctypes.byref(wb)) == nv.PKV_E_LAYOUT


def test_adapter_and_cooling_entry_points_check_arguments_first():
    from phasekv_b200 import _native as nv
    L = nv.lib()
    p = 0x30000000
    ok = dict(q=p, k=p, v=p, dtype=nv.PKV_DTYPE_F16, qs=28 * 128, ks=4 * 128, vs=4 * 128, cos=p, sin=p, rdt=nv.PKV_DTYPE_F32,
              rs=128, n=3, hq=28, hkv=4, hd=128, qo=p, hk=p, hv=p, cap=48, slot=10)

    def rope(**over):
        a = dict(ok, **over)
        return L.pkv_rope_append(a["q"], a["k"], a["v"], a["dtype"], a["qs"], a["ks"], a["vs"], a["cos"], a["sin"], a["rdt"],
                                 a["rs"], a["n"], a["hq"], a["hkv"], a["hd"], a["qo"], a["hk"], a["hv"], a["cap"], a["slot"],
                                 a.get("slot_dev"), None)
    assert rope(q=None) == nv.PKV_E_NULL and rope(hv=None) == nv.PKV_E_NULL
    assert rope(n=0) == nv.PKV_E_SHAPE and rope(hd=63) == nv.PKV_E_SHAPE
    assert rope(slot=46) == nv.PKV_E_SHAPE          # three tokens do not fit behind slot 46 of 48
    assert rope(n=49, slot=0, slot_dev=p) == nv.PKV_E_SHAPE   # with a device-resident slot only the capacity is checkable
    assert rope(qs=100) == nv.PKV_E_SHAPE           # a token stride shorter than a token
    assert rope(dtype=nv.PKV_DTYPE_F32) == nv.PKV_E_LAYOUT
    # cooling of all layers: (layers, n_layers, rows, capacity, hd, hot_len, aged, keep, bits, group, pitches..., offsets...)
    def cool(layers=p, n_layers=2, rows=4, capacity=48, hd=128, hot_len=48, aged=16, keep=8, bits=4, group=32):
        return L.pkv_cold_select_pack_layers(layers, n_layers, rows, capacity, hd, hot_len, aged, keep, bits, group,
                                             64 * 16, 64, 64 * 32, 0, 0, 0, None)
    assert cool(layers=None) == nv.PKV_E_NULL
    assert cool(n_layers=0) == nv.PKV_E_LIMIT
    assert cool(bits=3) == nv.PKV_E_BITS
    assert cool(keep=17) == nv.PKV_E_SHAPE and cool(hot_len=49) == nv.PKV_E_SHAPE


def test_hardware_spec_has_the_planner_fields(tmp_path):
    """planner.HardwareSpec of the reference (planner.py:43-59): name, peak_flops, hbm_bandwidth, ridge_intensity."""
    from phasekv_b200.hardware import HardwareSpec, b200
    spec = b200()
    assert spec.name == "B200" and spec.hbm_bandwidth > 6e12 and spec.peak_flops > 1e15
    assert abs(spec.ridge_intensity - spec.peak_flops / spec.hbm_bandwidth) < 1e-9
    # decode attention over 2-bit KV (37 FLOP per byte) is bandwidth-bound on this GPU, as on the reference's
    assert 37 < spec.ridge_intensity and 37 < HardwareSpec("RTX 4080 SUPER", 50.0e12, 736.0e9).ridge_intensity
    path = tmp_path / "peaks.json"
    path.write_text(json.dumps({"hbm_gbs": 6555.8, "bf16_tflops": 1500.0}))
    measured = b200(str(path))
    assert measured.hbm_bandwidth == 6555.8e9 and measured.peak_flops == 1.5e15 and "measured" in measured.name
