"""The allocation-free decode entry point against the regular one.

Collected last on purpose (file name): a run that stops at the first failure has then already run
every other test.  It calls the C ABI directly, twice in a row, because the second call starts from
scratch contents the first call left behind."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _decode(nv, fn_static, q, arr, n, hq, hkv, hd, sms, ws):
    out = torch.empty((hq, hd), dtype=torch.float16, device=q.device)
    m = torch.empty((hq,), dtype=torch.float32, device=q.device)
    l = torch.empty_like(m)
    acc = torch.empty((hq, hd), dtype=torch.float32, device=q.device)
    stream = nv.stream_of(q.device)
    L = nv.lib()
    if fn_static:
        nv.check(L.pkv_decode_attention_static(q.data_ptr(), arr, n, hq, hkv, hd, hd ** -0.5, sms, out.data_ptr(),
                                               m.data_ptr(), l.data_ptr(), acc.data_ptr(), stream))
    else:
        nv.check(L.pkv_decode_attention(q.data_ptr(), arr, n, hq, hkv, hd, hd ** -0.5, sms, ws.data_ptr(), ws.numel(),
                                        out.data_ptr(), m.data_ptr(), l.data_ptr(), acc.data_ptr(), stream))
    torch.cuda.synchronize()
    return out, m, l, acc


def test_static_scratch_entry_point_matches_regular_one(oracle):
    from phasekv_b200 import _native as nv
    from phasekv_b200 import workloads
    from phasekv_b200.kernels.attention_cuda import layer_segments
    from conftest import attention_close
    from util import make_tiers
    shape = workloads.QWEN2_5_7B
    gen = torch.Generator().manual_seed(2024)
    cases = []
    for prompt, cold, hot in ((4096, 256, 128), (1000, 70, 33)):  # tensor-core path, then the generic path
        segs = []
        for length, bits in ((prompt, 2), (cold, 4)):
            k, v = workloads.make_kv(gen, shape.num_kv_heads, length, shape.head_dim)
            segs.append((oracle.quantize_pack(k, bits, -2, 32), oracle.quantize_pack(v, bits, -1, 32)))
        hk, hv = workloads.make_kv(gen, shape.num_kv_heads, hot, shape.head_dim)
        q_cpu = workloads.make_query(gen, shape.num_q_heads, shape.head_dim)[0, :, 0, :]
        want = oracle.segments_decode_reference(q_cpu, segs, hk, hv, shape.num_q_heads)
        cases.append((make_tiers(segs, hk, hv, hot_len=hot), q_cpu.cuda(), want))
    sms = nv.sm_count(torch.device("cuda", 0))
    for rep in range(2):  # two calls in a row per case: the array keeps what the previous call wrote
        for tiers, q, want in cases:
            seg_list, keep, hkv, hd = layer_segments(tiers)
            arr = (nv.Segment * len(seg_list))(*seg_list)
            need = ctypes.c_size_t(0)
            nv.check(nv.lib().pkv_decode_workspace_bytes(arr, len(seg_list), 28, hkv, hd, sms, ctypes.byref(need)))
            ws = torch.empty(need.value, dtype=torch.uint8, device="cuda")
            ref = _decode(nv, False, q, arr, len(seg_list), 28, hkv, hd, sms, ws)
            got = _decode(nv, True, q, arr, len(seg_list), 28, hkv, hd, sms, None)
            for a, b in zip(got, ref):
                torch.testing.assert_close(a.float(), b.float(), atol=2e-3, rtol=1e-2)
            assert torch.equal(got[0], ref[0])  # same kernels, same order of operations
            attention_close(got[0], want)       # and the parity bar against the oracle itself


def test_static_scratch_rejects_oversized_requests():
    from phasekv_b200 import _native as nv
    # 4096 segments of one tile each need far more than the built-in array
    big = [nv.Segment(1, 1, 1, 1, 1, 1, 64, 0, nv.PKV_SEG_KIVI, 2, 2, 32, 32, 0) for _ in range(4096)]
    arr = (nv.Segment * len(big))(*big)
    rc = nv.lib().pkv_decode_attention_static(None, arr, len(big), 28, 4, 128, 0.1, 148, None, None, None, None, None)
    assert rc == nv.PKV_E_LIMIT
