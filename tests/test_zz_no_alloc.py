"""cg_decode_dequant_static: the decode entry point for callers that cannot allocate device memory on
their decode path (an engine whose KV pool already owns all free HBM, or a worker that must keep the
device-synchronising cudaMalloc off its latency path).  It keeps the group offsets in an array built
into the library; here it is called straight through the C ABI and must reproduce, bit for bit, what
cg_decode_offsets + cg_decode_dequant give with a caller-allocated workspace -- on two calls in a row
with different inputs, so that whatever the first call leaves in the shared array cannot leak into
the second."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _encode(tokens, seed, heads):
    from cachegen_b200.config import LMCacheEngineConfig, LMCacheEngineMetadata
    from cachegen_b200.serde import CacheGenDeserializer, CacheGenSerializer
    from cachegen_b200.synth import generate_kv
    config = LMCacheEngineConfig.from_defaults(chunk_size=1024)
    meta = LMCacheEngineMetadata(model_name="lmsys/longchat-7b-16k", world_size=1, worker_id=0, fmt="vllm")
    ser = CacheGenSerializer(config, meta)
    de = CacheGenDeserializer(config, meta, out_dtype=torch.float16)
    kv = generate_kv(32, heads, 128, tokens, seed=seed, device="cpu", dtype=torch.float16).cuda()
    return ser.encode(kv), de


def _decode_static(eo, de):
    from cachegen_b200 import _lib
    plan = de.plan([eo])  # reuse the plan's device-resident inputs and job descriptors
    out = torch.full_like(plan.out, float("nan"))
    L, H, D, C, lp, NL, T = plan.dims
    o_layer, o_kv, o_token, o_head = out.stride(0), out.stride(1), out.stride(2), out.stride(3)
    lib = _lib.lib()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    for arr, n, _ in plan.batches:
        jobs = (_lib.DecodeJob * n)()
        for j in range(n):
            ctypes.memmove(ctypes.byref(jobs[j]), ctypes.byref(arr[j]), ctypes.sizeof(_lib.DecodeJob))
            jobs[j].group_off = None  # ignored by the entry point
            jobs[j].out = out.data_ptr() + (arr[j].out - plan.out.data_ptr())
        rc = lib.cg_decode_dequant_static(jobs, n, L, H, D, lp, ctypes.c_void_p(plan.bins.data_ptr()),
                                          plan.dtypes[0], plan.dtypes[1], o_layer, o_kv, o_token, o_head,
                                          ctypes.c_void_p(status.data_ptr()),
                                          ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
        assert rc == 0, lib.cg_status_string(rc)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    return out


def test_static_workspace_decode_matches_workspace_decode_twice():
    # first call: three sub-chunks of a 700-token chunk; second call: other data, other shape
    for tokens, seed, heads in ((700, 21, 4), (256, 22, 8)):
        eo, de = _encode(tokens, seed, heads)
        want = de.decode(eo)
        de.check_status()
        got = _decode_static(eo, de)
        assert not torch.isnan(got.float()).any()
        assert torch.equal(got.view(torch.int16), want.view(torch.int16))


def test_static_workspace_rejects_oversized_requests():
    from cachegen_b200 import _lib
    lib = _lib.lib()
    jobs = (_lib.DecodeJob * 40)()
    one = ctypes.c_void_p(16)  # never dereferenced: the call is rejected before anything is launched
    # 40 jobs x 2*160 rows x 64 groups of 128 channels = 819,200 entries > 131,072
    rc = lib.cg_decode_dequant_static(jobs, 40, 160, 64, 128, 33, one, 0, 0, 1, 1, 1, 1, None, None)
    assert rc == -6
    assert b"workspace" in lib.cg_status_string(rc)
