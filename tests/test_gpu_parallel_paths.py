"""The device paths of cachegen_b200.parallel that need no second GPU: the two-dimensional token-range
copy and the pipelined decode + delivery, on one device, against a plain decode_many."""
import pytest
import torch

pytestmark = pytest.mark.gpu

MODEL_7B = "lmsys/longchat-7b-16k"


def make_serde(chunk_size=256):
    from cachegen_b200.config import LMCacheEngineConfig, LMCacheEngineMetadata
    from cachegen_b200.serde import CacheGenDeserializer, CacheGenSerializer
    config = LMCacheEngineConfig.from_defaults(chunk_size=chunk_size)
    metadata = LMCacheEngineMetadata(model_name=MODEL_7B, world_size=1, worker_id=0, fmt="vllm")
    return CacheGenSerializer(config, metadata), CacheGenDeserializer(config, metadata, out_dtype=torch.float16)


def test_token_range_copy_moves_exactly_that_range():
    from cachegen_b200.parallel import copy_token_range_async
    L, T, H, D = 5, 40, 3, 16
    src = torch.randn(L, 2, T, H, D, device="cuda").to(torch.float16)
    dst = torch.full((L, 2, T, H, D), -7.0, dtype=torch.float16, device="cuda")
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    copy_token_range_async(dst[:, :, 8:29], src[:, :, 8:29], stream)
    torch.cuda.current_stream().wait_stream(stream)
    torch.cuda.synchronize()
    assert torch.equal(dst[:, :, 8:29], src[:, :, 8:29])
    assert bool((dst[:, :, :8] == -7.0).all()) and bool((dst[:, :, 29:] == -7.0).all())
    # a destination of another total length (the consumer's blob is usually larger than a rank's slab)
    big = torch.zeros((L, 2, 2 * T, H, D), dtype=torch.float16, device="cuda")
    copy_token_range_async(big[:, :, 50:60], src[:, :, 0:10], stream)
    stream.synchronize()
    assert torch.equal(big[:, :, 50:60], src[:, :, 0:10]) and not big[:, :, :50].any() and not big[:, :, 60:].any()
    with pytest.raises(RuntimeError):
        copy_token_range_async(dst[:, :, 0:4], src[:, :, 0:5], stream)
    with pytest.raises(RuntimeError):  # not a token range of a contiguous blob
        copy_token_range_async(dst[:, :, 0:4, :, ::2], src[:, :, 0:4, :, ::2], stream)


@pytest.mark.parametrize("parts", [1, 3, 8])
def test_pipelined_delivery_equals_a_plain_decode(parts):
    """Decode in parts into the rank's own slab, each part copied to the target while the next is decoded:
    the delivered blob must hold exactly what decode_many gives."""
    from cachegen_b200.parallel import PipelinedDelivery
    from cachegen_b200.synth import generate_kv
    L, H, D, T = 32, 2, 128, 256 * 5 + 100
    kv = generate_kv(L, H, D, T, seed=21, device="cuda", dtype=torch.float16)
    ser, de = make_serde()
    chunks = ser.encode_many(kv, 256, batch=4)
    want = de.decode_many(chunks)
    de.check_status()
    local = torch.zeros((L, 2, T, H, D), dtype=torch.float16, device="cuda")
    target = torch.zeros_like(local)
    pipe = PipelinedDelivery(de, chunks, local, target, parts=parts, target_is_local=False)
    assert len(pipe.parts) <= parts
    pipe.run()
    torch.cuda.synchronize()
    assert pipe.status() == 0
    assert torch.equal(target, want) and torch.equal(local, want)
    # straight into the target when it is this GPU's own memory: the staging slab stays untouched
    local.zero_()
    target.zero_()
    direct = PipelinedDelivery(de, chunks, local, target, parts=parts, target_is_local=True)
    direct.run()
    torch.cuda.synchronize()
    assert torch.equal(target, want) and not local.any()
