"""Anchor-token delta coding on the GPU (cg_quantize_cdf_delta / cg_decode_dequant_delta) against its
definition in the CPU oracle: symbols, scales, tables, streams and decoded KV, bit for bit."""
import numpy as np
import pytest
import torch

from gpu_util import bits_np, kv_rows

pytestmark = pytest.mark.gpu
MODEL_7B = "lmsys/longchat-7b-16k"


def make_serde(delta, fmt="vllm", out_dtype=torch.float16, wire_format="pickle"):
    from cachegen_b200.config import LMCacheEngineConfig, LMCacheEngineMetadata
    from cachegen_b200.serde import CacheGenDeserializer, CacheGenSerializer
    config = LMCacheEngineConfig.from_defaults(chunk_size=1024)
    metadata = LMCacheEngineMetadata(model_name=MODEL_7B, world_size=1, worker_id=0, fmt=fmt)
    return (CacheGenSerializer(config, metadata, delta=delta, wire_format=wire_format),
            CacheGenDeserializer(config, metadata, out_dtype=out_dtype, delta=delta))


def oracle_delta(oracle, kv_cpu, ser, delta, code):
    rows = kv_rows(kv_cpu)
    bins = torch.cat((ser.key_bins, ser.value_bins)).cpu().numpy().astype(np.float32)
    res = delta.residual_bins(ser.key_bins, ser.value_bins, "cpu").numpy()
    sym, mx = oracle.quantize_delta(bits_np(rows), bins, res, delta.group, code)
    cdf = oracle.calculate_cdf(sym, int(bins.max()))
    return sym, mx, cdf, bins, res


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("group,divisor,rows,T,H,D", [(4, 2, "keys", 300, 2, 64), (8, 4, "all", 256, 1, 128),
                                                     (2, 1, "keys", 40, 3, 20), (256, 2, "all", 600, 2, 64)])
def test_delta_encode_and_decode_match_the_oracle(oracle, dtype, group, divisor, rows, T, H, D):
    from cachegen_b200.serde import DeltaCoding
    from cachegen_b200.synth import generate_kv
    code = oracle.F16 if dtype == torch.float16 else oracle.BF16
    L = 32
    delta = DeltaCoding(group, divisor, rows)
    kv = generate_kv(L, H, D, T, seed=group + T, device="cpu", dtype=dtype)
    kv[5, 0, 8:12] = 0          # an all-zero anchor and all-zero residual rows
    kv[6, 0, 13] = kv[6, 0, 12]  # a residual that is exactly zero
    ser, de = make_serde(delta, out_dtype=dtype)
    eo = ser.encode(kv.cuda())
    sym, mx, cdf, bins, res = oracle_delta(oracle, kv, ser, delta, code)
    assert (eo.cdf.cpu().numpy() == cdf).all()
    assert (bits_np(eo.max_tensors_key).reshape(L, T) == mx[:L].reshape(L, T)).all()
    assert (bits_np(eo.max_tensors_value).reshape(L, T) == mx[L:].reshape(L, T)).all()
    for j, dc in enumerate(eo.data_chunks):
        want_bytes, want_len = oracle.encode_chunk(cdf, sym[:, 256 * j:256 * (j + 1)])
        assert (dc.bytestream_lengths.cpu().numpy() == want_len).all()
        assert dc.bytestream.cpu().numpy().tobytes() == want_bytes.tobytes()
    want = oracle.dequantize_delta(sym, bins, res, group, mx, code, code)
    got = de.decode(eo)
    de.check_status()
    assert (bits_np(kv_rows(got)) == want).all()
    # and it is a useful reconstruction: within the plain quantiser's error of the original on anchors
    anchors = kv_rows(got)[:, ::group].float()
    assert torch.allclose(anchors.cpu(), kv_rows(kv)[:, ::group].float(), atol=float(kv.abs().max()) / 3)


def test_delta_settings_must_match_and_plain_chunks_are_untouched(oracle):
    from cachegen_b200.serde import DeltaCoding
    from cachegen_b200.synth import generate_kv
    kv = generate_kv(32, 2, 64, 256, seed=9, device="cuda", dtype=torch.float16)
    plain_ser, plain_de = make_serde(None)
    ser, de = make_serde(DeltaCoding(4))
    # delta off: the very same chunk as before
    a, b = plain_ser.encode(kv), make_serde(None)[0].encode(kv)
    assert torch.equal(a.cdf, b.cdf) and torch.equal(a.data_chunks[0].bytestream, b.data_chunks[0].bytestream)
    # containers carry a checksum of the settings: a reader configured otherwise refuses them
    flat_ser, _ = make_serde(DeltaCoding(4), wire_format="flat")
    blob = flat_ser.to_bytes(kv)
    with pytest.raises(RuntimeError, match="other bin or delta settings"):
        plain_de.from_bytes(blob)
    with pytest.raises(RuntimeError, match="other bin or delta settings"):
        make_serde(DeltaCoding(8))[1].from_bytes(blob)
    got = de.from_bytes(blob)
    assert torch.equal(got, de.decode(ser.encode(kv)))
    with pytest.raises(ValueError):
        DeltaCoding(3)
    # fewer payload bytes on smooth keys at half the residual bins
    smooth = generate_kv(32, 2, 64, 256, seed=9, key_rho=0.97, device="cuda", dtype=torch.float16)
    n_plain = sum(dc.bytestream.numel() for dc in plain_ser.encode(smooth).data_chunks)
    n_delta = sum(dc.bytestream.numel() for dc in ser.encode(smooth).data_chunks)
    assert n_delta < n_plain
