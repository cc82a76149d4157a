"""The fused product path (cg_quantize_cdf / cg_encode_chunk / cg_compact_streams / cg_decode_offsets /
cg_decode_dequant) and the serializer classes on the GPU against the CPU oracle."""
import os

import numpy as np
import pytest
import torch

from gpu_util import bits_np, kv_rows

pytestmark = pytest.mark.gpu

MODEL_7B = "lmsys/longchat-7b-16k"


def make_serde(chunk_size, fmt, model=MODEL_7B, **kw):
    from cachegen_b200.config import LMCacheEngineConfig, LMCacheEngineMetadata
    from cachegen_b200.serde import CacheGenDeserializer, CacheGenSerializer
    config = LMCacheEngineConfig.from_defaults(chunk_size=chunk_size)
    metadata = LMCacheEngineMetadata(model_name=model, world_size=1, worker_id=0, fmt=fmt)
    ser_kw = {k: v for k, v in kw.items() if k == "cachegen_config"}
    return CacheGenSerializer(config, metadata, **ser_kw), CacheGenDeserializer(config, metadata, **kw)


def oracle_encode(oracle, kv_cpu, key_bins, value_bins, dtype_code):
    """The reference pipeline on the CPU oracle for a vllm-format blob -> dict of numpy results."""
    rows = kv_rows(kv_cpu)
    bins = np.concatenate((key_bins, value_bins)).astype(np.float32)
    sym, mx = oracle.quantize(bits_np(rows), bins, dtype_code)
    cdf = oracle.calculate_cdf(sym, int(bins.max()))
    chunks = []
    T = rows.shape[1]
    for s in range(0, T, 256):
        e = min(s + 256, T)
        chunks.append(oracle.encode_chunk(cdf, sym[:, s:e, :]))
    return dict(sym=sym, max=mx, cdf=cdf, chunks=chunks, bins=bins)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("T", [1, 16, 236, 256, 700])
def test_encode_is_bit_exact_and_decode_matches_reference_formula(oracle, dtype, T):
    from cachegen_b200.synth import generate_kv
    code = oracle.F16 if dtype == torch.float16 else oracle.BF16
    L, H, D = 32, 2, 64
    kv = generate_kv(L, H, D, T, seed=T, device="cpu", dtype=dtype)
    kv[3, 0, T // 2] = 0  # an all-zero token row
    ser, de = make_serde(max(T, 256), "vllm")
    eo = ser.encode(kv.cuda())
    ref = oracle_encode(oracle, kv, ser.key_bins.cpu().numpy(), ser.value_bins.cpu().numpy(), code)

    assert (eo.cdf.cpu().numpy() == ref["cdf"]).all()
    assert (bits_np(eo.max_tensors_key).reshape(L, T) == ref["max"][:L].reshape(L, T)).all()
    assert (bits_np(eo.max_tensors_value).reshape(L, T) == ref["max"][L:].reshape(L, T)).all()
    assert eo.max_tensors_key.dtype == dtype and tuple(eo.max_tensors_key.shape) == (L, T, 1)
    assert len(eo.data_chunks) == len(ref["chunks"])
    for dc, (want_bytes, want_len) in zip(eo.data_chunks, ref["chunks"]):
        assert (dc.bytestream_lengths.cpu().numpy() == want_len).all()
        assert dc.bytestream.cpu().numpy().tobytes() == want_bytes.tobytes()
        assert dc.bytestream.dtype == torch.uint8 and dc.bytestream_lengths.dtype == torch.int32

    # decode: exact equality with the reference's fp32 formula + one cast, in every output type
    for out_dtype, out_code in ((torch.float16, oracle.F16), (torch.bfloat16, oracle.BF16)):
        de.out_dtype = out_dtype
        got = de.decode(eo)
        de.check_status()
        assert got.dtype == out_dtype and tuple(got.shape) == tuple(kv.shape)
        want = oracle.dequantize(ref["sym"].view(np.uint8), ref["bins"], ref["max"], code, out_code)
        assert (bits_np(kv_rows(got)) == want).all()


@pytest.mark.parametrize("fmt", ["vllm", "huggingface"])
def test_formats_agree_and_blobs_round_trip_through_pickle(oracle, fmt):
    from cachegen_b200.serde.cachegen_basics import CacheGenEncoderOutput
    from cachegen_b200.synth import generate_kv
    L, H, D, T = 32, 8, 128, 128
    kv = generate_kv(L, H, D, T, seed=5, device="cpu", dtype=torch.float16).cuda()
    ser_v, de_v = make_serde(256, "vllm", out_dtype=torch.float16)
    ser_h, de_h = make_serde(256, "huggingface")
    blob_v = ser_v.to_bytes(kv)
    kv_h = kv.permute(0, 1, 3, 2, 4).contiguous()
    blob_h = ser_h.to_bytes(kv_h)
    # the reference's test asserts equal lengths (LMCache/tests/test_serde.py:42); pickling a CUDA tensor
    # goes through torch's legacy storage format, which embeds each storage's address as a decimal
    # string, so two blobs of identical content can differ by a few bytes
    assert abs(len(blob_v) - len(blob_h)) <= 64
    a, b = CacheGenEncoderOutput.from_bytes(blob_v), CacheGenEncoderOutput.from_bytes(blob_h)
    assert a.num_heads == H and a.head_size == D
    assert torch.equal(a.cdf, b.cdf) and torch.equal(a.data_chunks[0].bytestream, b.data_chunks[0].bytestream)
    out_v = de_v.from_bytes(blob_v)
    out_h = de_h.from_bytes(blob_h)
    assert out_h.dtype == torch.float16 and tuple(out_h.shape) == (L, 2, H, T, D)
    assert torch.equal(out_v, out_h.permute(0, 1, 3, 2, 4))
    err = (out_v.float() - kv.float()).abs().max().item()
    assert 0 < err < kv.float().abs().max().item()


@pytest.mark.parametrize("fmt", ["vllm", "huggingface"])
@pytest.mark.parametrize("chunk_size", [16, 128, 256])
def test_reference_serde_cases(monkeypatch, fmt, chunk_size):
    """The reference's own serde tests (LMCache/tests/test_serde.py:27-76): torch.rand KV of 32 layers x
    8 heads x 128, bf16 for vllm / fp16 for huggingface, Mistral model name (QUANT_LEVEL lookup),
    chunk sizes 16/128/256 and a chunk 20 tokens short."""
    monkeypatch.setenv("QUANT_LEVEL", "2")
    from cachegen_b200.serde.cachegen_basics import CacheGenEncoderOutput
    model = "mistralai/Mistral-7B-Instruct-v0.2"
    dtype = torch.bfloat16 if fmt == "vllm" else torch.float16
    for ntok in (chunk_size, max(1, chunk_size - 20)):
        shape = [32, 2, ntok, 8, 128] if fmt == "vllm" else [32, 2, 8, ntok, 128]
        g = torch.Generator(device="cuda").manual_seed(ntok)
        kv = torch.rand(shape, dtype=dtype, device="cuda", generator=g)
        ser, de = make_serde(chunk_size, fmt, model=model)
        blob = ser.to_bytes(kv)
        eo = CacheGenEncoderOutput.from_bytes(blob)
        assert eo.num_heads == 8 and eo.head_size == 128
        decoded = de.from_bytes(blob)
        de.check_status()
        assert decoded.shape == kv.shape and decoded.dtype == dtype
        assert decoded.mean() != 0
        assert (decoded.float() - kv.float()).abs().max() < 0.2  # rand in [0,1): step is at most 1/7
    with pytest.raises(RuntimeError, match="chunk_size"):
        big = torch.rand([32, 2, chunk_size + 1, 8, 128] if fmt == "vllm" else [32, 2, 8, chunk_size + 1, 128],
                         dtype=dtype, device="cuda")
        de.from_bytes(ser.to_bytes(big))


def test_quality_levels_and_70b_config(oracle):
    """Half and quarter bin counts (tables of 17 and 9 entries) and the 80-layer configuration."""
    from cachegen_b200.serde.cachegen_basics import CacheGenConfig
    from cachegen_b200.synth import generate_kv
    base = CacheGenConfig.from_model_name(MODEL_7B)
    for cfg, T in ((base.with_bins_divided(2), 100), (base.with_bins_divided(4), 256)):
        kv = generate_kv(32, 1, 128, T, seed=cfg.max_bins, device="cpu", dtype=torch.float16)
        ser, de = make_serde(256, "vllm", cachegen_config=cfg, out_dtype=torch.float16)
        eo = ser.encode(kv.cuda())
        assert eo.cdf.shape[2] == cfg.max_bins + 1
        ref = oracle_encode(oracle, kv, ser.key_bins.cpu().numpy(), ser.value_bins.cpu().numpy(), oracle.F16)
        assert (eo.cdf.cpu().numpy() == ref["cdf"]).all()
        assert eo.data_chunks[0].bytestream.cpu().numpy().tobytes() == ref["chunks"][0][0].tobytes()
        want = oracle.dequantize(ref["sym"].view(np.uint8), ref["bins"], ref["max"], oracle.F16, oracle.F16)
        assert (bits_np(kv_rows(de.decode(eo))) == want).all()
    kv = generate_kv(80, 1, 128, 64, seed=3, device="cpu", dtype=torch.float16)
    ser, de = make_serde(256, "vllm", model="Yukang/LongAlpaca-70B-16k", out_dtype=torch.float16)
    eo = ser.encode(kv.cuda())
    ref = oracle_encode(oracle, kv, ser.key_bins.cpu().numpy(), ser.value_bins.cpu().numpy(), oracle.F16)
    assert eo.data_chunks[0].bytestream.cpu().numpy().tobytes() == ref["chunks"][0][0].tobytes()
    want = oracle.dequantize(ref["sym"].view(np.uint8), ref["bins"], ref["max"], oracle.F16, oracle.F16)
    assert (bits_np(kv_rows(de.decode(eo))) == want).all()


def test_odd_channel_count_takes_the_scalar_path(oracle):
    """Head size 20 (not a multiple of 8) and a non-contiguous input."""
    from cachegen_b200.serde.cachegen_encoder import quantize_and_tables
    from cachegen_b200.serde.cachegen_basics import CacheGenConfig, make_key_bins, make_value_bins
    g = torch.Generator().manual_seed(2)
    L, T, H, D = 32, 40, 3, 20
    full = torch.randn(L, 2, T, H, D + 4, generator=g).to(torch.float16)
    kv = full[..., :D]
    cfg = CacheGenConfig.from_model_name(MODEL_7B)
    kb, vb = make_key_bins(cfg), make_value_bins(cfg)
    sym, scales, cdf = quantize_and_tables(kv.cuda(), kb, vb, 32)
    rows = kv_rows(kv.contiguous())
    bins = torch.cat((kb, vb)).cpu().numpy()
    want_sym, want_max = oracle.quantize(bits_np(rows), bins, oracle.F16)
    assert (sym.cpu().numpy() == want_sym).all()
    assert (bits_np(scales) == want_max.reshape(2 * L, T)).all()
    assert (cdf.cpu().numpy() == oracle.calculate_cdf(want_sym, 32)).all()


def test_full_size_chunk_properties():
    """One chunk at the benchmark's full width (32 layers x 32 heads x 128, 256 tokens): encode ->
    decode -> re-encode is a fixed point, and the decoded values obey the quantiser's error bound."""
    from cachegen_b200.synth import generate_kv
    kv = generate_kv(32, 32, 128, 256, seed=1, device="cuda", dtype=torch.float16)
    ser, de = make_serde(256, "vllm", out_dtype=torch.float16)
    eo = ser.encode(kv)
    out = de.decode(eo)
    de.check_status()
    eo2 = ser.encode(out)
    # re-quantising dequantised values with the same per-token maximum reproduces the symbols, so the
    # second encode must give the same tables and streams whenever the maximum itself is a grid point
    same = torch.equal(eo2.max_tensors_key, eo.max_tensors_key) and torch.equal(eo2.max_tensors_value, eo.max_tensors_value)
    assert same
    assert torch.equal(eo2.cdf, eo.cdf)
    assert torch.equal(eo2.data_chunks[0].bytestream, eo.data_chunks[0].bytestream)
    L = 32
    cq = torch.cat((ser.key_bins, ser.value_bins)).div(2, rounding_mode="floor") - 1
    step = torch.cat((eo.max_tensors_key, eo.max_tensors_value)).float().reshape(2 * L, 256, 1) / cq[:, None, None]
    err = (kv_rows(out).float() - kv_rows(kv).float()).abs()
    # half a quantisation step, plus the rounding of the result to fp16 (half an ulp at the row maximum)
    assert (err <= 0.5 * step * 1.001 + step * cq[:, None, None] * 2.0 ** -10 + 1e-6).all()


def test_benchmark_config_one_full_round_trip_against_the_oracle(oracle):
    """The first benchmark configuration at full size: Llama-7B shape (32 layers x 32 heads x 128, fp16), 1,024
    tokens, seed 0, 7B-default bins, one serializer call per 256 tokens.  Every table, length and
    stream byte and every decoded fp16 value is compared with the CPU oracle (2.7e8 symbols)."""
    from cachegen_b200.synth import WORKLOADS, generate_kv
    spec = WORKLOADS["llama7b-1k"]
    L, H, D, T = spec["num_layers"], spec["num_heads"], spec["head_size"], spec["num_tokens"]
    kv = generate_kv(L, H, D, T, spec["seed"], key_rho=spec["key_rho"], device="cpu", dtype=torch.float16)
    ser, de = make_serde(256, "vllm", model=spec["model_name"], out_dtype=torch.float16)
    kb, vb = ser.key_bins.cpu().numpy(), ser.value_bins.cpu().numpy()
    chunks = []
    for s in range(0, T, 256):
        part = kv[:, :, s:s + 256].contiguous()
        eo = ser.encode(part.cuda())
        ref = oracle_encode(oracle, part, kb, vb, oracle.F16)
        assert (eo.cdf.cpu().numpy() == ref["cdf"]).all()
        want_bytes, want_len = ref["chunks"][0]
        assert (eo.data_chunks[0].bytestream_lengths.cpu().numpy() == want_len).all()
        assert eo.data_chunks[0].bytestream.cpu().numpy().tobytes() == want_bytes.tobytes()
        chunks.append((eo, ref))
    out = de.decode_many([c[0] for c in chunks])
    de.check_status()
    assert tuple(out.shape) == (L, 2, T, H, D)
    for i, (_, ref) in enumerate(chunks):
        want = oracle.dequantize(ref["sym"].view(np.uint8), ref["bins"], ref["max"], oracle.F16, oracle.F16)
        assert (bits_np(kv_rows(out[:, :, i * 256:(i + 1) * 256])) == want).all()


@pytest.mark.parametrize("chunk_tokens", [256, 512])
def test_encode_many_equals_chunk_by_chunk_encode(chunk_tokens):
    from cachegen_b200.synth import generate_kv
    T = 700
    kv = generate_kv(32, 2, 128, T, seed=11, device="cuda", dtype=torch.float16)
    ser, de = make_serde(chunk_tokens, "vllm", out_dtype=torch.float16)
    many = ser.encode_many(kv, batch=2)
    assert len(many) == (T + chunk_tokens - 1) // chunk_tokens
    for i, eo in enumerate(many):
        one = ser.encode(kv[:, :, i * chunk_tokens:(i + 1) * chunk_tokens])
        assert torch.equal(eo.cdf, one.cdf)
        assert torch.equal(eo.max_tensors_key, one.max_tensors_key) and torch.equal(eo.max_tensors_value, one.max_tensors_value)
        assert len(eo.data_chunks) == len(one.data_chunks)
        for a, b in zip(eo.data_chunks, one.data_chunks):
            assert a.ntokens == b.ntokens and torch.equal(a.bytestream, b.bytestream)
            assert torch.equal(a.bytestream_lengths, b.bytestream_lengths)
            assert a.bytestream.untyped_storage().nbytes() == a.bytestream.numel()  # pickles without padding
    want = torch.cat([de.decode(ser.encode(kv[:, :, s:s + chunk_tokens])) for s in range(0, T, chunk_tokens)], dim=2)
    assert torch.equal(de.decode_many(many), want)


@pytest.mark.parametrize("streams,batch", [(1, 1), (2, 3), (3, 16), (4, 2)])
def test_encode_many_on_side_streams_gives_the_same_chunks(streams, batch):
    """Consecutive chunks go to side streams in turn; the caller's stream -- here not the default one, with
    the cache produced on it just before the call -- waits for them, so the chunks can be used at once."""
    from cachegen_b200.synth import generate_kv
    T = 256 * 6 + 40
    base = generate_kv(32, 2, 128, T, seed=12, device="cuda", dtype=torch.float16)
    ser, de = make_serde(256, "vllm", out_dtype=torch.float16)
    want = [ser.encode(base[:, :, s:s + 256]) for s in range(0, T, 256)]
    want_kv = de.decode_many(want)
    torch.cuda.synchronize()
    caller = torch.cuda.Stream()
    with torch.cuda.stream(caller):
        kv = base * 1.0  # made on the caller's stream: the side streams must wait for it
        many = ser.encode_many(kv, batch=batch, streams=streams)
        got_kv = de.decode_many(many)
    caller.synchronize()
    assert len(many) == len(want)
    for a, b in zip(many, want):
        assert torch.equal(a.cdf, b.cdf) and torch.equal(a.max_tensors_key, b.max_tensors_key)
        assert torch.equal(a.data_chunks[0].bytestream, b.data_chunks[0].bytestream)
        assert torch.equal(a.data_chunks[0].bytestream_lengths, b.data_chunks[0].bytestream_lengths)
    assert torch.equal(got_kv, want_kv)


@pytest.mark.parametrize("L,T", [(32, 256 * 8 + 100), (4, 8192)])
def test_whole_context_call_decodes_to_the_values_of_chunked_calls(oracle, L, T):
    """One serializer call over the whole context (chunk_size = context length, as the reference's
    evaluation scripts call it: one table per stream group over all tokens, one stream per 256-token
    sub-chunk).  Quantisation is per token row, so the decoded values cannot depend on how the context was
    cut into calls: the result must equal the chunk-by-chunk result bit for bit; its tables and first
    sub-chunk are checked against the oracle, and the blob goes through bytes and back."""
    from cachegen_b200.synth import generate_kv
    kv = generate_kv(L, 2, 128, T, seed=17, device="cuda", dtype=torch.float16)
    # the 7B settings cover 32 layers; a shorter blob uses the first L of them, as the reference would
    whole_ser, whole_de = make_serde(T, "vllm", out_dtype=torch.float16)
    ser, de = make_serde(256, "vllm", out_dtype=torch.float16)
    if L != 32:
        from cachegen_b200.serde.cachegen_basics import CacheGenConfig
        cfg = CacheGenConfig.from_model_name(MODEL_7B).layer_slice(0, L)
        whole_ser, whole_de = make_serde(T, "vllm", out_dtype=torch.float16, cachegen_config=cfg)
        ser, de = make_serde(256, "vllm", out_dtype=torch.float16, cachegen_config=cfg)
    eo = whole_ser.encode(kv)
    nsub = (T + 255) // 256
    assert len(eo.data_chunks) == nsub and [c.ntokens for c in eo.data_chunks] == [min(256, T - 256 * j) for j in range(nsub)]
    got = whole_de.decode(eo)
    want = de.decode_many(ser.encode_many(kv))
    whole_de.check_status()
    de.check_status()
    assert torch.equal(got, want)
    assert torch.equal(whole_de.from_bytes(whole_ser.to_bytes(kv)), want)
    # tables over all T tokens and the first sub-chunk's streams against the oracle (a few layers of it)
    nl = min(L, 2)
    from cachegen_b200.serde.cachegen_basics import make_key_bins, make_value_bins
    kb = make_key_bins(whole_ser.cachegen_config, "cpu").numpy()[:nl]
    vb = make_value_bins(whole_ser.cachegen_config, "cpu").numpy()[:nl]
    ref = oracle_encode(oracle, kv[:nl].cpu(), kb, vb, oracle.F16)
    rows = list(range(nl)) + list(range(L, L + nl))
    if int(max(kb.max(), vb.max())) == eo.cdf.shape[2] - 1:
        assert (eo.cdf[rows].cpu().numpy() == ref["cdf"]).all()
        want_bytes, want_len = ref["chunks"][0]
        assert (eo.data_chunks[0].bytestream_lengths[rows].cpu().numpy() == want_len).all()


def test_layer_shard_encodes_like_the_whole_model():
    """Layers 20..29 of the 70B configuration have 32 key bins and 16 value bins.  Encoded as a shard
    with the whole model's table length they give exactly the whole model's tables, lengths and
    decoded values for those layers."""
    from cachegen_b200.serde.cachegen_basics import CacheGenConfig
    from cachegen_b200.synth import generate_kv
    model = "Yukang/LongAlpaca-70B-16k"
    full = CacheGenConfig.from_model_name(model)
    kv = generate_kv(80, 1, 128, 64, seed=3, device="cuda", dtype=torch.float16)
    ser, de = make_serde(256, "vllm", model=model, out_dtype=torch.float16)
    whole = ser.encode(kv)
    want = de.decode(whole)
    lo, hi = 20, 30
    part_cfg = full.layer_slice(lo, hi)
    with pytest.raises(RuntimeError, match="must match"):
        make_serde(256, "vllm", model=model, cachegen_config=part_cfg)[0].encode(kv[lo:hi])
    from cachegen_b200.config import LMCacheEngineConfig, LMCacheEngineMetadata
    from cachegen_b200.serde import CacheGenDeserializer, CacheGenSerializer
    config = LMCacheEngineConfig.from_defaults(chunk_size=256)
    meta = LMCacheEngineMetadata(model_name=model, world_size=8, worker_id=2, fmt="vllm")
    pser = CacheGenSerializer(config, meta, cachegen_config=part_cfg, table_max_bins=full.max_bins)
    pde = CacheGenDeserializer(config, meta, cachegen_config=part_cfg, out_dtype=torch.float16)
    part = pser.encode(kv[lo:hi])
    rows = list(range(lo, hi)) + list(range(80 + lo, 80 + hi))
    assert torch.equal(part.cdf, whole.cdf[rows])
    assert torch.equal(part.data_chunks[0].bytestream_lengths, whole.data_chunks[0].bytestream_lengths[rows])
    assert torch.equal(pde.decode(part), want[lo:hi])
    assert torch.equal(pde.decode(pser.encode_flat(kv[lo:hi])), want[lo:hi])


@pytest.mark.parametrize("level", ["1", "2", "3"])
def test_quant_levels_of_the_mistral_lookup_against_the_oracle(monkeypatch, oracle, level):
    """The three QUANT_LEVEL settings (cachegen_basics.py:33-68 of the reference): level 1 mixes 16 and
    12 bins (17-entry tables, 11-symbol rows), level 3 is 32 bins everywhere."""
    monkeypatch.setenv("QUANT_LEVEL", level)
    from cachegen_b200.synth import generate_kv
    model = "mistralai/Mistral-7B-Instruct-v0.2"
    T = 200
    kv = generate_kv(32, 3, 40, T, seed=int(level), device="cpu", dtype=torch.float16)  # 120 channels: a ragged slab
    ser, de = make_serde(256, "vllm", model=model, out_dtype=torch.float16)
    eo = ser.encode(kv.cuda())
    ref = oracle_encode(oracle, kv, ser.key_bins.cpu().numpy(), ser.value_bins.cpu().numpy(), oracle.F16)
    assert eo.cdf.shape[2] == (17 if level == "1" else 33)
    assert (eo.cdf.cpu().numpy() == ref["cdf"]).all()
    assert eo.data_chunks[0].bytestream.cpu().numpy().tobytes() == ref["chunks"][0][0].tobytes()
    want = oracle.dequantize(ref["sym"].view(np.uint8), ref["bins"], ref["max"], oracle.F16, oracle.F16)
    assert (bits_np(kv_rows(de.decode(eo))) == want).all()
    assert (bits_np(kv_rows(de.decode(ser.encode_flat(kv.cuda())))) == want).all()
    de.check_status()


@pytest.mark.parametrize("fmt,T", [("vllm", 256), ("huggingface", 300)])
def test_levels_encoded_together_equal_levels_encoded_alone(monkeypatch, fmt, T):
    """encode_levels (shared max|x| pass, one host synchronisation) returns, per QUANT_LEVEL, the blob
    a serializer configured for that level alone produces, and the sizes drive the level choice."""
    from cachegen_b200.serde.adaptation import config_selection, level_sizes
    from cachegen_b200.serde.cachegen_basics import CacheGenConfig
    from cachegen_b200.synth import generate_kv
    model = "mistralai/Mistral-7B-Instruct-v0.2"
    kv = generate_kv(32, 2, 64, T, seed=T, device="cuda", dtype=torch.bfloat16)
    blob = kv if fmt == "vllm" else kv.permute(0, 1, 3, 2, 4).contiguous()
    configs, alone = [], []
    for level in ("1", "2", "3"):
        monkeypatch.setenv("QUANT_LEVEL", level)
        configs.append(CacheGenConfig.from_model_name(model))
        ser, de = make_serde(512, fmt, model=model)
        alone.append(ser.encode(blob))
    together = ser.encode_levels(blob, configs)
    assert len(together) == 3
    for a, b in zip(alone, together):
        assert torch.equal(a.cdf, b.cdf)
        assert torch.equal(a.max_tensors_key, b.max_tensors_key) and torch.equal(a.max_tensors_value, b.max_tensors_value)
        assert len(a.data_chunks) == len(b.data_chunks)
        for x, y in zip(a.data_chunks, b.data_chunks):
            assert x.ntokens == y.ntokens and torch.equal(x.bytestream, y.bytestream)
            assert torch.equal(x.bytestream_lengths, y.bytestream_lengths)
    sizes = level_sizes(together)
    assert sizes[1] < sizes[2] < sizes[3]
    # a link that carries level 2 but not level 3 within the chunk's share of the target
    bw = sizes[2] * 8 / 1e9 / 0.09
    ttft, cfg = config_selection([bw], chunk_delay=1.0, slo=0.1, sizes=[sizes])
    assert cfg == [2] and abs(ttft - 0.09) < 1e-9


def test_gqa_long_context_shape_decodes_streams_the_oracle_encoded(oracle):
    """The third benchmark configuration's shape (32 layers x 8 KV heads x 128, key rho 0.95, seed 2) at
    three chunks: decode only, from blobs whose tables and streams come from the CPU oracle, not from
    this package's encoder; every decoded value against the oracle's dequantisation."""
    from cachegen_b200.serde.cachegen_basics import CacheGenGPUBytestream, CacheGenGPUEncoderOutput
    from cachegen_b200.synth import WORKLOADS, generate_kv
    spec = WORKLOADS["mistral7b-gqa-32k"]
    L, H, D, T = spec["num_layers"], spec["num_heads"], spec["head_size"], 768
    kv = generate_kv(L, H, D, T, spec["seed"], key_rho=spec["key_rho"], device="cpu", dtype=torch.float16)
    ser, de = make_serde(256, "vllm", model=spec["model_name"], out_dtype=torch.float16)
    kb, vb = ser.key_bins.cpu().numpy(), ser.value_bins.cpu().numpy()
    blobs, wants = [], []
    for s in range(0, T, 256):
        part = kv[:, :, s:s + 256].contiguous()
        ref = oracle_encode(oracle, part, kb, vb, oracle.F16)
        stream_bytes, lengths = ref["chunks"][0]
        mx = torch.from_numpy(ref["max"].reshape(2 * L, 256).view(np.float16).copy())
        blobs.append(CacheGenGPUEncoderOutput(
            [CacheGenGPUBytestream(torch.from_numpy(stream_bytes.copy()).cuda(),
                                   torch.from_numpy(lengths.astype(np.int32).reshape(2 * L, H * D)).cuda(), 256)],
            torch.from_numpy(ref["cdf"].copy()).cuda(), mx[:L].unsqueeze(-1).cuda(), mx[L:].unsqueeze(-1).cuda(), H, D))
        wants.append(oracle.dequantize(ref["sym"].view(np.uint8), ref["bins"], ref["max"], oracle.F16, oracle.F16))
    out = de.decode_many(blobs)
    de.check_status()
    assert tuple(out.shape) == (L, 2, T, H, D)
    for i, want in enumerate(wants):
        assert (bits_np(kv_rows(out[:, :, i * 256:(i + 1) * 256])) == want).all()
    # the same blobs through the pickle, one by one
    got = de.from_bytes(blobs[1].to_bytes())
    assert (bits_np(kv_rows(got)) == wants[1]).all()


def test_blob_writer_and_loader_on_cuda_tensors_agree_with_pickle():
    """to_bytes / from_bytes against plain pickle on an encoded chunk whose tensors are on the GPU."""
    import io
    import pickle
    from cachegen_b200.serde.cachegen_basics import CacheGenGPUEncoderOutput
    from cachegen_b200.synth import generate_kv
    kv = generate_kv(32, 2, 128, 300, seed=8, device="cuda", dtype=torch.float16)
    ser, de = make_serde(512, "vllm", out_dtype=torch.float16)
    eo = ser.encode(kv)
    f = io.BytesIO()
    pickle.dump(eo, f)
    blob = eo.to_bytes()
    assert blob == f.getvalue()
    back, plain = CacheGenGPUEncoderOutput.from_bytes(blob), pickle.load(io.BytesIO(blob))
    assert back.cdf.is_cuda and torch.equal(back.cdf, plain.cdf) and torch.equal(back.max_tensors_key, plain.max_tensors_key)
    for a, b in zip(back.data_chunks, plain.data_chunks):
        assert torch.equal(a.bytestream, b.bytestream) and torch.equal(a.bytestream_lengths, b.bytestream_lengths)
    assert torch.equal(de.from_bytes(blob), de.decode(eo))
    # two loads in a row share the thread's staging memory: the first one's tensors must survive the second
    first = CacheGenGPUEncoderOutput.from_bytes(blob)
    second = CacheGenGPUEncoderOutput.from_bytes(ser.to_bytes(kv * 0.5))
    torch.cuda.synchronize()
    assert torch.equal(first.cdf, plain.cdf) and torch.equal(first.data_chunks[1].bytestream, plain.data_chunks[1].bytestream)
    assert not torch.equal(second.max_tensors_key, first.max_tensors_key)


def test_from_bytes_many_equals_from_bytes_chunk_by_chunk():
    from cachegen_b200.config import LMCacheEngineConfig, LMCacheEngineMetadata
    from cachegen_b200.serde import CacheGenSerializer
    from cachegen_b200.synth import generate_kv
    kv = generate_kv(32, 2, 128, 256 * 5, seed=12, device="cuda", dtype=torch.float16)
    ser, de = make_serde(256, "vllm", out_dtype=torch.float16)
    flat_ser = CacheGenSerializer(LMCacheEngineConfig.from_defaults(chunk_size=256),
                                  LMCacheEngineMetadata(model_name=MODEL_7B, world_size=1, worker_id=0, fmt="vllm"),
                                  wire_format="flat")
    parts = [kv[:, :, s:s + 256] for s in range(0, kv.shape[2], 256)]
    blobs = [(flat_ser if i == 2 else ser).to_bytes(p) for i, p in enumerate(parts)]   # one CGB2 container among pickles
    want = torch.cat([de.from_bytes(b) for b in blobs], dim=2)
    got = de.from_bytes_many(blobs)
    de.check_status()
    assert torch.equal(got, want)


@pytest.mark.parametrize("H,D", [(3, 21), (5, 26), (1, 130)])
def test_decode_kernels_of_both_layouts_against_the_oracle(oracle, H, D):
    """An odd head size cannot use the two-channels-per-thread kernel (its packed 32-bit stores need
    both channels of a pair in one head): the one-channel-per-thread kernel takes over.  Even head
    sizes that leave the last 128-channel group partly empty run the paired kernel with idle lanes."""
    from cachegen_b200.synth import generate_kv
    L, T = 32, 300
    kv = generate_kv(L, H, D, T, seed=H * D, device="cpu", dtype=torch.float16)
    ser, de = make_serde(512, "vllm", out_dtype=torch.float16)
    eo = ser.encode(kv.cuda())
    ref = oracle_encode(oracle, kv, ser.key_bins.cpu().numpy(), ser.value_bins.cpu().numpy(), oracle.F16)
    for dc, (want_bytes, want_len) in zip(eo.data_chunks, ref["chunks"]):
        assert (dc.bytestream_lengths.cpu().numpy() == want_len).all()
        assert dc.bytestream.cpu().numpy().tobytes() == want_bytes.tobytes()
    want = oracle.dequantize(ref["sym"].view(np.uint8), ref["bins"], ref["max"], oracle.F16, oracle.F16)
    got = de.decode(eo)
    de.check_status()
    assert (bits_np(kv_rows(got)) == want).all()
    # the same into a blob whose token stride is odd (a view of a wider allocation): no packed stores
    wide = torch.zeros((L, 2, T, H, D + 1), dtype=torch.float16, device="cuda")
    view = wide[..., :D]
    from cachegen_b200.serde.cachegen_decoder import DecodePlan
    bins = torch.cat((de.key_bins, de.value_bins))
    try:
        plan = DecodePlan([eo], bins, "vllm", torch.float16, out=view)
    except RuntimeError:
        return  # the plan insists on a contiguous blob: nothing more to check here
    plan.run()
    assert (bits_np(kv_rows(view.contiguous())) == want).all()
    assert not wide[..., D].any()
