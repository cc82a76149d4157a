"""The CGB2 container on the GPU: decoding it gives bit for bit what decoding the reference-format
blob of the same chunk gives, with every table form, and the byte-count forms fall back to full tables
when a count does not fit a byte."""
import numpy as np
import pytest
import torch

from gpu_util import bits_np, kv_rows
from test_gpu_serde import MODEL_7B, make_serde, oracle_encode

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("fmt,dtype,T", [("vllm", torch.float16, 700), ("huggingface", torch.bfloat16, 256),
                                         ("vllm", torch.bfloat16, 37)])
def test_flat_container_decodes_like_the_pickle_blob(oracle, fmt, dtype, T):
    from cachegen_b200.serde import flat_format as ff
    from cachegen_b200.synth import generate_kv
    L, H, D = 32, 4, 64
    kv = generate_kv(L, H, D, T, seed=T, device="cpu", dtype=dtype).cuda()
    blob_kv = kv if fmt == "vllm" else kv.permute(0, 1, 3, 2, 4).contiguous()
    ser, de = make_serde(1024, fmt, out_dtype=torch.float16)
    want = de.decode(ser.encode(blob_kv))
    sizes = {}
    kinds = {True: ff.TABLES_SPARSE, "counts": ff.TABLES_COUNTS, False: ff.TABLES_CDF}
    for compact in (True, "counts", False):
        chunk = ser.encode_flat(blob_kv, compact_tables=compact)
        # tables over more than 255 tokens can hold counts that do not fit a byte: full tables then
        assert chunk.header.table_kind == (kinds[compact] if T <= 256 else ff.TABLES_CDF)
        assert chunk.header.length_kind == ff.LENGTHS_U16 and chunk.header.nsub == (T + 255) // 256
        got = de.decode(chunk)
        de.check_status()
        assert torch.equal(got.view(torch.int16), want.view(torch.int16))
        sizes[compact] = chunk.header.total
        # through bytes, and from pinned host memory
        raw = chunk.tobytes()
        assert ff.is_flat(raw) and len(raw) == chunk.header.total
        assert torch.equal(de.from_bytes(raw).view(torch.int16), want.view(torch.int16))
        assert torch.equal(de.decode(chunk.pin_memory()).view(torch.int16), want.view(torch.int16))
    assert sizes[True] < sizes["counts"] < sizes[False] or T > 256
    # streams in the container are the oracle's
    if fmt == "vllm" and dtype == torch.float16:
        ref = oracle_encode(oracle, kv.cpu(), ser.key_bins.cpu().numpy(), ser.value_bins.cpu().numpy(), oracle.F16)
        chunk = ser.encode_flat(blob_kv)
        for j, (want_bytes, want_len) in enumerate(ref["chunks"]):
            assert chunk.payload(j).cpu().numpy().tobytes() == want_bytes.tobytes()
            assert (chunk.lengths(j).cpu().numpy().view(np.uint16) == want_len).all()
        assert (bits_np(chunk.scales()) == ref["max"].reshape(2 * L, T)).all()


def test_flat_serializer_wire_format_and_mixed_batches():
    from cachegen_b200.config import LMCacheEngineConfig, LMCacheEngineMetadata
    from cachegen_b200.serde import CacheGenSerializer
    from cachegen_b200.synth import generate_kv
    kv = generate_kv(32, 2, 128, 512, seed=9, device="cuda", dtype=torch.float16)
    ser, de = make_serde(256, "vllm", out_dtype=torch.float16)
    config = LMCacheEngineConfig.from_defaults(chunk_size=256)
    meta = LMCacheEngineMetadata(model_name=MODEL_7B, world_size=1, worker_id=0, fmt="vllm")
    flat_ser = CacheGenSerializer(config, meta, wire_format="flat")
    a, b = kv[:, :, :256], kv[:, :, 256:]
    blob = flat_ser.to_bytes(a)
    assert blob[:4] == b"CGB2"
    want = torch.cat((de.decode(ser.encode(a)), de.decode(ser.encode(b))), dim=2)
    assert torch.equal(de.from_bytes(blob), want[:, :, :256])
    # one call, one chunk in each container
    got = de.decode_many([ser.encode(a), flat_ser.encode_flat(b)])
    assert torch.equal(got, want)
    got = de.decode_many_host([flat_ser.encode_flat(a).pin_memory(), flat_ser.encode_flat(b).pin_memory()], groups=2)
    de.check_status()
    assert torch.equal(got, want)


def test_byte_counts_fall_back_when_a_count_overflows():
    """A channel that sits at the row maximum for all 256 tokens has 256 occurrences of a non-centre
    symbol: the byte-count tables cannot hold that, so the container carries full tables."""
    from cachegen_b200.serde import flat_format as ff
    g = torch.Generator().manual_seed(3)
    L, H, D, T = 32, 1, 128, 256
    kv = torch.randn(L, 2, T, H, D, generator=g).clamp(-2, 2).to(torch.float16)
    kv[5, 0, :, 0, 7] = 3.0  # always the largest value of its token row -> always the top symbol
    kv = kv.cuda()
    ser, de = make_serde(256, "vllm", out_dtype=torch.float16)
    chunk = ser.encode_flat(kv)
    assert chunk.header.table_kind == ff.TABLES_CDF
    want = de.decode(ser.encode(kv))
    assert torch.equal(de.decode(chunk), want)
    kv[5, 0, 100, 0, 7] = 0.0  # 255 + 1: fits again
    chunk = ser.encode_flat(kv)
    assert chunk.header.table_kind == ff.TABLES_SPARSE
    assert torch.equal(de.decode(chunk), de.decode(ser.encode(kv)))
    chunk = ser.encode_flat(kv, compact_tables="counts")
    assert chunk.header.table_kind == ff.TABLES_COUNTS
    assert torch.equal(de.decode(chunk), de.decode(ser.encode(kv)))


def test_mismatched_bins_are_refused_not_misread():
    from cachegen_b200.serde.cachegen_basics import CacheGenConfig
    from cachegen_b200.synth import generate_kv
    kv = generate_kv(32, 1, 128, 64, seed=1, device="cuda", dtype=torch.float16)
    half = CacheGenConfig.from_model_name(MODEL_7B).with_bins_divided(2)
    ser, _ = make_serde(256, "vllm", cachegen_config=half)
    _, de_full = make_serde(256, "vllm")
    with pytest.raises(RuntimeError):
        de_full.decode(ser.encode_flat(kv))  # 17-entry tables against a 33-entry configuration's counts


def test_corrupt_lengths_in_a_container_are_flagged_not_followed():
    """Lengths that do not add up to the payload (or run far past it) must be reported through the
    status word; the decode still completes and touches nothing outside the container."""
    from cachegen_b200.serde import flat_format as ff
    from cachegen_b200.synth import generate_kv
    kv = generate_kv(32, 1, 128, 100, seed=4, device="cuda", dtype=torch.float16)
    ser, de = make_serde(256, "vllm", out_dtype=torch.float16)
    chunk = ser.encode_flat(kv)
    good = de.decode(chunk)
    de.check_status()
    bad = ff.FlatChunk(chunk.blob.clone(), chunk.header)
    ln = bad.lengths(0)
    ln[3, 17] = 30000          # one stream claims far more bytes than the payload holds
    ln[40, :] = 0              # a whole row of empty streams
    out = de.decode(bad)
    with pytest.raises(RuntimeError, match="lengths"):
        de.check_status()
    torch.cuda.synchronize()
    assert out.shape == good.shape
    # rows before the first damaged stream are untouched by the damage
    assert torch.equal(out[:3, 0], good[:3, 0])
    # and the decoder is usable afterwards
    assert torch.equal(de.decode(chunk), good)
    de.check_status()


def sparse_tables_np(counts, bins, C):
    """The sparse table parts from the dense byte counts, in numpy (the layout include/cachegen_b200.h
    gives for CG_TABLES_SPARSE)."""
    from cachegen_b200.serde import flat_format as ff
    nrows, G = len(bins), (C + 127) // 128
    row_off = ff.table_row_offsets(torch.tensor(bins), C)
    moffs = ff.mask_row_offsets(torch.tensor(bins), C)
    off_masks, off_counts = ff.sparse_parts(nrows, C, moffs[-1])
    goff = np.zeros(nrows * G + 1, np.uint32)
    masks = np.zeros(off_counts - off_masks, np.uint8)
    packed = []
    for r, b in enumerate(bins):
        n = 2 * (int(b) // 2 - 1)
        dense = counts[row_off[r]:row_off[r] + n * C].reshape(n, C)       # [symbol][channel]
        m = ((dense != 0).astype(np.uint64) << np.arange(n, dtype=np.uint64)[:, None]).sum(0)
        mt = np.uint16 if n <= 16 else np.uint32
        masks[moffs[r]:moffs[r] + C * np.dtype(mt).itemsize] = m.astype(mt).view(np.uint8)
        for g in range(G):
            goff[r * G + g] = sum(len(x) for x in packed)
            for c in range(128 * g, min(C, 128 * g + 128)):
                col = dense[:, c]
                packed.append(col[col != 0])
    goff[-1] = sum(len(x) for x in packed)
    head = np.zeros(off_masks, np.uint8)
    head[:goff.nbytes] = goff.view(np.uint8)
    return np.concatenate([head, masks] + packed)


@pytest.mark.parametrize("H,D,T", [(4, 64, 256), (1, 120, 77), (3, 40, 200)])
def test_sparse_tables_hold_the_byte_counts_without_their_zeros(H, D, T):
    """Byte for byte the layout the header describes, from the dense counts of the same chunk; ragged
    channel counts (not a multiple of 128) and odd ones (2-byte mask rows before 4-byte ones)."""
    from cachegen_b200.serde import flat_format as ff
    from cachegen_b200.synth import generate_kv
    kv = generate_kv(32, H, D, T, seed=H * D + T, device="cuda", dtype=torch.float16)
    ser, de = make_serde(256, "vllm", out_dtype=torch.float16)
    dense = ser.encode_flat(kv, compact_tables="counts")
    sparse = ser.encode_flat(kv)
    assert dense.header.table_kind == ff.TABLES_COUNTS and sparse.header.table_kind == ff.TABLES_SPARSE
    bins = torch.cat((ser.key_bins, ser.value_bins)).cpu().tolist()
    want = sparse_tables_np(dense.tables().cpu().numpy(), bins, H * D)
    got = sparse.tables().cpu().numpy()
    assert got[:want.size].tobytes() == want.tobytes()
    assert sparse.header.off_lengths - sparse.header.off_tables < want.size + ff.ALIGN
    assert torch.equal(de.decode(sparse), de.decode(dense))
    assert sparse.payload(0).cpu().numpy().tobytes() == dense.payload(0).cpu().numpy().tobytes()


def test_corrupt_sparse_offsets_are_flagged_not_followed():
    """Group offsets that point past the table set are reported and read as zero counts."""
    from cachegen_b200.serde import flat_format as ff
    from cachegen_b200.synth import generate_kv
    kv = generate_kv(32, 2, 128, 100, seed=6, device="cuda", dtype=torch.float16)
    ser, de = make_serde(256, "vllm", out_dtype=torch.float16)
    chunk = ser.encode_flat(kv)
    assert chunk.header.table_kind == ff.TABLES_SPARSE
    good = de.decode(chunk)
    de.check_status()
    bad = ff.FlatChunk(chunk.blob.clone(), chunk.header)
    goff = bad.tables()[:4 * (64 * 2 + 1)].view(torch.int32)
    goff[5] = 0x7FFFFFF0       # far past the container
    goff[9] = -16              # 0xFFFFFFF0 as the unsigned offset it is read as
    out = de.decode(bad)
    with pytest.raises(RuntimeError, match="sparse table"):
        de.check_status()
    torch.cuda.synchronize()
    assert out.shape == good.shape
    assert torch.equal(out[:2, 0], good[:2, 0])  # rows 0 and 1 (groups 0..3) are untouched by the damage
    assert torch.equal(de.decode(chunk), good)


def test_the_same_kv_gives_the_same_container_bytes():
    """The alignment gaps of a container are zeroed: two encodes of one chunk agree byte for byte, whatever
    the allocator handed out (stored chunks can be hashed and de-duplicated)."""
    from cachegen_b200.config import LMCacheEngineConfig, LMCacheEngineMetadata
    from cachegen_b200.serde import CacheGenSerializer
    from cachegen_b200.synth import generate_kv
    kv = generate_kv(32, 2, 128, 200, seed=5, device="cuda", dtype=torch.float16)
    ser = CacheGenSerializer(LMCacheEngineConfig.from_defaults(chunk_size=256),
                             LMCacheEngineMetadata(model_name="lmsys/longchat-7b-16k", world_size=1, worker_id=0, fmt="vllm"))
    first = ser.encode_flat(kv).tobytes()
    junk = torch.full((64 << 20,), 0xAB, dtype=torch.uint8, device="cuda")  # dirty the allocator's free blocks
    del junk
    second = ser.encode_flat(kv).tobytes()
    assert first == second
