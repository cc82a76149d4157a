"""Randomised parity sweep on the GPU: random layer / head / token counts (scalar and vector paths,
one to three sub-chunks), both dtypes, both layouts, random layer-group boundaries and bin counts from
4 to 62 (tables of 5 to 63 entries, all search depths), against the CPU oracle: tables, lengths,
streams, decoded values, the pickle round trip and every table form of the flat container."""
import numpy as np
import pytest
import torch

from gpu_util import bits_np, kv_rows

pytestmark = pytest.mark.gpu

BIN_CHOICES = [4, 6, 8, 12, 16, 24, 32, 34, 48, 62]


@pytest.mark.parametrize("seed", [11, 12, 13])
def test_random_configurations_against_the_oracle(oracle, seed):
    from cachegen_b200.config import LMCacheEngineConfig, LMCacheEngineMetadata
    from cachegen_b200.serde import CacheGenDeserializer, CacheGenSerializer
    from cachegen_b200.serde.cachegen_basics import CacheGenConfig
    rng = np.random.default_rng(seed)
    for it in range(25):
        L, H = int(rng.integers(1, 7)), int(rng.integers(1, 6))
        D = int(rng.choice([8, 16, 40, 64, 128, 7, 24]))
        T = int(rng.choice([1, 2, 17, 100, 255, 256, 257, 300, 513, 700]))
        dtype = torch.float16 if rng.random() < 0.5 else torch.bfloat16
        out_dtype = torch.float16 if rng.random() < 0.5 else torch.bfloat16
        fmt = "vllm" if rng.random() < 0.5 else "huggingface"
        top = int(rng.choice(BIN_CHOICES))           # key and value tables must have the same length
        lower = [c for c in BIN_CHOICES if c <= top]
        ks, kt, vs = (int(rng.choice(lower)) for _ in range(3))
        l1 = int(rng.integers(1, L + 1))
        l2, v1 = int(rng.integers(l1, L + 1)), int(rng.integers(1, L + 1))
        cfg = CacheGenConfig(l1, l2, L, top, ks, kt, v1, top, vs)
        kb = np.array([top if i < l1 else ks if i < l2 else kt for i in range(L)], np.float32)
        vb = np.array([top if i < v1 else vs for i in range(L)], np.float32)
        scale = np.exp(rng.normal(0, 1.0, (L, 2, 1, H, D))).astype(np.float32)
        x = torch.from_numpy(rng.standard_normal((L, 2, T, H, D)).astype(np.float32) * scale).to(dtype)
        if rng.random() < 0.3:
            x[:, :, int(rng.integers(0, T))] = 0     # an all-zero token row
        what = f"case {it}: L={L} H={H} D={D} T={T} {dtype} {fmt} key bins {kb.tolist()} value bins {vb.tolist()}"
        config = LMCacheEngineConfig.from_defaults(chunk_size=1024)
        meta = LMCacheEngineMetadata("lmsys/longchat-7b-16k", 1, 0, fmt)
        ser = CacheGenSerializer(config, meta, cachegen_config=cfg)
        de = CacheGenDeserializer(config, meta, cachegen_config=cfg, out_dtype=out_dtype)
        blob_kv = x.cuda() if fmt == "vllm" else x.permute(0, 1, 3, 2, 4).contiguous().cuda()

        def rows_of(o):
            o = o if fmt == "vllm" else o.permute(0, 1, 3, 2, 4)
            return bits_np(kv_rows(o.contiguous()))

        code = oracle.F16 if dtype == torch.float16 else oracle.BF16
        bins = np.concatenate((kb, vb))
        sym, mx = oracle.quantize(bits_np(kv_rows(x)), bins, code)
        cdf = oracle.calculate_cdf(sym, int(bins.max()))
        eo = ser.encode(blob_kv)
        assert (eo.cdf.cpu().numpy() == cdf).all(), what
        for j, s in enumerate(range(0, T, 256)):
            want_bytes, want_len = oracle.encode_chunk(cdf, sym[:, s:s + 256, :])
            assert (eo.data_chunks[j].bytestream_lengths.cpu().numpy() == want_len).all(), what
            assert eo.data_chunks[j].bytestream.cpu().numpy().tobytes() == want_bytes.tobytes(), what
        want = oracle.dequantize(sym.view(np.uint8), bins, mx, code,
                                 oracle.F16 if out_dtype == torch.float16 else oracle.BF16)
        assert (rows_of(de.decode(eo)) == want).all(), what
        assert (rows_of(de.from_bytes(ser.to_bytes(blob_kv))) == want).all(), what
        for compact in (True, "counts", False):
            chunk = ser.encode_flat(blob_kv, compact_tables=compact)
            assert (rows_of(de.decode(chunk)) == want).all(), (what, compact, chunk.header.table_kind)
            assert (rows_of(de.from_bytes(chunk.tobytes())) == want).all(), (what, compact)
        de.check_status()
