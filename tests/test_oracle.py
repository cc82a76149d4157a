"""The CPU oracle against hand-checkable known answers, the reference-Python fixtures and itself."""
import numpy as np
import pytest


def table_from(oracle, symbols, max_bins):
    sym = np.asarray(symbols, dtype=np.int8).reshape(1, -1, 1)
    return oracle.calculate_cdf(sym, max_bins)[0, 0]


# Known answers for single streams.  They were first computed with an independent bit-serial Python
# restatement of the reference kernels (cal_cdf.cu:29-49, torchac_kernel_enc_new.cu:255-306,
# torchac_kernel_dec_new.cu:248-302) and are re-derived below by `slow_encode`.
KATS = [
    # (max_bins, symbols to build the table from, symbols to code, hex of the stream)
    (4, [1, 1, 0, 2, 1, 1, 1, 2], None, "3ec0"),
    (32, [(t * t + 3 * t) % 31 for t in range(16)], None, "0157c2d9f4ba1924"),
    (16, [7] * 255 + [3], None, "a180"),
    (32, [(14 + ((t // 5) % 3)) if t % 5 == 0 else 15 for t in range(40)], None, "0da6a7c0"),
    (32, [15] * 100 + [14] * 20 + [16] * 8, [15, 15, 14, 16, 15, 0, 30, 15], "5e6b6714ed00"),
    (32, [5], None, "40"),
]


def slow_encode(cdf_u16, symbols):
    """Bit-serial encoder written straight from torchac_kernel_enc_new.cu:255-306, in Python."""
    lp = len(cdf_u16)
    low, high, pending = 0, 0xFFFFFFFF, 0
    bits = []

    def emit(b):
        nonlocal pending
        bits.append(b)
        bits.extend([1 - b] * pending)
        pending = 0

    for s in symbols:
        span = high - low + 1
        c_low = int(cdf_u16[s])
        c_high = 0x10000 if s == lp - 2 else int(cdf_u16[s + 1])
        high = (low - 1 + ((span * c_high) >> 16)) & 0xFFFFFFFF
        low = (low + ((span * c_low) >> 16)) & 0xFFFFFFFF
        while True:
            if high < 0x80000000:
                emit(0)
            elif low >= 0x80000000:
                emit(1)
            elif low >= 0x40000000 and high < 0xC0000000:
                pending += 1
                low = (low << 1) & 0x7FFFFFFF
                high = ((high << 1) | 0x80000001) & 0xFFFFFFFF
                continue
            else:
                break
            low = (low << 1) & 0xFFFFFFFF
            high = ((high << 1) | 1) & 0xFFFFFFFF
    pending += 1
    emit(0 if low < 0x40000000 else 1)
    while len(bits) % 8:
        bits.append(0)
    return bytes(int("".join(map(str, bits[i:i + 8])), 2) for i in range(0, len(bits), 8))


@pytest.mark.parametrize("max_bins,train,code,hexstream", KATS)
def test_known_answers(oracle, max_bins, train, code, hexstream):
    cdf = table_from(oracle, train, max_bins)
    code = train if code is None else code
    stream = oracle.encode_stream(cdf, code)
    assert stream.tobytes().hex() == hexstream
    assert slow_encode(cdf.view(np.uint16), code).hex() == hexstream
    assert oracle.decode_stream(cdf, stream, len(code)).tolist() == list(code)


def test_known_tables(oracle):
    assert table_from(oracle, [1, 1, 0, 2, 1, 1, 1, 2], 4).view(np.uint16).tolist() == [0, 8192, 49150, 65534, 65535]
    t = table_from(oracle, [7] * 255 + [3], 16).view(np.uint16)
    assert t[:9].tolist() == [0, 1, 2, 3, 259, 260, 261, 262, 65527]
    assert t[-1] == 65535 and np.all(np.diff(t.astype(np.int64)) > 0)


def test_worst_case_stream_length(oracle):
    # 256 symbols that the table has never seen: 16 bits each plus the flush
    cdf = table_from(oracle, [15] * 4096, 32)
    stream = oracle.encode_stream(cdf, [3] * 256)
    assert len(stream) == 513
    assert (oracle.decode_stream(cdf, stream, 256) == 3).all()
    with pytest.raises(OverflowError):
        oracle.encode_stream(cdf, [3] * 256, cap=256)


def test_single_token_streams_are_one_byte(oracle):
    rng = np.random.default_rng(0)
    sym = rng.integers(0, 15, size=(3, 1, 40)).astype(np.int8)
    cdf = oracle.calculate_cdf(sym, 16)
    stream_bytes, lengths = oracle.encode_chunk(cdf, sym, threads=2)
    assert (lengths == 1).all() and len(stream_bytes) == 120
    assert (oracle.decode_chunk(cdf, stream_bytes, lengths, 1, threads=2) == sym.view(np.uint8)).all()


@pytest.mark.parametrize("max_bins", [4, 8, 16, 32, 12, 63])
@pytest.mark.parametrize("T", [1, 16, 236, 256])
def test_chunk_round_trip_and_slow_encoder(oracle, max_bins, T):
    rng = np.random.default_rng(max_bins * 1000 + T)
    rows, C = 3, 37
    nsym = 2 * (max_bins // 2 - 1) + 1
    p = rng.dirichlet(np.full(nsym, 0.3))
    sym = rng.choice(nsym, size=(rows, T, C), p=p).astype(np.int8)
    cdf = oracle.calculate_cdf(sym, max_bins)
    assert cdf.shape == (rows, C, max_bins + 1)
    u = cdf.view(np.uint16).astype(np.int64)
    assert (u[..., 0] == 0).all() and (u[..., -1] == 65535).all() and (np.diff(u, axis=-1) > 0).all()
    stream_bytes, lengths = oracle.encode_chunk(cdf, sym, threads=3)
    assert lengths.sum() == len(stream_bytes)
    dec = oracle.decode_chunk(cdf, stream_bytes, lengths, T, threads=3)
    assert (dec == sym.view(np.uint8)).all()
    # spot-check streams against the Python bit-serial encoder
    offs = np.concatenate(([0], np.cumsum(lengths.reshape(-1))))
    for g in rng.choice(rows * C, size=4, replace=False):
        r, c = divmod(int(g), C)
        want = slow_encode(cdf[r, c].view(np.uint16), sym[r, :, c].tolist())
        assert stream_bytes[offs[g]:offs[g + 1]].tobytes() == want


def test_strided_symbols(oracle):
    rng = np.random.default_rng(5)
    full = rng.integers(0, 31, size=(2, 300, 16)).astype(np.int8)
    cdf = oracle.calculate_cdf(full, 32)
    view = full[:, 40:296, :]
    a, la = oracle.encode_chunk(cdf, view)
    b, lb = oracle.encode_chunk(cdf, np.ascontiguousarray(view))
    assert (la == lb).all() and (a == b).all()


def test_quantize_matches_reference_python(oracle, golden_cpu):
    z = golden_cpu
    for tag, dt in (("f16", oracle.F16), ("bf16", oracle.BF16)):
        sym, mx = oracle.quantize(z[f"quant_{tag}_x"], z[f"quant_{tag}_bins"], dt)
        assert (sym == z[f"quant_{tag}_sym"]).all()
        assert (mx == z[f"quant_{tag}_max"]).all()
        assert (sym[1, 3] == 0).all()  # the all-zero token row


def test_dequantize_matches_reference_python(oracle, golden_cpu):
    z = golden_cpu
    for tag, dt in (("f16", oracle.F16), ("bf16", oracle.BF16)):
        for name, od in (("f16", oracle.F16), ("bf16", oracle.BF16)):
            got = oracle.dequantize(z[f"deq_{tag}_sym"], z[f"quant_{tag}_bins"], z[f"quant_{tag}_max"], dt, od)
            assert (got == z[f"deq_{tag}_{name}"]).all()


def test_quantizer_tie_rule(oracle):
    # bins = 16 -> MAX = 7; x*7+7 = [10.5, 0, 8.75, 14] -> round-half-even -> [10, 0, 9, 14]
    x = oracle.float_to_half(np.array([[[0.5, -1.0, 0.25, 1.0]]], dtype=np.float32))
    sym, mx = oracle.quantize(x, np.array([16.0], dtype=np.float32))
    assert sym.reshape(-1).tolist() == [10, 0, 9, 14]
    assert oracle.half_to_float(mx).reshape(-1).tolist() == [1.0]


def test_half_conversions_match_torch(oracle):
    import torch
    rng = np.random.default_rng(3)
    f = np.concatenate([rng.standard_normal(20000).astype(np.float32) * 10.0 ** rng.integers(-9, 6, 20000),
                        np.array([0.0, -0.0, 65504.0, 65519.9, 65520.0, 1e-8, 5.96e-8, 2.98e-8, 6.1e-5], np.float32)])
    t = torch.from_numpy(f)
    assert (oracle.float_to_half(f, oracle.F16) == t.to(torch.float16).view(torch.int16).numpy().view(np.uint16)).all()
    assert (oracle.float_to_half(f, oracle.BF16) == t.to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)).all()
    h = np.arange(0, 65536, dtype=np.uint16)
    th = torch.from_numpy(h.view(np.int16)).view(torch.float16).float().numpy()
    got = oracle.half_to_float(h, oracle.F16)
    assert ((got == th) | (np.isnan(got) & np.isnan(th))).all()


def test_decode_dequant_chunk_matches_separate_steps(oracle):
    rng = np.random.default_rng(9)
    L, T, H, D = 2, 50, 2, 40
    C = H * D
    bins = np.array([32, 16, 32, 16], dtype=np.float32)
    x = oracle.float_to_half((rng.standard_normal((2 * L, T, C)) * 3).astype(np.float32))
    sym, mx = oracle.quantize(x, bins)
    cdf = oracle.calculate_cdf(sym, 32)
    stream_bytes, lengths = oracle.encode_chunk(cdf, sym)
    want = oracle.dequantize(sym.view(np.uint8), bins, mx)
    out = np.zeros((2 * L, T, C), dtype=np.uint16)
    oracle.decode_dequant_chunk(cdf, stream_bytes, lengths, T, bins, mx, out, [T * C, C, 1], threads=2)
    assert (out == want).all()
