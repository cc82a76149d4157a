"""The four torchac_cuda entry points on the GPU against the CPU oracle: bit-exact tables, streams,
lengths and symbols, over the reference's shapes and the edge cases it leaves untested."""
import numpy as np
import pytest
import torch

from gpu_util import peaked_symbols

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def tc():
    import cachegen_b200.torchac_cuda as m
    return m


def encode_gpu(tc, cdf_t, sym_t, row_bytes=None):
    NL, T, C = sym_t.shape
    row_bytes = row_bytes or 2 * T + 8
    row_bytes = (row_bytes + 3) // 4 * 4
    buf = torch.zeros((NL, C, row_bytes), dtype=torch.uint8, device="cuda")
    lens = torch.zeros((NL, C), dtype=torch.int32, device="cuda")
    tc.encode_fast_new(cdf_t, sym_t, buf, lens)
    tc.check_status()
    return buf, lens


def gather(buf, lens):
    b, l = buf.cpu().numpy(), lens.cpu().numpy()
    return np.concatenate([b[r, c, :l[r, c]] for r in range(b.shape[0]) for c in range(b.shape[1])])


@pytest.mark.parametrize("max_bins", [4, 8, 16, 32, 12, 63])
@pytest.mark.parametrize("T", [1, 16, 236, 256])
@pytest.mark.parametrize("C", [37, 128, 320])
def test_cdf_encode_decode_match_oracle(oracle, tc, max_bins, T, C):
    if max_bins == 63 and C == 320:
        pytest.skip("covered by the smaller channel counts")
    rng = np.random.default_rng(max_bins * 7919 + T * 31 + C)
    NL = 3
    nsym = 2 * (max_bins // 2 - 1) + 1
    sym = peaked_symbols(rng, (NL, T, C), nsym)
    sym_t = torch.from_numpy(sym).cuda()
    cdf_t = tc.calculate_cdf(sym_t, max_bins)
    cdf = oracle.calculate_cdf(sym, max_bins)
    assert cdf_t.dtype == torch.int16 and tuple(cdf_t.shape) == (NL, C, max_bins + 1)
    assert (cdf_t.cpu().numpy() == cdf).all()

    if max_bins + 1 <= tc.MAX_LP_ENCODE:
        want_bytes, want_len = oracle.encode_chunk(cdf, sym)
        buf, lens = encode_gpu(tc, cdf_t, sym_t)
        assert (lens.cpu().numpy() == want_len).all()
        got = gather(buf, lens)
        assert got.tobytes() == want_bytes.tobytes()
    else:  # the reference's encoder stops at 48 table entries; decode goes to 64
        with pytest.raises(RuntimeError):
            encode_gpu(tc, cdf_t, sym_t)
        want_bytes, want_len = oracle.encode_chunk(cdf, sym)
        got = want_bytes
        buf = None

    # decode_fast_prefsum from the flat array
    flat = torch.from_numpy(got.copy()).cuda()
    pref = torch.from_numpy(np.cumsum(want_len.reshape(-1).astype(np.int64)).reshape(NL, C)).cuda()
    out = torch.full((NL, T, C), 255, dtype=torch.uint8, device="cuda")
    tc.decode_fast_prefsum(cdf_t, flat, pref, out)
    tc.check_status()
    assert (out.cpu().numpy() == sym.view(np.uint8)).all()

    # decode_fast_new from the padded rows
    if buf is not None:
        out2 = torch.full((NL, T, C), 255, dtype=torch.uint8, device="cuda")
        tc.decode_fast_new(cdf_t, buf, lens, out2)
        tc.check_status()
        assert (out2.cpu().numpy() == sym.view(np.uint8)).all()


def test_strided_slices_like_the_reference_loops(oracle, tc):
    """encode_function passes encode_input[:, s:e, :] and decode_chunk writes output[:, s:e, :]
    (cachegen_encoder.py:285, cachegen_decoder.py:106): non-contiguous token slices."""
    rng = np.random.default_rng(11)
    NL, T, C = 4, 600, 256
    sym = peaked_symbols(rng, (NL, T, C), 31)
    sym_t = torch.from_numpy(sym).cuda()
    cdf_t = tc.calculate_cdf(sym_t, 32)
    cdf = oracle.calculate_cdf(sym, 32)
    assert (cdf_t.cpu().numpy() == cdf).all()
    out = torch.zeros((NL, T, C), dtype=torch.uint8, device="cuda")
    for s in range(0, T, 256):
        e = min(s + 256, T)
        buf, lens = encode_gpu(tc, cdf_t, sym_t[:, s:e, :], row_bytes=256)
        want_bytes, want_len = oracle.encode_chunk(cdf, sym[:, s:e, :])
        assert (lens.cpu().numpy() == want_len).all()
        got = gather(buf, lens)
        assert got.tobytes() == want_bytes.tobytes()
        pref = lens.flatten().cumsum(0).reshape(lens.shape)
        assert pref.dtype == torch.int64
        tc.decode_fast_prefsum(cdf_t, torch.from_numpy(got.copy()).cuda(), pref, out[:, s:e, :])
    tc.check_status()
    assert (out.cpu().numpy() == sym.view(np.uint8)).all()


def test_foreign_table_and_worst_case_length(oracle, tc):
    """Symbols the table has never seen cost 16 bits each: 513-byte streams.  The reference overruns
    its 256-byte row; here a 256-byte row is reported and a full-capacity row is exact."""
    NL, T, C = 1, 256, 128
    train = np.full((NL, 4096, C), 15, dtype=np.int8)
    cdf = oracle.calculate_cdf(train, 32)
    cdf_t = torch.from_numpy(cdf).cuda()
    sym = np.full((NL, T, C), 3, dtype=np.int8)
    sym[:, :, ::2] = 15  # every other channel is the cheap symbol
    sym_t = torch.from_numpy(sym).cuda()
    buf, lens = encode_gpu(tc, cdf_t, sym_t)
    want_bytes, want_len = oracle.encode_chunk(cdf, sym)
    assert want_len.max() == 513
    assert (lens.cpu().numpy() == want_len).all()
    assert gather(buf, lens).tobytes() == want_bytes.tobytes()
    small = torch.zeros((NL, C, 256), dtype=torch.uint8, device="cuda")
    lens2 = torch.zeros((NL, C), dtype=torch.int32, device="cuda")
    tc.encode_fast_new(cdf_t, sym_t, small, lens2)
    with pytest.raises(RuntimeError, match="outgrew"):
        tc.check_status()
    assert (lens2.cpu().numpy() == want_len).all()  # full lengths are still reported
    ok = want_len[0] <= 256
    b = small.cpu().numpy()
    for c in np.nonzero(ok)[0][:8]:
        assert b[0, c, :want_len[0, c]].tobytes() == oracle.encode_stream(cdf[0, c], sym[0, :, c]).tobytes()


def test_truncated_and_malformed_streams_do_not_fault(oracle, tc):
    rng = np.random.default_rng(13)
    NL, T, C = 2, 200, 128
    sym = peaked_symbols(rng, (NL, T, C), 15, conc=1.0)
    cdf = oracle.calculate_cdf(sym, 16)
    want_bytes, want_len = oracle.encode_chunk(cdf, sym)
    cdf_t = torch.from_numpy(cdf).cuda()
    # (a) every stream cut to half its length: same symbols as the oracle's zero-padding decode
    half = (want_len // 2).astype(np.int32)
    offs = np.concatenate(([0], np.cumsum(want_len.reshape(-1))))
    pieces = [want_bytes[offs[g]:offs[g] + half.reshape(-1)[g]] for g in range(NL * C)]
    cut = np.concatenate(pieces)
    ref = oracle.decode_chunk(cdf, cut, half, T)
    out = torch.zeros((NL, T, C), dtype=torch.uint8, device="cuda")
    pref = torch.from_numpy(np.cumsum(half.reshape(-1).astype(np.int64)).reshape(NL, C)).cuda()
    tc.decode_fast_prefsum(cdf_t, torch.from_numpy(cut).cuda(), pref, out)
    tc.check_status()
    assert (out.cpu().numpy() == ref).all()
    # (b) prefix sums that run past the byte array: flagged, no fault, launch completes
    bad = pref.clone()
    bad[-1, -1] += 10_000_000
    bad[0, 5] = -7
    tc.decode_fast_prefsum(cdf_t, torch.from_numpy(cut).cuda(), bad, out)
    with pytest.raises(RuntimeError, match="lengths"):
        tc.check_status()
    torch.cuda.synchronize()


def test_argument_checks_raise_like_the_reference(tc):
    cdf = torch.zeros((2, 128, 33), dtype=torch.int16, device="cuda")
    sym = torch.zeros((2, 300, 128), dtype=torch.int8, device="cuda")
    buf = torch.zeros((2, 128, 256), dtype=torch.uint8, device="cuda")
    lens = torch.zeros((2, 128), dtype=torch.int32, device="cuda")
    with pytest.raises(RuntimeError, match="Number of tokens"):
        tc.encode_fast_new(cdf, sym, buf, lens)
    with pytest.raises(RuntimeError, match="same number of layers"):
        tc.encode_fast_new(cdf[:1], sym[:, :16], buf, lens)
    with pytest.raises(RuntimeError, match="should be on GPU"):
        tc.encode_fast_new(cdf.cpu(), sym[:, :16], buf, lens)
    with pytest.raises(RuntimeError, match="Max bins"):
        tc.calculate_cdf(sym, 64)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        tc.calculate_cdf(sym.cpu(), 32)
    out = torch.zeros((2, 300, 128), dtype=torch.uint8, device="cuda")
    pref = torch.zeros((2, 128), dtype=torch.int64, device="cuda")
    with pytest.raises(RuntimeError, match="Number of tokens"):
        tc.decode_fast_prefsum(cdf, torch.zeros(8, dtype=torch.uint8, device="cuda"), pref, out)
    # element types the reference's accessors reject too: the kernels address bytes
    with pytest.raises(RuntimeError, match="int8 input symbols"):
        tc.encode_fast_new(cdf, sym[:, :16].to(torch.int32), buf, lens)
    with pytest.raises(RuntimeError, match="uint8 bytestreams and output"):
        tc.decode_fast_prefsum(cdf, torch.zeros(8, dtype=torch.uint8, device="cuda"), pref, out[:, :16].to(torch.int32))
    with pytest.raises(RuntimeError, match="uint8 bytestreams and output"):
        tc.decode_fast_new(cdf, buf.to(torch.int16), lens, out[:, :16])
    with pytest.raises(RuntimeError, match="rank"):
        tc.decode_fast_new(cdf, buf.reshape(2, -1), lens, out[:, :16])


@pytest.mark.parametrize("max_bins,T,C", [(32, 256, 320), (16, 77, 37), (8, 1, 128), (12, 200, 130)])
def test_warp_per_stream_decoder_gives_the_same_symbols(oracle, tc, max_bins, T, C):
    """The one-warp-per-stream layout (ballot search, table in registers) against the oracle and
    against the thread-per-stream kernel, on whole and on truncated streams."""
    rng = np.random.default_rng(max_bins * 101 + T + C)
    NL = 2
    sym = peaked_symbols(rng, (NL, T, C), 2 * (max_bins // 2 - 1) + 1)
    cdf = oracle.calculate_cdf(sym, max_bins)
    cdf_t = torch.from_numpy(cdf).cuda()
    want_bytes, want_len = oracle.encode_chunk(cdf, sym)
    pref = torch.from_numpy(np.cumsum(want_len.reshape(-1).astype(np.int64)).reshape(NL, C)).cuda()
    flat = torch.from_numpy(want_bytes.copy()).cuda()
    out = torch.full((NL, T, C), 255, dtype=torch.uint8, device="cuda")
    tc.decode_fast_prefsum_warp(cdf_t, flat, pref, out)
    tc.check_status()
    assert (out.cpu().numpy() == sym.view(np.uint8)).all()

    # every stream cut to half its bytes: both kernels read zeros past the end and must agree
    half = (want_len.reshape(-1) // 2).astype(np.int64)
    starts = np.concatenate([[0], np.cumsum(want_len.reshape(-1).astype(np.int64))[:-1]])
    cut = np.concatenate([want_bytes[s:s + h] for s, h in zip(starts, half)] + [np.zeros(0, np.uint8)])
    cut_t = torch.from_numpy(np.ascontiguousarray(cut)).cuda() if cut.size else torch.zeros(4, dtype=torch.uint8, device="cuda")
    pref2 = torch.from_numpy(np.cumsum(half).reshape(NL, C)).cuda()
    a = torch.full((NL, T, C), 255, dtype=torch.uint8, device="cuda")
    b = torch.full((NL, T, C), 254, dtype=torch.uint8, device="cuda")
    tc.decode_fast_prefsum(cdf_t, cut_t, pref2, a)
    tc.decode_fast_prefsum_warp(cdf_t, cut_t, pref2, b)
    tc.check_status()
    assert torch.equal(a, b)


def test_warp_per_stream_decoder_rejects_long_tables(tc):
    cdf = torch.zeros((1, 4, 49), dtype=torch.int16, device="cuda")
    pref = torch.zeros((1, 4), dtype=torch.int64, device="cuda")
    out = torch.zeros((1, 8, 4), dtype=torch.uint8, device="cuda")
    with pytest.raises(RuntimeError):
        tc.decode_fast_prefsum_warp(cdf, torch.zeros(8, dtype=torch.uint8, device="cuda"), pref, out)


def test_reference_named_helpers_around_the_entry_points(oracle, tc):
    """torch_quant_vectorized, encode_ntokens / collect_bytes, recombine_bytes and bytes_to_tensor with
    the reference's signatures (cachegen_encoder.py:42-59,210-242, cachegen_decoder.py:37-49): the
    legacy padded-row path end to end against the oracle."""
    from cachegen_b200.serde import cachegen_decoder as D
    from cachegen_b200.serde import cachegen_encoder as E
    rng = np.random.default_rng(77)
    R, T, C = 5, 100, 200                     # an odd row count and a ragged channel count
    bins = np.array([32, 16, 16, 8, 32], dtype=np.float32)
    x = (rng.standard_normal((R, T, C)) * rng.lognormal(0, 0.5, (R, 1, C))).astype(np.float16)
    x[2, 7] = 0                               # an all-zero token row: symbol 0 everywhere
    xq, max1 = E.torch_quant_vectorized(torch.from_numpy(bins).cuda(), torch.from_numpy(x).cuda())
    want_sym, want_max = oracle.quantize(x.view(np.uint16), bins, oracle.F16)
    assert xq.dtype == torch.int8 and tuple(max1.shape) == (R, T, 1)
    assert (xq.cpu().numpy() == want_sym).all()
    assert (max1.cpu().numpy().view(np.uint16).reshape(R, T) == want_max.reshape(R, T)).all()
    assert torch.equal(E.concat_max([max1[i] for i in range(R)]), max1)

    cdf_t = tc.calculate_cdf(xq, 32)
    cdf = oracle.calculate_cdf(want_sym, 32)
    buf = torch.zeros((R, C, 256), dtype=torch.uint8, device="cuda")
    lens = torch.zeros((R, C), dtype=torch.int32, device="cuda")
    stream_bytes = E.encode_ntokens(cdf_t, xq, buf, lens)
    want_bytes, want_len = oracle.encode_chunk(cdf, want_sym)
    assert (lens.cpu().numpy() == want_len).all()
    assert stream_bytes.cpu().numpy().tobytes() == want_bytes.tobytes()
    with pytest.raises(RuntimeError):
        E.collect_bytes(buf, lens + 300)      # lengths beyond the row are refused, not followed

    wire = D.bytes_to_tensor(stream_bytes.cpu().numpy().tobytes())
    assert wire.is_cuda and torch.equal(wire, stream_bytes)
    rows = D.recombine_bytes(wire, lens)
    assert tuple(rows.shape) == (R, C, 256)
    flat, starts = want_bytes, np.concatenate(([0], np.cumsum(want_len.reshape(-1))[:-1]))
    pick = np.minimum(starts[:, None] + np.arange(256), flat.size - 1)
    assert (rows.cpu().numpy().reshape(-1, 256) == flat[pick]).all()
    out = torch.zeros((R, T, C), dtype=torch.uint8, device="cuda")
    tc.decode_fast_new(cdf_t, rows, lens, out)
    tc.check_status()
    assert (out.cpu().numpy() == want_sym.view(np.uint8)).all()
