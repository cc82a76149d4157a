"""The product's per-stream coder loops (cachegen_b200/csrc/cg_coder.cuh, compiled for the host by
tests/host_model/coder_host.cpp) against the oracle: bit-exact streams, symbols and zero-padding
behaviour on truncated streams, for every table length the kernels dispatch on."""
import ctypes

import numpy as np
import pytest


def P(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def random_table(oracle, rng, lp, kind):
    mb = lp - 1
    if kind == 0:  # as calculate_cdf builds them
        T = int(rng.integers(1, 300))
        p = rng.dirichlet(np.full(mb, rng.choice([0.05, 0.3, 2.0])))
        syms = rng.choice(mb, size=T, p=p).astype(np.int8)
        return oracle.calculate_cdf(syms.reshape(1, -1, 1), mb)[0, 0].view(np.uint16).copy()
    c = np.sort(rng.choice(np.arange(1, 65536), size=lp - 1, replace=False)).astype(np.uint16)
    return np.concatenate(([0], c)).astype(np.uint16)  # any strictly increasing table from 0


@pytest.mark.parametrize("seed", range(8))
def test_coder_loops_match_oracle(oracle, host_model, seed):
    rng = np.random.default_rng(seed)
    for _ in range(300):
        lp = int(rng.integers(2, 65)) if rng.random() < 0.7 else int(rng.choice([5, 9, 17, 33]))
        cdf = random_table(oracle, rng, lp, int(rng.integers(0, 2)))
        n = int(rng.integers(1, 257))
        maxsym = lp - 2
        mode = int(rng.integers(0, 3))
        if mode == 0:
            sym = rng.integers(0, maxsym + 1, size=n)
        elif mode == 1:
            sym = np.full(n, rng.integers(0, maxsym + 1))
        else:
            sym = np.where(rng.random(n) < 0.9, maxsym // 2, rng.integers(0, maxsym + 1, size=n))
        sym = sym.astype(np.int8)
        want = oracle.encode_stream(cdf, sym)
        cap = 2 * n + 8
        out = np.zeros(cap + 8, dtype=np.uint8)
        tid = int(rng.integers(0, 128))
        ln = host_model.hm_encode_stream(P(cdf), lp, P(sym), n, P(out), cap, tid)
        assert ln == len(want) and (out[:ln] == want).all()
        # decode from every byte alignment, with garbage on both sides of the stream
        off = int(rng.integers(0, 8))
        big = rng.integers(0, 256, size=off + len(want) + 16).astype(np.uint8)
        big[off:off + len(want)] = want
        dec = np.zeros(n, dtype=np.uint8)
        host_model.hm_decode_stream(P(cdf), lp, ctypes.c_void_p(big.ctypes.data + off), len(want), n, P(dec), tid)
        assert (dec == sym.view(np.uint8)).all()
        # a truncated stream decodes as if zero-padded, exactly like the reference's staging row
        tl = int(rng.integers(0, len(want) + 1))
        dec2 = np.zeros(n, dtype=np.uint8)
        host_model.hm_decode_stream(P(cdf), lp, ctypes.c_void_p(big.ctypes.data + off), tl, n, P(dec2), tid)
        assert (dec2 == oracle.decode_stream(cdf, want[:tl], n)).all()


def test_capacity_overflow_is_reported_not_written(oracle, host_model):
    cdf = oracle.calculate_cdf(np.full((1, 4096, 1), 15, dtype=np.int8), 32)[0, 0].view(np.uint16).copy()
    sym = np.full(256, 3, dtype=np.int8)
    out = np.full(300, 0xAB, dtype=np.uint8)
    ln = host_model.hm_encode_stream(P(cdf), 33, P(sym), 256, P(out), 256, 0)
    assert ln == 513
    assert (out[256:] == 0xAB).all()
    assert (out[:256] == oracle.encode_stream(cdf, sym)[:256]).all()


@pytest.mark.parametrize("seed", range(6))
def test_pair_decode_loop_matches_oracle_at_every_search_depth(oracle, host_model, seed):
    """decode_streams (two streams per lane, fast search over the first 2^fl entries with the exact
    search as its fallback) must give the oracle's symbols whatever depth the caller picks: too
    shallow a depth for the symbols that occur only costs time."""
    rng = np.random.default_rng(100 + seed)
    for _ in range(150):
        lp = int(rng.integers(2, 65)) if rng.random() < 0.5 else int(rng.choice([5, 9, 13, 17, 33]))
        full = 0
        while (1 << full) < lp - 1:
            full += 1
        n = int(rng.integers(1, 257))
        maxsym = lp - 2
        cdfs, syms, streams = [], [], []
        for _s in range(2):
            cdf = random_table(oracle, rng, lp, int(rng.integers(0, 2)))
            mode = int(rng.integers(0, 4))
            if mode == 0:
                sym = rng.integers(0, maxsym + 1, size=n)
            elif mode == 1:
                sym = np.full(n, rng.integers(0, maxsym + 1))
            elif mode == 2:  # what a row quantised to fewer bins than the table holds looks like
                hi = int(rng.integers(0, maxsym + 1))
                sym = rng.integers(0, hi + 1, size=n)
            else:
                sym = np.where(rng.random(n) < 0.9, maxsym // 2, rng.integers(0, maxsym + 1, size=n))
            sym = sym.astype(np.int8)
            cdfs.append(cdf)
            syms.append(sym)
            streams.append(oracle.encode_stream(cdf, sym))
        off = int(rng.integers(0, 8))
        big = rng.integers(0, 256, size=off + len(streams[0]) + len(streams[1]) + 16).astype(np.uint8)
        big[off:off + len(streams[0])] = streams[0]
        big[off + len(streams[0]):off + len(streams[0]) + len(streams[1])] = streams[1]
        p0 = big.ctypes.data + off
        p1 = p0 + len(streams[0])
        tid = int(rng.integers(0, 64))
        for fl in range(2, max(full, 2) + 1):
            dec = np.zeros(2 * n, dtype=np.uint8)
            rc = host_model.hm_decode_pair(P(cdfs[0]), P(cdfs[1]), lp, ctypes.c_void_p(p0), len(streams[0]),
                                           ctypes.c_void_p(p1), len(streams[1]), n, P(dec), tid, fl)
            assert rc == 0
            assert (dec[0::2] == syms[0].view(np.uint8)).all(), (lp, fl)
            assert (dec[1::2] == syms[1].view(np.uint8)).all(), (lp, fl)
        # truncated streams decode as if zero-padded, like the reference's staging row
        t0, t1 = int(rng.integers(0, len(streams[0]) + 1)), int(rng.integers(0, len(streams[1]) + 1))
        fl = int(rng.integers(2, max(full, 2) + 1))
        dec = np.zeros(2 * n, dtype=np.uint8)
        host_model.hm_decode_pair(P(cdfs[0]), P(cdfs[1]), lp, ctypes.c_void_p(p0), t0, ctypes.c_void_p(p1), t1, n,
                                  P(dec), tid, fl)
        assert (dec[0::2] == oracle.decode_stream(cdfs[0], streams[0][:t0], n)).all()
        assert (dec[1::2] == oracle.decode_stream(cdfs[1], big[off + len(streams[0]):off + len(streams[0]) + t1], n)).all()


def test_search_depth_for_a_bin_count(host_model):
    # symbols 0 .. bins-2 of a row with `bins` bins: the depth's top entry must lie above them
    for bins, want in ((4, 2), (8, 3), (12, 4), (16, 4), (32, 5), (62, 6)):
        nsym = 2 * (bins // 2 - 1) + 1
        assert host_model.hm_fast_levels_for(nsym, 6) == want
    assert host_model.hm_fast_levels_for(31, 4) == 4  # never deeper than the table
    assert host_model.hm_fast_levels_for(1, 0) == 2   # and never below the two register levels
