"""Byte-for-byte comparison with the reference's CUDA extension on the benchmark workload itself:
the 8,192-token Llama-7B-shape cache (seed 1), quantised by this package, every one of its 32
chunks encoded and decoded by both implementations (needs oracle/_ref, built by oracle/build_ref.py).

The synthetic generator's K rows are very peaked (a fraction of a bit per symbol), which is where the
coder's runs of pending underflow bits are longest -- the case random Dirichlet symbols do not reach.
"""
import glob
import importlib.util
import os

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_ROW_BYTES = 256  # the reference encoder's shared-memory row per stream (torchac_kernel_enc_new.cu:11,236)


@pytest.fixture(scope="module")
def ref():
    hits = glob.glob(os.path.join(ROOT, "oracle", "_ref", "torchac_cuda*.so"))
    if not hits:
        pytest.skip("reference extension not built (oracle/build_ref.py)")
    spec = importlib.util.spec_from_file_location("torchac_cuda", hits[0])
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_all_chunks_of_the_8k_workload_match_the_reference_extension(ref):
    import cachegen_b200.torchac_cuda as mine
    from cachegen_b200.serde.cachegen_basics import CacheGenConfig, make_key_bins, make_value_bins
    from cachegen_b200.serde.cachegen_encoder import encode_streams, quantize_and_tables
    from cachegen_b200.synth import WORKLOADS, generate_kv

    spec = WORKLOADS["llama7b-8k"]
    L, H, D, T = spec["num_layers"], spec["num_heads"], spec["head_size"], spec["num_tokens"]
    C, CH = H * D, 256
    cfg = CacheGenConfig.from_model_name(spec["model_name"])
    kb, vb = make_key_bins(cfg, "cuda"), make_value_bins(cfg, "cuda")
    max_bins = cfg.max_bins
    encoded_by_both = 0
    buf_r = torch.zeros((2 * L, C, REF_ROW_BYTES), dtype=torch.uint8, device="cuda")
    len_r = torch.zeros((2 * L, C), dtype=torch.int32, device="cuda")
    out_r = torch.empty((2 * L, CH, C), dtype=torch.uint8, device="cuda")
    out_m = torch.empty_like(out_r)
    column = torch.arange(REF_ROW_BYTES, device="cuda")[None, None, :]
    # the generator is seeded per layer, so chunks can be produced a few layers at a time; here the
    # whole cache is made once (4 GiB) and sliced
    kv = generate_kv(L, H, D, T, spec["seed"], key_rho=spec["key_rho"], device="cuda", dtype=torch.float16)
    for s in range(0, T, CH):
        chunk = kv[:, :, s:s + CH]
        sym, _, cdf = quantize_and_tables(chunk, kb, vb, max_bins)
        # tables: the reference builds key and value tables separately and concatenates them
        cdf_r = torch.cat((ref.calculate_cdf(sym[:L], max_bins), ref.calculate_cdf(sym[L:], max_bins)))
        assert torch.equal(cdf_r, cdf), f"tables differ in chunk {s // CH}"
        payload, lengths, _ = encode_streams(cdf, sym)
        lengths = lengths[0]
        # the reference encoder overruns its 256-byte row on a longer stream: only hand it chunks
        # whose streams all fit, and compare the decoders alone otherwise
        if int(lengths.max()) <= REF_ROW_BYTES:
            buf_r.zero_()
            len_r.zero_()
            ref.encode_fast_new(cdf, sym, buf_r, len_r)
            assert torch.equal(len_r, lengths), f"stream lengths differ in chunk {s // CH}"
            keep = column < len_r[:, :, None]
            assert torch.equal(buf_r[keep], payload), f"stream bytes differ in chunk {s // CH}"
            encoded_by_both += 1
        pref = lengths.flatten().to(torch.int64).cumsum(0).reshape(lengths.shape)
        ref.decode_fast_prefsum(cdf, payload, pref, out_r)
        mine.decode_fast_prefsum(cdf, payload, pref, out_m)
        mine.check_status()
        assert torch.equal(out_r, sym.view(torch.uint8)), f"the reference decoder misreads chunk {s // CH}"
        assert torch.equal(out_m, out_r), f"decoded symbols differ in chunk {s // CH}"
    assert encoded_by_both > 0
