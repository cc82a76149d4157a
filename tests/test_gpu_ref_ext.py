"""Live comparison with the reference's own CUDA extension (oracle/_ref, built unmodified from the
reference sources by oracle/build_ref.py), when that build is present: this package's kernels must
produce byte-identical tables and streams, and each decoder must read the other's streams."""
import glob
import importlib.util
import os

import numpy as np
import pytest
import torch

from gpu_util import peaked_symbols

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def ref():
    hits = glob.glob(os.path.join(ROOT, "oracle", "_ref", "torchac_cuda*.so"))
    if not hits:
        pytest.skip("reference extension not built (oracle/build_ref.py)")
    spec = importlib.util.spec_from_file_location("torchac_cuda", hits[0])
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


@pytest.mark.parametrize("NL,T,C,max_bins,conc", [(4, 256, 256, 32, 0.3), (2, 100, 1024, 16, 0.1),
                                                  (64, 256, 4096, 32, 0.2), (3, 17, 96, 8, 1.0)])
def test_same_bytes_as_the_reference_extension(ref, NL, T, C, max_bins, conc):
    import cachegen_b200.torchac_cuda as mine
    rng = np.random.default_rng(NL * T + C)
    nsym = 2 * (max_bins // 2 - 1) + 1
    if NL * T * C > 1 << 24:  # full-width chunk: draw on the GPU
        g = torch.Generator(device="cuda").manual_seed(1)
        probs = torch.tensor(rng.dirichlet(np.full(nsym, conc)), device="cuda", dtype=torch.float32)
        sym_t = torch.multinomial(probs, NL * T * C, replacement=True, generator=g).to(torch.int8).reshape(NL, T, C)
    else:
        sym_t = torch.from_numpy(peaked_symbols(rng, (NL, T, C), nsym, conc)).cuda()
    cdf_r = ref.calculate_cdf(sym_t, max_bins)
    cdf_m = mine.calculate_cdf(sym_t, max_bins)
    assert torch.equal(cdf_r, cdf_m)
    buf_r = torch.zeros((NL, C, 256), dtype=torch.uint8, device="cuda")
    len_r = torch.zeros((NL, C), dtype=torch.int32, device="cuda")
    ref.encode_fast_new(cdf_r, sym_t, buf_r, len_r)
    buf_m = torch.zeros((NL, C, 256), dtype=torch.uint8, device="cuda")
    len_m = torch.zeros((NL, C), dtype=torch.int32, device="cuda")
    mine.encode_fast_new(cdf_m, sym_t, buf_m, len_m)
    mine.check_status()
    torch.cuda.synchronize()
    assert int(len_r.max()) <= 256
    assert torch.equal(len_r, len_m)
    keep = torch.arange(256, device="cuda")[None, None, :] < len_r[:, :, None]
    assert torch.equal(buf_r * keep, buf_m * keep)
    # cross-decoding
    flat = buf_m[keep]
    pref = len_m.flatten().cumsum(0).reshape(len_m.shape)
    out_r = torch.zeros((NL, T, C), dtype=torch.uint8, device="cuda")
    out_m = torch.zeros((NL, T, C), dtype=torch.uint8, device="cuda")
    ref.decode_fast_prefsum(cdf_r, flat, pref, out_r)
    mine.decode_fast_prefsum(cdf_r, flat, pref, out_m)
    mine.check_status()
    assert torch.equal(out_r, sym_t.view(torch.uint8)) and torch.equal(out_m, out_r)
    out_m2 = torch.zeros_like(out_m)
    mine.decode_fast_new(cdf_r, buf_r, len_r, out_m2)
    assert torch.equal(out_m2, out_r)
