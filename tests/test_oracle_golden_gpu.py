"""The CPU oracle against outputs recorded from the reference's own CUDA extension
(tests/golden/ref_cuda_ext.npz, written on a GPU by tests/golden/make_golden_gpu.py)."""
import os

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PATH = os.path.join(ROOT, "tests", "golden", "ref_cuda_ext.npz")


def cases():
    if not os.path.exists(PATH):
        return []
    z = np.load(PATH)
    return sorted(k[:-5] for k in z.files if k.endswith("_meta"))


@pytest.mark.skipif(not os.path.exists(PATH), reason="fixture not generated yet")
@pytest.mark.parametrize("name", cases())
def test_oracle_reproduces_reference_extension(oracle, name):
    z = np.load(PATH)
    rows, T, C, mb, nsym, seed = (int(v) for v in z[f"{name}_meta"])
    rng = np.random.default_rng(seed)
    p = rng.dirichlet(np.full(nsym, float(z[f"{name}_conc"][0])))
    sym = rng.choice(nsym, size=(rows, T, C), p=p).astype(np.int8)
    cdf = oracle.calculate_cdf(sym, mb)
    assert (cdf == z[f"{name}_cdf"]).all()
    stream_bytes, lengths = oracle.encode_chunk(cdf, sym)
    assert (lengths == z[f"{name}_lengths"]).all()
    assert stream_bytes.tobytes() == z[f"{name}_bytes"].tobytes()
    assert (oracle.decode_chunk(z[f"{name}_cdf"], z[f"{name}_bytes"], z[f"{name}_lengths"], T) == sym.view(np.uint8)).all()


@pytest.mark.skipif(not os.path.exists(PATH), reason="fixture not generated yet")
def test_zero_row_symbols_match_cuda_cast(oracle):
    z = np.load(PATH)
    x = np.zeros((1, 2, 8), dtype=np.float32)
    x[0, 1] = [0.5, -1.0, 0.25, 1.0] * 2
    sym, _ = oracle.quantize(oracle.float_to_half(x), np.array([16.0], dtype=np.float32))
    assert (sym == z["cuda_quant_zero_row"]).all()
