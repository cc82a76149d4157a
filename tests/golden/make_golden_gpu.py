"""Generates tests/golden/ref_cuda_ext.npz by running the REFERENCE's own CUDA extension.

Needs a GPU and oracle/_ref/torchac_cuda*.so (the reference's torchac_cuda sources compiled unmodified
by oracle/build_ref.py).  For seeded symbol tensors it records what the reference's
calculate_cdf / encode_fast_new / decode_fast_prefsum / decode_fast_new return, so that the CPU oracle
(and through it the CUDA kernels of this package) can be pinned to the reference without a GPU:

    python tests/golden/make_golden_gpu.py [output.npz]

It also prints whether the CPU oracle already agrees with every recorded output.
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "oracle", "_ref"))

CASES = [
    # name, rows, tokens, channels, max_bins, number of distinct symbols, dirichlet concentration, seed
    ("lp33_t200", 2, 200, 128, 32, 31, 0.3, 101),
    ("lp33_t256_peaked", 2, 256, 128, 32, 31, 0.05, 102),
    ("lp17_t256", 2, 256, 128, 16, 15, 0.5, 103),
    ("lp9_t37", 3, 37, 64, 8, 7, 1.0, 104),
    ("lp33_t1", 2, 1, 128, 32, 31, 0.3, 105),
]


def symbols(rows, T, C, nsym, conc, seed):
    rng = np.random.default_rng(seed)
    p = rng.dirichlet(np.full(nsym, conc))
    return rng.choice(nsym, size=(rows, T, C), p=p).astype(np.int8)


def main():
    import torchac_cuda as ref  # the reference build
    from oracle import cg_oracle as oracle
    out = {}
    all_ok = True
    for name, rows, T, C, mb, nsym, conc, seed in CASES:
        sym = symbols(rows, T, C, nsym, conc, seed)
        sym_t = torch.from_numpy(sym).cuda()
        cdf_t = ref.calculate_cdf(sym_t, mb)
        buf = torch.zeros((rows, C, 256), dtype=torch.uint8, device="cuda")
        lens = torch.zeros((rows, C), dtype=torch.int32, device="cuda")
        ref.encode_fast_new(cdf_t, sym_t, buf, lens)
        torch.cuda.synchronize()
        b, l = buf.cpu().numpy(), lens.cpu().numpy()
        assert l.max() <= 256
        flat = np.concatenate([b[r, c, :l[r, c]] for r in range(rows) for c in range(C)])
        pref = lens.flatten().cumsum(0).reshape(lens.shape)
        dec = torch.zeros((rows, T, C), dtype=torch.uint8, device="cuda")
        ref.decode_fast_prefsum(cdf_t, torch.from_numpy(flat).cuda(), pref, dec)
        dec2 = torch.zeros((rows, T, C), dtype=torch.uint8, device="cuda")
        ref.decode_fast_new(cdf_t, buf, lens, dec2)
        torch.cuda.synchronize()
        assert torch.equal(dec.cpu(), torch.from_numpy(sym.view(np.uint8))), name
        assert torch.equal(dec2, dec), name
        out[f"{name}_meta"] = np.array([rows, T, C, mb, nsym, seed], dtype=np.int64)
        out[f"{name}_conc"] = np.array([conc])
        out[f"{name}_cdf"] = cdf_t.cpu().numpy()
        out[f"{name}_lengths"] = l
        out[f"{name}_bytes"] = flat
        o_cdf = oracle.calculate_cdf(sym, mb)
        o_bytes, o_len = oracle.encode_chunk(o_cdf, sym)
        ok = (o_cdf == out[f"{name}_cdf"]).all() and (o_len == l).all() and o_bytes.tobytes() == flat.tobytes()
        print(f"{name}: oracle {'==' if ok else '!='} reference extension "
              f"({flat.size} stream bytes, max stream {l.max()} B)")
        all_ok &= bool(ok)
    # what a CUDA float -> int8 cast makes of the NaN an all-zero token row produces
    # (torch_quant_vectorized, cachegen_encoder.py:54-57 of the reference, on the GPU)
    x = torch.zeros(1, 2, 8, dtype=torch.float16, device="cuda")
    x[0, 1] = torch.tensor([0.5, -1.0, 0.25, 1.0] * 2, dtype=torch.float16)
    bins = torch.tensor([16.0], device="cuda")
    MAX = (bins // 2 - 1)[:, None, None]
    max1 = torch.amax(torch.abs(x), dim=-1, keepdim=True)
    xq = torch.round(x * (MAX / max1) + MAX).to(torch.int8)
    out["cuda_quant_zero_row"] = xq.cpu().numpy()
    print("CUDA symbols of an all-zero row:", xq[0, 0].tolist(), " tie row:", xq[0, 1].tolist())
    path = sys.argv[1] if len(sys.argv) > 1 else os.path.join(ROOT, "tests", "golden", "ref_cuda_ext.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes; oracle agrees with the reference:", all_ok)
    return 0 if all_ok else 1


if __name__ == "__main__":
    sys.exit(main())
