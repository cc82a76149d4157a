"""Generates tests/golden/ref_python_cpu.npz by running the REFERENCE's own Python functions on CPU.

Needs the reference checkout (path in CACHEGEN_REFERENCE_ROOT or the first argument); the modules it
imports at top level but that are absent offline (torchac, torchac_cuda, nvtx, redis) are stubbed, and
only pure-torch functions are called:

    torch_quant_vectorized   LMCache/lmcache/storage_backend/serde/cachegen_encoder.py:42-59
    do_dequantize            LMCache/lmcache/storage_backend/serde/cachegen_decoder.py:24-34
    CacheGenConfig.from_model_name / make_key_bins / make_value_bins   cachegen_basics.py:23-96,
                                                                       cachegen_encoder.py:311-322

The fixture pins the oracle's quantise / dequantise arithmetic (tests/test_oracle_golden.py) and,
through the oracle, the CUDA kernels.  Inputs are small seeded tensors that include exact rounding
ties, an all-zero token row, negative zero and outlier channels.
"""
import os
import sys
import types

import numpy as np
import torch


def import_reference(root):
    for name in ("torchac", "torchac_cuda", "redis"):
        sys.modules.setdefault(name, types.ModuleType(name))
    nvtx = types.ModuleType("nvtx")
    nvtx.annotate = lambda *a, **k: (lambda f: f)
    nvtx.start_range = lambda *a, **k: None
    nvtx.end_range = lambda *a, **k: None
    sys.modules.setdefault("nvtx", nvtx)
    sys.path.insert(0, os.path.join(root, "LMCache"))
    import lmcache.storage_backend.serde.cachegen_basics as basics
    import lmcache.storage_backend.serde.cachegen_decoder as dec
    import lmcache.storage_backend.serde.cachegen_encoder as enc
    return basics, enc, dec


def bits(t):
    return t.contiguous().view(torch.int16).numpy().view(np.uint16).copy()


def main():
    root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("CACHEGEN_REFERENCE_ROOT", "/root/reference")
    basics, enc, dec = import_reference(root)
    out = {}
    g = torch.Generator().manual_seed(1234)
    L, T, C = 6, 9, 64
    for tag, dtype in (("f16", torch.float16), ("bf16", torch.bfloat16)):
        x = torch.randn(L, T, C, generator=g) * torch.exp(0.5 * torch.randn(1, 1, C, generator=g))
        x[:, :, 5] *= 10.0                       # outlier channel
        x[1, 3, :] = 0.0                         # all-zero token row (0 * inf -> NaN -> int8)
        x[2, 4, :] = torch.tensor([0.5, -1.0, 0.25, 1.0] * (C // 4))   # exact ties at bins=16
        x[3, 0, 7] = -0.0
        x = x.to(dtype)
        bins = torch.tensor([32, 32, 16, 16, 12, 8], dtype=torch.float32)
        xq, max1 = enc.torch_quant_vectorized(bins, x)
        assert xq.dtype == torch.int8 and max1.dtype == dtype
        out[f"quant_{tag}_x"] = bits(x)
        out[f"quant_{tag}_bins"] = bins.numpy()
        out[f"quant_{tag}_sym"] = xq.numpy()
        out[f"quant_{tag}_max"] = bits(max1)
        # dequantise every symbol value of every row against a spread of scales
        sym = torch.arange(31, dtype=torch.uint8).repeat(L, T, 3)[:, :, :C].contiguous()
        for r, b in enumerate(bins.tolist()):
            sym[r] %= int(2 * (b // 2 - 1) + 1)
        deq = dec.do_dequantize(sym.float(), bins, max1)
        out[f"deq_{tag}_sym"] = sym.numpy()
        out[f"deq_{tag}_f16"] = bits(deq.to(torch.float16))
        out[f"deq_{tag}_bf16"] = bits(deq.to(torch.bfloat16))
    # the bins vectors of the built-in configurations
    os.environ["QUANT_LEVEL"] = "2"
    for name in ("lmsys/longchat-7b-16k", "Yukang/LongAlpaca-70B-16k", "mistralai/Mistral-7B-Instruct-v0.2"):
        cfg = basics.CacheGenConfig.from_model_name(name)
        kb = torch.zeros(cfg.key_third_layers)
        kb.fill_(cfg.key_third_bins)
        kb[:cfg.key_second_layers] = cfg.key_second_bins
        kb[:cfg.key_first_layers] = cfg.key_first_bins
        vb = torch.zeros(cfg.key_third_layers)
        vb.fill_(cfg.value_second_bins)
        vb[:cfg.value_first_layers] = cfg.value_first_bins
        key = name.split("/")[1]
        out[f"bins_{key}_k"] = kb.numpy()
        out[f"bins_{key}_v"] = vb.numpy()
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "ref_python_cpu.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
