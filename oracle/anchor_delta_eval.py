"""What anchor-token delta coding would do to the payload with this codec's quantiser (CPU, numpy/torch).

Test infrastructure, like the rest of oracle/: nothing in the product imports it.  It reproduces the
figures quoted for the "anchor delta" idea: tokens in groups of G, the first token of a group coded as
today, every other token coded as its difference from the *dequantised* anchor (closed loop) with its
own per-(row, token) scale, anchors and residuals with separate per-channel tables.  The cost of a
stream is taken as its empirical entropy under a per-channel table, which is what the arithmetic coder
reaches to within a fraction of a percent.

    python oracle/anchor_delta_eval.py            # ratio of payload with delta / without, G = 2, 4, 8, 16

The quantiser scales every token row by its own max|x| before rounding (cachegen_encoder.py:54-57 of
the reference), so a residual of smaller magnitude spreads over the bins just as the value did: the
ratio stays above 1.
"""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from cachegen_b200.serde.cachegen_basics import CacheGenConfig, make_key_bins, make_value_bins  # noqa: E402
from cachegen_b200.synth import generate_kv  # noqa: E402

ROWS = [0, 5, 12, 20, 31, 32, 33, 40, 50, 63]   # key rows of every bin group, then value rows


def quantize(x, bins):
    """x [T, C] float32 -> (symbols, per-token max, MAX) as torch_quant_vectorized computes them."""
    half = bins // 2 - 1
    m = x.abs().amax(-1, keepdim=True)
    return torch.round(x * (half / m) + half).long(), m, half


def table_entropy_bits(q, nsym):
    """Sum over channels of T * H(channel's symbol distribution)."""
    T, C = q.shape
    counts = torch.zeros(C, nsym).scatter_add_(1, q.t(), torch.ones(C, T))
    p = counts / T
    return float(-(p * torch.log2(p.clamp_min(1e-12))).sum() * T)


def payload_bytes(rows, bins, group):
    plain = delta = 0.0
    T = rows.shape[1]
    t = torch.arange(T)
    for r in ROWS:
        b, x = float(bins[r]), rows[r]
        q, m, half = quantize(x, b)
        nsym = int(2 * half + 1)
        plain += table_entropy_bits(q, nsym)
        anchor_value = ((q - half) / half * m).to(torch.float16).float()      # what a decoder would hold
        residual = x - anchor_value[(t // group) * group]
        is_anchor = t % group == 0
        delta += table_entropy_bits(quantize(x[is_anchor], b)[0], nsym)
        delta += table_entropy_bits(quantize(residual[~is_anchor], b)[0], nsym)
    return plain / 8, delta / 8


def main():
    L, H, D, T = 32, 32, 128, 256
    kv = generate_kv(L, H, D, T, 1, device="cpu", dtype=torch.float16)
    cfg = CacheGenConfig.from_model_name("lmsys/longchat-7b-16k")
    bins = torch.cat((make_key_bins(cfg, "cpu"), make_value_bins(cfg, "cpu")))
    rows = kv.reshape(L, 2, T, H * D).transpose(0, 1).reshape(2 * L, T, H * D).float()
    for group in (2, 4, 8, 16):
        plain, delta = payload_bytes(rows, bins, group)
        print(f"groups of {group:2d}: {plain / 1e3:9.1f} KB plain, {delta / 1e3:9.1f} KB with delta, ratio {delta / plain:.3f}")


if __name__ == "__main__":
    main()
