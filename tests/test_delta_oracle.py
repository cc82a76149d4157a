"""The anchor-token delta definition (oracle/cg_oracle.c: cgo_quantize_delta / cgo_dequantize_delta): its
invariants, and the rate-distortion evaluation that says where it pays.  CPU only."""
import math

import numpy as np
import pytest
import torch


def bits(t):
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def to_float(b):
    return torch.from_numpy(np.ascontiguousarray(b).view(np.int16)).view(torch.float16).float()


def test_delta_off_and_anchor_tokens_equal_the_plain_quantiser(oracle):
    g = torch.Generator().manual_seed(3)
    x = (torch.randn(4, 96, 200, generator=g).cumsum(1) * 0.2).to(torch.float16)
    bins = np.array([32, 16, 32, 16], dtype=np.float32)
    s0, m0 = oracle.quantize(bits(x), bins)
    s1, m1 = oracle.quantize_delta(bits(x), bins, np.zeros(4, dtype=np.float32), 8)
    assert (s0 == s1).all() and (m0 == m1).all()
    res = np.array([16, 8, 0, 4], dtype=np.float32)
    s2, m2 = oracle.quantize_delta(bits(x), bins, res, 8)
    assert (s2[2] == s0[2]).all() and (m2[2] == m0[2]).all()           # a row without residual bins
    assert (s2[:, ::8] == s0[:, ::8]).all() and (m2[:, ::8] == m0[:, ::8]).all()  # anchors
    # residual symbols stay inside [Cq_a - Cq_r, Cq_a + Cq_r]
    for r, (b, rb) in enumerate(zip(bins, res)):
        if rb > 0:
            cqa, cqr = int(b) // 2 - 1, int(rb) // 2 - 1
            rest = np.delete(s2[r], np.s_[::8], axis=0)
            assert rest.min() >= cqa - cqr and rest.max() <= cqa + cqr
    with pytest.raises(ValueError):
        oracle.quantize_delta(bits(x), bins, np.array([64, 0, 0, 0], dtype=np.float32), 8)  # Cq_r > Cq_a


def test_delta_round_trip_stays_within_the_residual_quantiser_step(oracle):
    g = torch.Generator().manual_seed(4)
    x = (torch.randn(2, 64, 512, generator=g).cumsum(1) * 0.1).to(torch.float16)
    bins = np.array([32, 32], dtype=np.float32)
    res = np.array([16, 16], dtype=np.float32)
    sym, mx = oracle.quantize_delta(bits(x), bins, res, 4)
    rec = to_float(oracle.dequantize_delta(sym, bins, res, 4, mx))
    step = to_float(mx).reshape(2, 64, 1)
    cq = torch.full((2, 64, 1), 7.0)
    cq[:, ::4] = 15.0
    # half a quantiser step of the token's own scale, plus the fp16 round-off of the sum
    bound = 0.5 * step / cq * 1.001 + x.float().abs() * 2.0 ** -10 + 1e-3
    assert bool(((rec - x.float()).abs() <= bound).all())


def _entropy_bits(q, nsym):
    T, C = q.shape
    counts = torch.zeros(C, nsym).scatter_add_(1, q.t().long(), torch.ones(C, T))
    p = counts / T
    return float(-(p * torch.log2(p.clamp_min(1e-12))).sum() * T)


def _point(oracle, x, bins_value, res_value, group):
    """(payload bytes, mean squared error) of rows x [R, T, C] at one setting; res_value 0 = no delta.
    Anchors and residuals get separate per-channel tables: the best case for delta."""
    R, T, C = x.shape
    bins = np.full(R, bins_value, dtype=np.float32)
    res = np.full(R, res_value, dtype=np.float32)
    sym, mx = oracle.quantize_delta(bits(x), bins, res, group)
    rec = to_float(oracle.dequantize_delta(sym, bins, res, group, mx))
    mse = float(((rec - x.float()) ** 2).mean())
    nsym = 2 * (int(bins_value) // 2 - 1) + 1
    total = 0.0
    for r in range(R):
        q = torch.from_numpy(sym[r].astype(np.int64))
        if res_value > 0:
            anchors = torch.arange(T) % group == 0
            total += _entropy_bits(q[anchors], nsym) + _entropy_bits(q[~anchors], nsym)
        else:
            total += _entropy_bits(q, nsym)
    return total / 8, mse


def _interpolate(curve, mse):
    curve = sorted(curve, key=lambda p: p[1])
    for (b0, m0), (b1, m1) in zip(curve, curve[1:]):
        if m0 <= mse <= m1:
            w = (math.log(mse) - math.log(m0)) / (math.log(m1) - math.log(m0))
            return math.exp(math.log(b0) * (1 - w) + math.log(b1) * w)
    return None


def test_where_anchor_delta_pays_at_equal_distortion(oracle):
    """Bytes at equal mean squared error on the benchmark generator (one key row and one value row of
    a 256-token Llama-7B-shape chunk, 1,024 of the 4,096 channels): values never gain, keys gain with
    groups of 4 and coarser residual bins, the more the smoother the series is; longer groups lose."""
    from cachegen_b200.synth import generate_kv
    wins = {}
    for rho in (0.9, 0.95):
        kv = generate_kv(1, 8, 128, 256, 1, key_rho=rho, device="cpu", dtype=torch.float16, first_layer=12)
        for name, which in (("K", 0), ("V", 1)):
            x = kv[0, which].reshape(1, 256, 1024)
            curve = [_point(oracle, x, b, 0, 1) for b in (24, 20, 16, 12, 8, 6, 4)]
            for group in (4, 16):
                for res in (8, 4):
                    b, m = _point(oracle, x, 16, res, group)
                    ref = _interpolate(curve, m)
                    if ref is not None:
                        wins[(rho, name, group, res)] = b / ref
    assert all(v > 1.0 for k, v in wins.items() if k[1] == "V")            # values: always more bytes
    assert all(v > 1.0 for k, v in wins.items() if k[2] == 16)             # long groups: always more bytes
    assert wins[(0.95, "K", 4, 8)] < 0.97 and wins[(0.9, "K", 4, 8)] < 1.0  # keys, groups of 4, half the bins
    assert wins[(0.95, "K", 4, 8)] < wins[(0.9, "K", 4, 8)] + 0.02          # smoother keys gain at least as much
