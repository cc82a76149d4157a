"""Seeded synthetic KV caches with the statistics the benchmark configurations name.

Real KV caches need model weights and prompts that are not available offline, so the benchmark and
the parity tests use this generator instead:

    K[l, t, h, d] = s_K[l, h, d] * x,   x an AR(1) series along t (rho = 0.9 by default, unit-normal
                                         innovations, stationary start), s_K ~ lognormal(0, 0.5),
                                         2 % of the (h, d) channels scaled by 10 as outliers
    V[l, t, h, d] = s_V[l, h, d] * y,   y AR(1) with rho = 0.6, s_V ~ lognormal(0, 0.3), no outliers

Every (seed, layer, K-or-V) slab has its own torch.Generator, so a single layer can be regenerated
alone.  The values depend on the device the generator runs on (CPU and CUDA generators differ): use
device="cpu" wherever bit-reproducible inputs matter and move the result.
"""
import math

import torch

_BLOCK = 64


def _ar1(e: torch.Tensor, rho: float) -> torch.Tensor:
    """AR(1) filter along dim 0 of e [T, C]: x_t = rho * x_{t-1} + e_t, x_0 = e_0 / sqrt(1 - rho^2)."""
    T, C = e.shape
    e = e.clone()
    e[0] /= math.sqrt(1.0 - rho * rho)
    pad = (-T) % _BLOCK
    if pad:
        e = torch.cat((e, e.new_zeros(pad, C)))
    nb = e.shape[0] // _BLOCK
    idx = torch.arange(_BLOCK, device=e.device)
    lag = (idx[:, None] - idx[None, :]).clamp(min=0).to(e.dtype)
    M = torch.where(idx[:, None] >= idx[None, :], rho ** lag, torch.zeros((), dtype=e.dtype, device=e.device))
    y = torch.matmul(M, e.view(nb, _BLOCK, C))  # within-block response, zero carry-in
    decay = (rho ** (idx + 1).to(e.dtype))[:, None]  # effect of the carry on the block's rows
    carry = e.new_zeros(C)
    for b in range(nb):
        y[b] += decay * carry
        carry = y[b, -1]
    return y.view(nb * _BLOCK, C)[:T]


def _slab(seed: int, layer: int, which: int, T: int, C: int, rho: float, sigma: float, outlier_frac: float,
          device) -> torch.Tensor:
    g = torch.Generator(device=device)
    g.manual_seed((seed * 1000003 + layer) * 2 + which)
    scale = torch.exp(sigma * torch.randn(C, generator=g, device=device))
    if outlier_frac > 0:
        mask = torch.rand(C, generator=g, device=device) < outlier_frac
        scale = torch.where(mask, scale * 10.0, scale)
    e = torch.randn(T, C, generator=g, device=device)
    return _ar1(e, rho) * scale


def generate_kv(num_layers: int, num_heads: int, head_size: int, num_tokens: int, seed: int,
                key_rho: float = 0.9, value_rho: float = 0.6, device="cpu", dtype=torch.float16,
                out_device=None, first_layer: int = 0) -> torch.Tensor:
    """Returns a "vllm"-format blob [L, 2, T, H, D] in `dtype` on `out_device` (default: `device`):
    layers first_layer .. first_layer + num_layers - 1 of the cache with this seed."""
    C = num_heads * head_size
    out_device = out_device or device
    out = torch.empty((num_layers, 2, num_tokens, num_heads, head_size), dtype=dtype, device=out_device)
    for l in range(num_layers):
        k = _slab(seed, first_layer + l, 0, num_tokens, C, key_rho, 0.5, 0.02, device)
        v = _slab(seed, first_layer + l, 1, num_tokens, C, value_rho, 0.3, 0.0, device)
        out[l, 0] = k.view(num_tokens, num_heads, head_size).to(dtype).to(out_device)
        out[l, 1] = v.view(num_tokens, num_heads, head_size).to(dtype).to(out_device)
    return out


# The benchmark configurations: (layers, kv heads, head size, tokens, seed, key rho, model name)
WORKLOADS = {
    "llama7b-1k": dict(num_layers=32, num_heads=32, head_size=128, num_tokens=1024, seed=0, key_rho=0.9,
                       model_name="lmsys/longchat-7b-16k"),
    "llama7b-8k": dict(num_layers=32, num_heads=32, head_size=128, num_tokens=8192, seed=1, key_rho=0.9,
                       model_name="lmsys/longchat-7b-16k"),
    "mistral7b-gqa-32k": dict(num_layers=32, num_heads=8, head_size=128, num_tokens=32768, seed=2, key_rho=0.95,
                              model_name="lmsys/longchat-7b-16k"),
    "llama70b-gqa-16k": dict(num_layers=80, num_heads=8, head_size=128, num_tokens=16384, seed=3, key_rho=0.9,
                             model_name="Yukang/LongAlpaca-70B-16k"),
    "llama7b-4k": dict(num_layers=32, num_heads=32, head_size=128, num_tokens=4096, seed=100, key_rho=0.9,
                       model_name="lmsys/longchat-7b-16k"),
}
