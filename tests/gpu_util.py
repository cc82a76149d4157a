"""Helpers shared by the GPU parity tests."""
import numpy as np
import torch


def bits_np(t):
    """16-bit float tensor -> numpy uint16 bit patterns."""
    return t.detach().contiguous().cpu().view(torch.int16).numpy().view(np.uint16)


def from_bits(a, dtype, device="cuda"):
    return torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).view(dtype).to(device)


def peaked_symbols(rng, shape, nsym, conc=0.3):
    p = rng.dirichlet(np.full(nsym, conc))
    return rng.choice(nsym, size=shape, p=p).astype(np.int8)


def kv_rows(kv_vllm):
    """vllm blob [L,2,T,H,D] -> the codec's row order [2L, T, C] (keys then values)."""
    L, _, T, H, D = kv_vllm.shape
    return kv_vllm.reshape(L, 2, T, H * D).transpose(0, 1).reshape(2 * L, T, H * D).contiguous()
