"""Seeded synthetic workloads with the shapes and value distributions of the benchmark configurations.

The reference measures these operators on ``torch.randn`` tensors (benchmarks/evoattention_speed.py:59-77,
benchmarks/transition_speed.py:64-95); no dataset is involved.  Everything is generated on the CPU from
``torch.Generator().manual_seed(seed)`` so that the GPU run and the CPU oracle see identical inputs.
"""
from __future__ import annotations

import torch

__all__ = ["triangle_attention", "single_attention", "transition", "layernorm_linear", "CONFIGS"]


def triangle_attention(L=384, N=None, H=4, D=32, B=1, dtype=torch.bfloat16, pad=32, seed=0, bias_dtype=None):
    """q, k, v, d_out [B,N,L,H,D] ~ N(0,1); pair_bias [B,1,H,L,L] ~ N(0,1); res_mask True for the first
    L - pad tokens of every row (padding at the tail)."""
    N = L if N is None else N
    g = torch.Generator().manual_seed(seed)
    q, k, v = (torch.randn(B, N, L, H, D, generator=g).to(dtype) for _ in range(3))
    bias = torch.randn(B, 1, H, L, L, generator=g).to(bias_dtype or dtype)
    d_out = torch.randn(B, N, L, H, D, generator=g).to(dtype)
    mask = torch.ones(B, N, 1, 1, L, dtype=torch.bool)
    if pad:
        mask[..., L - pad:] = False
    return dict(q=q, k=k, v=v, mask=mask, bias=bias, d_out=d_out)


def single_attention(L=768, H=16, D=24, B=2, dtype=torch.bfloat16, drop=0.1, seed=0):
    """Single-representation attention with pair bias: N = 1, a random 10% of the keys masked per batch
    element (at least one kept)."""
    g = torch.Generator().manual_seed(seed)
    q, k, v = (torch.randn(B, 1, L, H, D, generator=g).to(dtype) for _ in range(3))
    bias = torch.randn(B, 1, H, L, L, generator=g).to(dtype)
    d_out = torch.randn(B, 1, L, H, D, generator=g).to(dtype)
    mask = torch.rand(B, 1, 1, 1, L, generator=g) >= drop
    mask[..., 0] = True
    return dict(q=q, k=k, v=v, mask=mask, bias=bias, d_out=d_out)


def layernorm_linear(M=147456, K=128, N=512, dtype=torch.bfloat16, seed=0, bias=True):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g).to(dtype)
    w = (torch.randn(K, N, generator=g) / K ** 0.5).to(dtype)
    return dict(x=x, ln_w=torch.ones(K, dtype=dtype), ln_b=torch.zeros(K, dtype=dtype), w=w,
                b=(torch.zeros(N, dtype=dtype) if bias else None),
                d_out=torch.randn(M, N, generator=g).to(dtype))


def transition(M=512 * 512, dim=128, expansion=4, dtype=torch.bfloat16, seed=0):
    """x [M, dim] ~ N(0,1); gamma 1, beta 0; w1 [dim, 2*inner] ~ N(0, 1/dim); w2 [dim, inner] ~ N(0, 1/inner)."""
    inner = dim * expansion
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, dim, generator=g).to(dtype)
    w1 = (torch.randn(dim, 2 * inner, generator=g) / dim ** 0.5).to(dtype)
    w2 = (torch.randn(dim, inner, generator=g) / inner ** 0.5).to(dtype)
    d_out = torch.randn(M, dim, generator=g).to(dtype)
    return dict(x=x, ln_w=torch.ones(dim, dtype=dtype), ln_b=torch.zeros(dim, dtype=dtype), w1=w1, w2=w2, d_out=d_out)


CONFIGS = {
    "cfg1_tiny_fp32": lambda: triangle_attention(L=64, N=64, dtype=torch.float32, pad=8),
    "cfg2_triangle_L384": lambda: triangle_attention(L=384),
    "cfg3_single_L768": lambda: single_attention(),
    "cfg4_transition_512": lambda: transition(),
}
