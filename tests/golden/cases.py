"""Seeded inputs shared by the golden-vector generator and the tests that read the vectors.

numpy's legacy ``RandomState`` is used because its streams are frozen across
numpy versions, so inputs that are too large to commit can be regenerated
bit-identically from the seed.
"""
import numpy as np
import torch


def _rs(seed):
    return np.random.RandomState(seed)


def randn(rs, *shape):
    return torch.from_numpy(rs.standard_normal(shape).astype(np.float32))


def evo_cfg1():
    """Triangle attention, fp32, q/k/v [1,64,64,4,32], bias [1,1,4,64,64],
    bool mask [1,64,1,1,64] with the last 8 keys of every row masked; seed 0."""
    rs = _rs(0)
    B, N, L, H, D = 1, 64, 64, 4, 32
    q, k, v = (randn(rs, B, N, L, H, D) for _ in range(3))
    bias = randn(rs, B, 1, H, L, L)
    d_out = randn(rs, B, N, L, H, D)
    mask = torch.ones(B, N, 1, 1, L, dtype=torch.bool)
    mask[..., L - 8:] = False
    return dict(q=q, k=k, v=v, mask=mask, bias=bias, d_out=d_out)


def evo_small():
    """Ragged small case: B=2, N=3, L=24, H=2, D=16, random key mask (>= 1 kept)."""
    rs = _rs(1)
    B, N, L, H, D = 2, 3, 24, 2, 16
    q, k, v = (randn(rs, B, N, L, H, D) * 0.5 for _ in range(3))
    bias = randn(rs, B, 1, H, L, L)
    d_out = randn(rs, B, N, L, H, D)
    mask = torch.from_numpy(rs.uniform(size=(B, N, 1, 1, L)) > 0.3)
    mask[..., 0] = True
    return dict(q=q, k=k, v=v, mask=mask, bias=bias, d_out=d_out)


LNL_SHAPES = [(18, 31, 99), (64, 48, 128), (7, 16, 128)]      # (M, N, K)
TRANSITION_SHAPES = [(40, 32, 4), (33, 64, 2)]               # (M, dim, expansion)

# strided sub-sampling applied to the cfg1 outputs that are too large to commit whole
CFG1_SUB = (slice(None), slice(None, None, 8), slice(None, None, 8))
