"""fp32/fp64 PyTorch restatement of the reference's own PyTorch paths.

TEST INFRASTRUCTURE ONLY: the shipped package never imports this file.

Each function follows one PyTorch code path of the reference (cited by
path:line inside the MegaFold project) and is pinned against outputs of the
reference's own classes, produced by ``tests/golden/make_golden.py`` and stored
under ``tests/golden/`` (checked by ``tests/test_oracle_golden.py``).

Conventions (identical to the reference's fused operators):
  q, k, v     [B, N, L, H, D]   N independent rows, L tokens, H heads
  res_mask    [B, N, 1, 1, L]   bool keep-mask (True = attend) or a floating
                                tensor that is ADDED to the logits
  pair_bias   [B, 1, H, L, L]   shared by the N rows
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

__all__ = [
    "evo_attention", "evo_attention_fwd_bwd", "layernorm_linear",
    "layernorm_linear_fwd_bwd", "swiglu", "transition", "transition_fwd_bwd",
    "evo_flops", "gemm_flops",
]


def evo_attention(q, k, v, res_mask, pair_bias, compute_dtype=torch.float32):
    """softmax(q*D^-1/2 @ k^T + pair_bias, masked) @ v, per row n.

    Follows ``Attend.forward`` default branch, megafold/model/attention.py:500-539:
    scale q (:502-504), einsum 'b h i d, b h j d' (:508), add attn_bias
    (:512-513), ``masked_fill(~mask, -finfo.max)`` (:522-524), softmax over j
    (:535), einsum with v (:539); with the [B,N,L,H,D] <-> [(B N),H,L,D]
    mapping of attention.py:469-480.  A floating mask is added to the logits,
    which is what the reference's test oracle does
    (tests/test_evoattention.py:35-36,49-56).
    """
    B, N, L, H, D = q.shape
    cd = compute_dtype
    qf = q.to(cd).permute(0, 1, 3, 2, 4).reshape(B * N, H, L, D)
    kf = k.to(cd).permute(0, 1, 3, 2, 4).reshape(B * N, H, L, D)
    vf = v.to(cd).permute(0, 1, 3, 2, 4).reshape(B * N, H, L, D)
    scale = D ** -0.5
    qf = qf * scale
    sim = torch.einsum("bhid,bhjd->bhij", qf, kf)
    bias = pair_bias.to(cd).expand(B, N, H, L, L).reshape(B * N, H, L, L)
    sim = sim + bias
    m = res_mask.reshape(B * N, L)
    if m.dtype in (torch.bool, torch.uint8):
        keep = m.bool()
        sim = sim.masked_fill(~keep[:, None, None, :], -torch.finfo(sim.dtype).max)
    else:
        sim = sim + m.to(cd)[:, None, None, :]
    attn = sim.softmax(dim=-1)
    out = torch.einsum("bhij,bhjd->bhid", attn, vf)
    return out.reshape(B, N, H, L, D).permute(0, 1, 3, 2, 4).contiguous()


def evo_attention_fwd_bwd(q, k, v, res_mask, pair_bias, d_out, compute_dtype=torch.float32):
    """Forward plus autograd gradients (dQ, dK, dV, dBias) in ``compute_dtype``.

    Gradient definitions match ``EvoformerAttention.backward``
    (megafold/model/FusedEvoAttention/evoattention.py:783-903): dBias is the
    sum of dS over the N rows that share the bias.
    """
    cd = compute_dtype
    qq, kk, vv, bb = (t.detach().to(cd).clone().requires_grad_(True) for t in (q, k, v, pair_bias))
    out = evo_attention(qq, kk, vv, res_mask, bb, compute_dtype=cd)
    out.backward(d_out.to(cd))
    return out.detach(), qq.grad, kk.grad, vv.grad, bb.grad


def layernorm_linear(x, ln_weight, ln_bias, linear_weight, linear_bias, eps=1e-5):
    """Y = LayerNorm_K(x) @ linear_weight[K,N] + linear_bias.

    This is the reference's torch fallback line,
    megafold/model/FusedLayernormLinear/fused_layernorm_linear.py:541
    (weight stored [K,N], :511; eps 1e-5, :368).
    """
    K = x.shape[-1]
    return F.linear(F.layer_norm(x, (K,), ln_weight, ln_bias, eps), linear_weight.T, linear_bias)


def layernorm_linear_fwd_bwd(x, ln_weight, ln_bias, linear_weight, linear_bias, d_out,
                             compute_dtype=torch.float32):
    cd = compute_dtype
    leaves = [t.detach().to(cd).clone().requires_grad_(True) if t is not None else None
              for t in (x, ln_weight, ln_bias, linear_weight, linear_bias)]
    y = layernorm_linear(*leaves)
    y.backward(d_out.to(cd))
    return (y.detach(),) + tuple(t.grad if t is not None else None for t in leaves)


def swiglu(x):
    """silu(right half) * left half; benchmarks/transition_speed.py:38-39 and
    megafold/model/FusedTransition/fused_transition.py:55-59."""
    a, gates = x.chunk(2, dim=-1)
    return F.silu(gates) * a


def transition(x, ln_weight, ln_bias, w1, w2, eps=1e-5):
    """LayerNorm -> Linear(dim -> 2*inner, no bias) -> SwiGLU -> Linear(inner -> dim, no bias).

    ``w1`` is stored [dim, 2*inner] (the LayernormLinear convention), ``w2`` is
    ``nn.Linear.weight`` [dim, inner].  Follows benchmarks/transition_speed.py:8-39
    and megafold/model/FusedTransition/fused_transition.py:128-132.  ``ln_weight``
    None means no LayerNorm (the include_ln=False variant, :140-145).
    """
    if ln_weight is not None:
        h = layernorm_linear(x, ln_weight, ln_bias, w1, None, eps)
    else:
        h = x @ w1
    return F.linear(swiglu(h), w2)


def transition_fwd_bwd(x, ln_weight, ln_bias, w1, w2, d_out, compute_dtype=torch.float32):
    cd = compute_dtype
    leaves = [t.detach().to(cd).clone().requires_grad_(True) if t is not None else None
              for t in (x, ln_weight, ln_bias, w1, w2)]
    y = transition(*leaves)
    y.backward(d_out.to(cd))
    return (y.detach(),) + tuple(t.grad if t is not None else None for t in leaves)


def evo_flops(B, N, H, L, D, mode="fwd+bwd"):
    """Algorithmic FLOPs: one matmul = 2*B*N*H*L*L*D; forward 2 matmuls,
    backward 5 (convention of benchmarks/evoattention_speed.py:110-116, with
    the 2.5x backward factor and an explicit N)."""
    one = 2.0 * B * N * H * L * L * D
    return {"fwd": 2 * one, "bwd": 5 * one, "fwd+bwd": 7 * one}[mode]


def gemm_flops(M, K, N, mode="fwd+bwd"):
    one = 2.0 * M * K * N
    return {"fwd": one, "bwd": 2 * one, "fwd+bwd": 3 * one}[mode]
