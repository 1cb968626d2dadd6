"""Pair-biased, key-masked attention with the call signature of the reference's ``TritonEvoformer``.

Mirrors ``EvoformerAttention`` / ``TritonEvoformer`` of
megafold/model/FusedEvoAttention/evoattention.py:688-905: five positional tensors
``(Q, K, V, res_mask, pair_bias)``, output ``[B, N, L, H, D]``, gradients
``(dQ, dK, dV, None, d_pair_bias)``.  The work is done by the CUDA library behind the C ABI
(``mf_evo_fwd`` / ``mf_evo_bwd``); tensors on any other device are rejected.

Differences from the reference, all on purpose:
  * no transposed copies: the kernels read and write the ``[B, N, L, H, D]`` layout directly and
    accept strided q/k/v;
  * a boolean (or uint8) ``res_mask`` is a keep-mask with the semantics of the reference's PyTorch
    attention (``masked_fill(~mask, -finfo.max)``, megafold/model/attention.py:522-524); a floating
    ``res_mask`` is added to the logits, which is what the reference kernel does (evoattention.py:66);
  * ``d_pair_bias`` is accumulated in fp32 in a fixed order on every kernel path (bit-reproducible; the
    reference adds rows with atomics, evoattention.py:465) and returned in ``pair_bias.dtype``; the reference
    rounds it to ``dO.dtype`` first (evoattention.py:903).  ``dQ`` is bit-reproducible too unless the
    tensor-core path has to sum partial rows with fp32 atomics (very few rows, or L > 768).
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib

__all__ = ["EvoformerAttention", "TritonEvoformer", "evo_attention_forward", "evo_attention_backward"]


def _check_shapes(q, k, v, res_mask, pair_bias):
    if q.dim() != 5:
        raise ValueError(f"Q must be [B, N_seq, N_res, Head, Dim], got {tuple(q.shape)}")
    B, N, L, H, D = q.shape
    if k.shape != q.shape or v.shape != q.shape:
        raise ValueError(f"Q, K, V shapes differ: {tuple(q.shape)} {tuple(k.shape)} {tuple(v.shape)}")
    if not (q.dtype == k.dtype == v.dtype):
        raise TypeError("Q, K, V must share a dtype")
    if res_mask is None or pair_bias is None:
        raise ValueError("res_mask and pair_bias are mandatory")
    if tuple(pair_bias.shape[1:]) != (1, H, L, L) or pair_bias.shape[0] not in (1, B):
        raise ValueError(f"pair_bias must be [B, 1, Head, N_res, N_res], got {tuple(pair_bias.shape)}")
    if res_mask.dim() != 5 or res_mask.shape[2:4] != (1, 1) or res_mask.shape[4] != L \
            or res_mask.shape[0] not in (1, B) or res_mask.shape[1] not in (1, N):
        raise ValueError(f"res_mask must be [B, N_seq, 1, 1, N_res], got {tuple(res_mask.shape)}")
    return B, N, L, H, D


def _fill_common(a, q, k, v, res_mask, pair_bias, flags):
    B, N, L, H, D = q.shape
    a.B, a.N, a.L, a.H, a.D = B, N, L, H, D
    a.dtype = _lib.dtype_code(q.dtype)
    a.bias_dtype = _lib.dtype_code(pair_bias.dtype)
    a.mask_dtype = _lib.dtype_code(res_mask.dtype)
    a.flags = flags
    a.q, a.k, a.v = q.data_ptr(), k.data_ptr(), v.data_ptr()
    a.q_strides[:] = q.stride()
    a.k_strides[:] = k.stride()
    a.v_strides[:] = v.stride()
    m = res_mask.expand(B, N, 1, 1, L)
    a.mask = m.data_ptr()
    a.mask_strides[:] = (m.stride(0), m.stride(1), m.stride(4))
    pb = pair_bias.expand(B, 1, H, L, L)
    a.bias = pb.data_ptr()
    a.bias_strides[:] = (pb.stride(0), pb.stride(2), pb.stride(3), pb.stride(4))


def evo_attention_forward(q, k, v, res_mask, pair_bias, flags: int = 0):
    """Returns ``(O [B,N,L,H,D], LSE fp32 [B,N,H,L])``; ``mf_evo_fwd`` of the C ABI."""
    _lib.require_cuda(q, k, v, res_mask, pair_bias)
    B, N, L, H, D = _check_shapes(q, k, v, res_mask, pair_bias)
    o = torch.empty((B, N, L, H, D), dtype=q.dtype, device=q.device)
    lse = torch.empty((B, N, H, L), dtype=torch.float32, device=q.device)
    a = _lib.EvoFwdArgs()
    _fill_common(a, q, k, v, res_mask, pair_bias, flags)
    a.o, a.lse = o.data_ptr(), lse.data_ptr()
    with torch.cuda.device(q.device):
        _lib.check(_lib.lib().mf_evo_fwd(C.byref(a), _lib.stream_ptr(q.device)), "mf_evo_fwd")
    return o, lse


def evo_attention_backward(d_o, q, k, v, res_mask, pair_bias, o, lse, flags: int = 0, dbias_ready=None):
    """Returns ``(dQ, dK, dV, dBias)``; dBias has ``pair_bias``'s shape and dtype. ``mf_evo_bwd``.

    ``dbias_ready``: an optional ``torch.cuda.Event`` that the library records on the current stream as soon as dBias is
    final (before dQ / dK / dV on the tensor-core path), for callers that reduce dBias over row shards on another stream."""
    _lib.require_cuda(d_o, q, k, v, res_mask, pair_bias, o, lse)
    B, N, L, H, D = _check_shapes(q, k, v, res_mask, pair_bias)
    d_o = d_o.contiguous()
    o = o.contiguous()
    dq, dk, dv = (torch.empty((B, N, L, H, D), dtype=q.dtype, device=q.device) for _ in range(3))
    direct = pair_bias.dtype in (torch.float32, q.dtype)
    db_dtype = pair_bias.dtype if direct else torch.float32
    d_bias = torch.empty((B, 1, H, L, L), dtype=db_dtype, device=q.device)
    a = _lib.EvoBwdArgs()
    _fill_common(a, q, k, v, res_mask, pair_bias, flags)
    a.dbias_dtype = _lib.dtype_code(db_dtype)
    a.o, a.d_o, a.lse = o.data_ptr(), d_o.data_ptr(), lse.data_ptr()
    a.dq, a.dk, a.dv, a.d_bias = dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), d_bias.data_ptr()
    L_ = _lib.lib()
    with torch.cuda.device(q.device):
        if dbias_ready is not None:
            dbias_ready.record()                     # creates the underlying cudaEvent_t; the library records it again
            a.dbias_ready_event = dbias_ready.cuda_event
        need = L_.mf_evo_bwd_workspace_bytes(C.byref(a))
        ws = _lib.workspace(need, q.device)
        a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
        _lib.check(L_.mf_evo_bwd(C.byref(a), _lib.stream_ptr(q.device)), "mf_evo_bwd")
    if pair_bias.shape[0] != B:                      # bias broadcast over the batch
        d_bias = d_bias.sum(dim=0, keepdim=True)
    if d_bias.dtype != pair_bias.dtype:
        d_bias = d_bias.to(pair_bias.dtype)
    return dq, dk, dv, d_bias


class EvoformerAttention(torch.autograd.Function):
    """Q, K, V: [Batch, N_seq, N_res, Head, Dim]; res_mask: [Batch, N_seq, 1, 1, N_res];
    pair_bias: [Batch, 1, Head, N_res, N_res] (shared by the N_seq rows)."""

    @staticmethod
    def forward(ctx, Q, K, V, res_mask, pair_bias):
        o, lse = evo_attention_forward(Q, K, V, res_mask, pair_bias)
        ctx.save_for_backward(Q, K, V, res_mask, pair_bias, o, lse)
        return o

    @staticmethod
    def backward(ctx, dO):
        Q, K, V, res_mask, pair_bias, o, lse = ctx.saved_tensors
        dq, dk, dv, d_bias = evo_attention_backward(dO, Q, K, V, res_mask, pair_bias, o, lse)
        return dq, dk, dv, None, d_bias


TritonEvoformer = EvoformerAttention.apply
