"""Row-sharded triangle attention for long crops.

The N rows of ``Q, K, V [B, N, L, H, D]`` are independent in the forward pass
(megafold/model/FusedEvoAttention/evoattention.py:179-185 maps one program to one (b, n, h)), so a
crop is split over ranks along N with no forward communication.  The only shared quantity is
``pair_bias [B, 1, H, L, L]``: its gradient is the sum of dS over ALL rows, so every rank's partial
d_pair_bias is all-reduced (NCCL over NVLink on GPUs, gloo in the CPU tests).  The reference never
shards a crop; this is an addition for the 8-GPU long-crop configuration.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

__all__ = ["AllReduceGradient", "row_shard", "sharded_evoformer"]


class AllReduceGradient(torch.autograd.Function):
    """Identity in forward; sums the gradient over the process group in backward."""

    @staticmethod
    def forward(ctx, x, group=None):
        ctx.group = group
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        if dist.is_available() and dist.is_initialized() and dist.get_world_size(ctx.group) > 1:
            g = g.contiguous()
            dist.all_reduce(g, op=dist.ReduceOp.SUM, group=ctx.group)
        return g, None


def row_shard(n_rows: int, rank: int, world: int):
    """Contiguous block ``[start, stop)`` of the N rows owned by ``rank`` (the first ``n_rows % world``
    ranks get one extra row)."""
    if not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world of {world}")
    base, extra = divmod(n_rows, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def sharded_evoformer(q, k, v, res_mask, pair_bias, group=None, attention=None):
    """``TritonEvoformer`` on this rank's rows; ``pair_bias`` is replicated and receives the
    all-reduced gradient.  ``attention`` defaults to the CUDA operator (the CPU tests pass an oracle)."""
    if attention is None:
        from .evoattention import TritonEvoformer as attention
    return attention(q, k, v, res_mask, AllReduceGradient.apply(pair_bias, group))
