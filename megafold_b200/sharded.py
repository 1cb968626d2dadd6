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

__all__ = ["AllReduceGradient", "ShardedEvoformerAttention", "evo_attention_backward_sharded", "row_shard", "sharded_evoformer"]


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


def evo_attention_backward_sharded(d_o, q, k, v, res_mask, pair_bias, o, lse, group=None):
    """Backward of the attention on this rank's rows with the all-reduce of d_pair_bias overlapped: the library computes
    d_pair_bias first and signals an event; the collective then runs on a side stream while dQ / dK / dV are computed on
    the current one, which waits for the collective at the end.  Returns ``(dQ, dK, dV, dBias)`` with dBias summed over
    the group."""
    from .evoattention import evo_attention_backward
    if not (dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1):
        return evo_attention_backward(d_o, q, k, v, res_mask, pair_bias, o, lse)
    dev = q.device
    cur = torch.cuda.current_stream(dev)
    side = _side_stream(dev)
    ready = torch.cuda.Event()
    dq, dk, dv, db = evo_attention_backward(d_o, q, k, v, res_mask, pair_bias, o, lse, dbias_ready=ready)
    if pair_bias.shape[0] != q.shape[0] or pair_bias.dtype not in (torch.float32, q.dtype):
        side.wait_stream(cur)        # dBias was post-processed on the current stream (batch broadcast / dtype change)
    else:
        side.wait_event(ready)
    with torch.cuda.stream(side):
        db.record_stream(side)
        dist.all_reduce(db, op=dist.ReduceOp.SUM, group=group)
    cur.wait_stream(side)
    return dq, dk, dv, db


_side_streams = {}


def _side_stream(dev):
    s = _side_streams.get(dev)
    if s is None:
        s = _side_streams[dev] = torch.cuda.Stream(dev)
    return s


class ShardedEvoformerAttention(torch.autograd.Function):
    """``EvoformerAttention`` on this rank's rows; the gradient of the replicated ``pair_bias`` comes back summed over the
    group, the collective hidden behind the dQ / dK / dV kernels (see ``evo_attention_backward_sharded``)."""

    @staticmethod
    def forward(ctx, Q, K, V, res_mask, pair_bias, group=None):
        from .evoattention import evo_attention_forward
        o, lse = evo_attention_forward(Q, K, V, res_mask, pair_bias)
        ctx.save_for_backward(Q, K, V, res_mask, pair_bias, o, lse)
        ctx.group = group
        return o

    @staticmethod
    def backward(ctx, dO):
        Q, K, V, res_mask, pair_bias, o, lse = ctx.saved_tensors
        dq, dk, dv, d_bias = evo_attention_backward_sharded(dO.contiguous(), Q, K, V, res_mask, pair_bias, o, lse, ctx.group)
        return dq, dk, dv, None, d_bias, None


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
        return ShardedEvoformerAttention.apply(q, k, v, res_mask, pair_bias, group)
    return attention(q, k, v, res_mask, AllReduceGradient.apply(pair_bias, group))
