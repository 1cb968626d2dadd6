"""Row-sharded Pairformer block built from the fused operators (the long-crop benchmark configuration).

Composition (one block, no dropout): pair += TriangleAttention(starting node); pair += TriangleAttention(ending
node); pair += Transition; single += AttentionPairBias.  It follows the modules that call the fused operators in
the reference - ``TriangleAttention`` (megafold/model/megafold.py:635-648), ``Attention.forward``
(megafold/model/attention.py:158-210: q with bias, k, v, sigmoid output gate, bias-free output projection),
``Transition`` (megafold.py:723) - with the four input projections of an attention merged into ONE
LayernormLinear (128 -> 4*128), which is what the fused operator is for.

Sharding: every rank holds a contiguous block of rows i of the pair representation ``[L, L, C]`` and a replica of
the single representation.  Row-wise operators (LayernormLinear, Transition, starting-node attention) need no
communication except for the pair bias, which is projected from the local rows and all-gathered (its gradient
comes back all-reduced, see ``sharded.AllReduceGradient``).  The ending-node attention is the same operator on the
transposed pair representation, reached by a block transpose between ranks (all-to-all) before and after.  The
single-track attention (N = 1, small) is computed on every rank from the gathered pair bias.

The operators are injectable (``ops``) so that the communication and autograd plumbing can be exercised on CPU
ranks with reference implementations; the default is the CUDA library.
"""
from __future__ import annotations

import math
from types import SimpleNamespace

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

from .sharded import AllReduceGradient, row_shard

__all__ = ["PairformerBlock", "GatherRows", "TransposeShards", "cuda_ops"]


def _world(group):
    return dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1


def _rank(group):
    return dist.get_rank(group) if dist.is_available() and dist.is_initialized() else 0


class GatherRows(torch.autograd.Function):
    """All-gather of row blocks ``[n_local, ...] -> [n_total, ...]`` (blocks as ``row_shard`` assigns them).

    Backward returns this rank's rows of the incoming gradient WITHOUT summing over ranks: the consumer must hand
    back the complete gradient on every rank (true for a pair bias behind ``AllReduceGradient`` and for anything
    computed identically on all ranks)."""

    @staticmethod
    def forward(ctx, x, n_total, group=None):
        world, rank = _world(group), _rank(group)
        ctx.span = row_shard(n_total, rank, world)
        if world == 1:
            return x.contiguous()
        most = row_shard(n_total, 0, world)
        most = most[1] - most[0]
        pad = x.new_zeros((most,) + tuple(x.shape[1:]))
        pad[: x.shape[0]] = x
        parts = [torch.empty_like(pad) for _ in range(world)]
        dist.all_gather(parts, pad, group=group)
        sizes = [row_shard(n_total, r, world) for r in range(world)]
        return torch.cat([p[: b - a] for p, (a, b) in zip(parts, sizes)], dim=0)

    @staticmethod
    def backward(ctx, g):
        a, b = ctx.span
        return g[a:b].contiguous(), None, None


def _exchange(send, recv, group):
    """send[r] goes to rank r, recv[r] arrives from rank r (sizes may differ between peers)."""
    world, rank = _world(group), _rank(group)
    recv[rank].copy_(send[rank])
    if world == 1:
        return
    if dist.get_backend(group) == "nccl":
        dist.all_to_all(recv, send, group=group)
        return
    ops = []
    for r in range(world):
        if r != rank:
            peer = dist.get_global_rank(group, r) if group is not None else r
            ops.append(dist.P2POp(dist.isend, send[r], peer, group))
            ops.append(dist.P2POp(dist.irecv, recv[r], peer, group))
    for w in dist.batch_isend_irecv(ops):
        w.wait()


class TransposeShards(torch.autograd.Function):
    """Block transpose of a row-sharded square matrix of vectors: in ``x[i_local, j, c]`` (my rows i, all j), out
    ``y[j_local, i, c] = x_global[i, j_local, c]`` (my rows j of the transposed matrix, all i).  It is its own
    inverse, hence also its own backward."""

    @staticmethod
    def forward(ctx, x, group=None):
        ctx.group = group
        return TransposeShards._run(x, group)

    @staticmethod
    def backward(ctx, g):
        return TransposeShards._run(g, ctx.group), None

    @staticmethod
    def _run(x, group):
        world, rank = _world(group), _rank(group)
        if world == 1:
            return x.transpose(0, 1).contiguous()
        n = x.shape[1]
        if n % world == 0 and dist.get_backend(group) == "nccl":
            # equal shards: one packing copy, one all-to-all on a single buffer, one transposing copy
            mine = n // world
            send = x.view(mine, world, mine, *x.shape[2:]).transpose(0, 1).contiguous()      # [their rank, my i, their j]
            recv = torch.empty_like(send)                                                    # [their rank, their i, my j]
            dist.all_to_all_single(recv, send, group=group)
            return recv.permute(2, 0, 1, *range(3, recv.dim())).reshape(mine, n, *x.shape[2:]).contiguous()
        spans = [row_shard(n, r, world) for r in range(world)]
        mine = spans[rank][1] - spans[rank][0]
        send = [x[:, a:b].contiguous() for a, b in spans]                       # [my i, their j]
        recv = [x.new_empty((b - a, mine) + tuple(x.shape[2:])) for a, b in spans]   # [their i, my j]
        _exchange(send, recv, group)
        return torch.cat(recv, dim=0).transpose(0, 1).contiguous()              # [my j, all i]


def cuda_ops():
    """The fused CUDA operators behind the three call sites of the block."""
    from .evoattention import TritonEvoformer
    from .fused_layernorm_linear import LayernormLinearFunction
    from .fused_transition import TransitionFunction

    def lnl(x, ln_w, ln_b, w, b):
        return LayernormLinearFunction.apply(x, w, b, ln_w, ln_b, ln_b is not None, b is not None)

    return SimpleNamespace(lnl=lnl, attention=TritonEvoformer, transition=TransitionFunction.apply)


class _Attn(nn.Module):
    """Parameters of one gated attention with pair bias: merged q/k/v/gate projection behind a LayerNorm, pair-bias
    projection behind its own LayerNorm, output projection."""

    def __init__(self, dim, heads, dim_head, dim_pair, device=None, dtype=None):
        super().__init__()
        kw = dict(device=device, dtype=dtype)
        inner = heads * dim_head
        self.heads, self.dim_head, self.inner = heads, dim_head, inner
        self.ln_w = nn.Parameter(torch.ones(dim, **kw))
        self.ln_b = nn.Parameter(torch.zeros(dim, **kw))
        self.w_qkvg = nn.Parameter(torch.randn(dim, 4 * inner, **kw) / math.sqrt(dim))
        bias = torch.zeros(4 * inner, **kw)
        bias[3 * inner:] = -2.0                    # gate bias as in attention.py:153 (init_gate_bias)
        self.b_qkvg = nn.Parameter(bias)
        self.pair_ln_w = nn.Parameter(torch.ones(dim_pair, **kw))
        self.pair_ln_b = nn.Parameter(torch.zeros(dim_pair, **kw))
        # the projection is padded to a multiple of 8 output columns (16-byte rows: the tensor-core kernels take it);
        # the extra columns are never used and receive zero gradients
        self.w_pair_bias = nn.Parameter(torch.randn(dim_pair, (heads + 7) // 8 * 8, **kw) / math.sqrt(dim_pair))
        self.w_out = nn.Parameter(torch.randn(dim, inner, **kw) / math.sqrt(inner))


class PairformerBlock(nn.Module):
    def __init__(self, dim_pair=128, dim_single=384, tri_heads=4, tri_dim_head=32, single_heads=16, single_dim_head=24,
                 expansion=4, group=None, ops=None, device=None, dtype=None):
        super().__init__()
        kw = dict(device=device, dtype=dtype)
        self.group, self.ops = group, ops
        self.tri_start = _Attn(dim_pair, tri_heads, tri_dim_head, dim_pair, **kw)
        self.tri_end = _Attn(dim_pair, tri_heads, tri_dim_head, dim_pair, **kw)
        self.single_attn = _Attn(dim_single, single_heads, single_dim_head, dim_pair, **kw)
        inner = dim_pair * expansion
        self.tr_ln_w = nn.Parameter(torch.ones(dim_pair, **kw))
        self.tr_ln_b = nn.Parameter(torch.zeros(dim_pair, **kw))
        self.tr_w1 = nn.Parameter(torch.randn(dim_pair, 2 * inner, **kw) / math.sqrt(dim_pair))
        self.tr_w2 = nn.Parameter(torch.randn(dim_pair, inner, **kw) / math.sqrt(inner))

    # ---- pieces ------------------------------------------------------------------------------------
    def _pair_bias(self, a: _Attn, pair_rows, n_total, reduce_grad):
        """[1, 1, H, L, L] bias projected from the local pair rows and gathered over the ranks."""
        n_loc, L, C = pair_rows.shape
        rows = self.ops.lnl(pair_rows.reshape(-1, C), a.pair_ln_w, a.pair_ln_b, a.w_pair_bias, None)
        full = GatherRows.apply(rows.view(n_loc, L, -1)[..., : a.heads], n_total, self.group)   # [L, L, H]
        bias = full.permute(2, 0, 1)[None, None].contiguous()
        return AllReduceGradient.apply(bias, self.group) if reduce_grad else bias

    def _attention(self, a: _Attn, x, mask, bias):
        """x [n, L, dim] -> [n, L, dim]; one attention row per leading index, keys masked by ``mask`` [L]."""
        n, L, C = x.shape
        y = self.ops.lnl(x.reshape(-1, C), a.ln_w, a.ln_b, a.w_qkvg, a.b_qkvg).view(1, n, L, 4, a.heads, a.dim_head)
        q, k, v, g = y.unbind(dim=3)                                # strided views, no copies
        res_mask = mask.view(1, 1, 1, 1, L).expand(1, n, 1, 1, L)
        o = self.ops.attention(q, k, v, res_mask, bias)             # [1, n, L, H, D]
        o = (o * torch.sigmoid(g)).reshape(n, L, a.inner)            # the gate is read through its strided view: no packing copy
        return F.linear(o, a.w_out)

    # ---- block -------------------------------------------------------------------------------------
    def forward(self, pair_rows, single, mask):
        """pair_rows [n_local, L, dim_pair] (this rank's rows), single [L, dim_single] (replicated), mask bool [L]."""
        if self.ops is None:
            self.ops = cuda_ops()
        L = pair_rows.shape[1]
        x = pair_rows
        x = x + self._attention(self.tri_start, x, mask, self._pair_bias(self.tri_start, x, L, True))
        xt = TransposeShards.apply(x, self.group)                   # rows j of the transposed pair representation
        yt = self._attention(self.tri_end, xt, mask, self._pair_bias(self.tri_end, xt, L, True))
        x = x + TransposeShards.apply(yt, self.group)
        x = x + self.ops.transition(x, self.tr_ln_w, self.tr_ln_b, self.tr_w1, self.tr_w2)
        s_bias = self._pair_bias(self.single_attn, x, L, False)     # identical on every rank: no gradient reduction
        s = single + self._attention(self.single_attn, single[None], mask, s_bias)[0]
        return x, s
