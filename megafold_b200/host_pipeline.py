"""Attention forward + backward for operands that live in HOST memory.

``evoformer_fwd_bwd_host`` is the call for a user whose q/k/v/dO sit in pinned host buffers (a data loader, an
off-loaded activation store): the N rows are independent in the forward pass and coupled only through the
sum that forms d_pair_bias, so the rows are cut into chunks that flow through three CUDA streams - upload of
chunk i+1, kernels of chunk i, download of chunk i-1 - and PCIe runs in both directions while the GPU computes.
The results land in pinned host tensors; d_pair_bias is accumulated on the device over the chunks.

A step issues a few hundred copies and launches, which costs the CPU more than the GPU work takes once the chunks
are small.  So the second call with the same host buffers records the whole three-stream schedule into a CUDA
graph and every later call replays it (one launch); a call with other buffers, or a failed capture, runs the
schedule directly.
"""
from __future__ import annotations

import warnings

import torch

from .evoattention import evo_attention_backward, evo_attention_forward

__all__ = ["evoformer_fwd_bwd_host", "HostPipeline"]


def _row_spans(n_rows, chunks):
    """Row chunks for the pipeline: about ``chunks`` full-size chunks in the middle, and short ones at both ends,
    because the first upload and the last compute + download are the only parts that nothing overlaps."""
    big = -(-n_rows // chunks)
    ramp = [r for r in (big // 8, big // 4, big // 2) if r >= 1] if n_rows >= 4 * chunks and big >= 8 else []
    left = n_rows - 2 * sum(ramp)
    n_mid = -(-left // big)
    mid = [left // n_mid + (1 if i < left % n_mid else 0) for i in range(n_mid)]
    sizes = ramp + mid + ramp[::-1]
    spans, s = [], 0
    for n in sizes:
        spans.append((s, s + n))
        s += n
    assert s == n_rows
    return spans


class HostPipeline:
    """Reusable state (streams, device staging buffers, pinned outputs) for one problem shape."""

    def __init__(self, shape, dtype, bias_shape, bias_dtype, device, chunks=4, mask_dtype=torch.bool):
        B, N, L, H, D = shape
        self.shape, self.dtype, self.device = tuple(shape), dtype, torch.device(device)
        self.spans = _row_spans(N, max(1, min(chunks, N)))
        self.chunks = len(self.spans)
        rows = max(e - s for s, e in self.spans)
        dev = self.device
        self.s_in, self.s_cmp, self.s_out = (torch.cuda.Stream(dev) for _ in range(3))
        mk = lambda: torch.empty((B, rows, L, H, D), dtype=dtype, device=dev)      # noqa: E731
        self.dev_in = [dict(q=mk(), k=mk(), v=mk(), d_out=mk(),
                            mask=torch.empty((B, rows, 1, 1, L), dtype=mask_dtype, device=dev)) for _ in range(2)]
        self.d_bias = torch.zeros(bias_shape, dtype=torch.float32, device=dev)
        self.bias = torch.empty(bias_shape, dtype=bias_dtype, device=dev)
        pin = lambda shp, dt: torch.empty(shp, dtype=dt, pin_memory=True)         # noqa: E731
        self.out = dict(o=pin(shape, dtype), dq=pin(shape, dtype), dk=pin(shape, dtype), dv=pin(shape, dtype),
                        d_bias=pin(bias_shape, bias_dtype))
        self.keep = []
        self.graph, self.graph_key, self.calls, self.use_graph, self.group = None, None, 0, True, None
        self.s_cap = torch.cuda.Stream(dev)

    def run(self, q, k, v, res_mask, pair_bias, d_out, group=None):
        """All arguments are pinned host tensors ([B,N,L,H,D], mask [B,N,1,1,L] bool, bias [B,1,H,L,L]).
        Returns the dict of pinned host results (valid after the call: it waits for the downloads).
        The returned tensors are this object's own buffers: the next call overwrites them.
        With ``group`` the tensors hold this rank's rows and d_pair_bias is all-reduced over the group on the device
        before it is downloaded (the collective is part of the replayed graph; every rank must call in step)."""
        host = dict(q=q, k=k, v=v, d_out=d_out, mask=res_mask, bias=pair_bias)
        self.group = group
        key = tuple(t.data_ptr() for t in host.values())
        cur = torch.cuda.current_stream(self.device)
        if self.graph is not None and key == self.graph_key:
            self.graph.replay()                      # on the current stream
            cur.synchronize()
            return self.out
        self.calls += 1
        if self.use_graph and self.calls >= 2 and all(t.is_pinned() for t in host.values()):
            try:
                self.s_cap.wait_stream(cur)
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=self.s_cap):
                    self._schedule(host, self.s_cap)
                self.graph, self.graph_key = g, key
                cur.wait_stream(self.s_cap)
            except Exception as e:                   # capture not possible here: keep the direct schedule
                warnings.warn(f"CUDA graph capture of the host pipeline failed ({type(e).__name__}: {e}); issuing the schedule directly")
                self.use_graph = False
                self.graph = None
                torch.cuda.synchronize(self.device)
            if group is not None:                    # every rank replays, or none does
                import torch.distributed as dist
                ok = torch.tensor([1 if self.graph is not None else 0], device=self.device)
                dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
                if not int(ok):
                    self.graph, self.use_graph = None, False
            if self.graph is not None:
                return self.run(q, k, v, res_mask, pair_bias, d_out, group)
        self._schedule(host, cur)
        cur.synchronize()
        return self.out

    def _schedule(self, host, cur):
        """Enqueue one step: the three streams fork from ``cur`` and join it again at the end."""
        self.s_in.wait_stream(cur)
        self.s_cmp.wait_stream(cur)
        self.s_out.wait_stream(cur)
        with torch.cuda.stream(self.s_in):
            self.bias.copy_(host["bias"], non_blocking=True)
        self.s_cmp.wait_stream(self.s_in)
        with torch.cuda.stream(self.s_cmp):
            self.d_bias.zero_()
        self.keep.clear()
        ev_free = [None, None]
        for i, (s, e) in enumerate(self.spans):
            slot = i & 1
            n = e - s
            buf = self.dev_in[slot]
            with torch.cuda.stream(self.s_in):
                if ev_free[slot] is not None:
                    self.s_in.wait_event(ev_free[slot])                 # kernels of chunk i-2 are done with this slot
                for name in ("q", "k", "v", "d_out", "mask"):
                    buf[name][:, :n].copy_(host[name][:, s:e], non_blocking=True)
                ev_in = torch.cuda.Event()
                ev_in.record(self.s_in)
            with torch.cuda.stream(self.s_cmp):
                self.s_cmp.wait_event(ev_in)
                qd, kd, vd, gd, md = (buf[x][:, :n] for x in ("q", "k", "v", "d_out", "mask"))
                o, lse = evo_attention_forward(qd, kd, vd, md, self.bias)
                dq, dk, dv, db = evo_attention_backward(gd, qd, kd, vd, md, self.bias, o, lse)
                self.d_bias.add_(db)
                done = torch.cuda.Event()
                done.record(self.s_cmp)
                ev_free[slot] = done
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(done)
                for name, t in (("o", o), ("dq", dq), ("dk", dk), ("dv", dv)):
                    self.out[name][:, s:e].copy_(t, non_blocking=True)
            self.keep.append((o, dq, dk, dv, db, lse))                  # keep alive until the copies have run
        if self.group is not None:
            import torch.distributed as dist
            with torch.cuda.stream(self.s_cmp):
                dist.all_reduce(self.d_bias, group=self.group)
        with torch.cuda.stream(self.s_out):
            self.s_out.wait_stream(self.s_cmp)
            self.out["d_bias"].copy_(self.d_bias, non_blocking=True)
        cur.wait_stream(self.s_in)
        cur.wait_stream(self.s_cmp)
        cur.wait_stream(self.s_out)


_cache = {}


def evoformer_fwd_bwd_host(q, k, v, res_mask, pair_bias, d_out, device="cuda", chunks=4, group=None):
    """Forward and backward of the pair-biased attention with pinned HOST operands and results.

    Returns ``dict(o, dq, dk, dv, d_bias)`` of pinned host tensors (buffers owned by the pipeline: the next call with
    the same shapes overwrites them); d_bias has ``pair_bias``'s dtype.  ``group``: a
    process group over which the rows are sharded (each rank passes its own rows; d_bias comes back summed)."""
    for t in (q, k, v, d_out, res_mask, pair_bias):
        if t.is_cuda:
            raise ValueError("evoformer_fwd_bwd_host takes host tensors; use TritonEvoformer for device tensors")
    dev = torch.device(device)
    if dev.index is None:
        dev = torch.device("cuda", torch.cuda.current_device())
    if res_mask.dtype not in (torch.bool, torch.uint8) and not res_mask.is_floating_point():
        raise TypeError(f"res_mask must be bool / uint8 (keep-mask) or floating (additive), got {res_mask.dtype}")
    key = (tuple(q.shape), q.dtype, tuple(pair_bias.shape), pair_bias.dtype, dev, chunks, res_mask.dtype)
    pipe = _cache.get(key)
    if pipe is None:
        _cache.clear()
        pipe = _cache[key] = HostPipeline(q.shape, q.dtype, pair_bias.shape, pair_bias.dtype, dev, chunks, res_mask.dtype)
    return pipe.run(q, k, v, res_mask, pair_bias, d_out, group)
