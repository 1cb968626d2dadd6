"""SwiGLU and the fused Transition block with the module interface of the reference.

Mirrors megafold/model/FusedTransition/fused_transition.py: ``FusedSwiGLUFunction`` / ``FusedSwiGLU``
(:96-116) and ``FusedTransition`` (:118-151).  ``FusedTransition`` keeps the reference's ``ff``
``nn.Sequential`` so that ``state_dict`` keys are unchanged (``ff.0.WEIGHT``, ``ff.0.BIAS``,
``ff.0.linear_weight``, ``ff.2.weight``), but its forward runs LN -> Linear -> SwiGLU -> Linear as one
operator (``mf_transition_fwd`` / ``mf_transition_bwd``) that does not keep the hidden activations:
backward recomputes them from ``x``.  SwiGLU backward writes to a new buffer (the reference
overwrites its saved input, :49-52).
"""
from __future__ import annotations

import ctypes as C

import torch
from torch import nn

from . import _lib
from .fused_layernorm_linear import LayernormLinear

__all__ = ["FusedSwiGLUFunction", "FusedSwiGLU", "FusedTransition", "TransitionFunction",
           "transition_forward", "transition_backward"]


class FusedSwiGLUFunction(torch.autograd.Function):
    @staticmethod
    @torch.amp.custom_fwd(device_type="cuda", cast_inputs=torch.bfloat16)
    def forward(ctx, input):
        _lib.require_cuda(input)
        two_i = input.shape[-1]
        if two_i % 2:
            raise ValueError("SwiGLU needs an even last dimension")
        inner = two_i // 2
        x = input.reshape(-1, two_i).contiguous()
        y = torch.empty((x.shape[0], inner), dtype=x.dtype, device=x.device)
        with torch.cuda.device(x.device):
            _lib.check(_lib.lib().mf_swiglu_fwd(x.data_ptr(), y.data_ptr(), x.shape[0], inner,
                                                _lib.dtype_code(x.dtype), _lib.stream_ptr(x.device)), "mf_swiglu_fwd")
        ctx.save_for_backward(x)
        ctx.in_shape = input.shape
        return y.view(*input.shape[:-1], inner)

    @staticmethod
    @torch.amp.custom_bwd(device_type="cuda")
    def backward(ctx, grad_output):
        (x,) = ctx.saved_tensors
        inner = x.shape[1] // 2
        dy = grad_output.reshape(-1, inner).to(x.dtype).contiguous()
        dx = torch.empty_like(x)
        with torch.cuda.device(x.device):
            _lib.check(_lib.lib().mf_swiglu_bwd(x.data_ptr(), dy.data_ptr(), dx.data_ptr(), x.shape[0], inner,
                                                _lib.dtype_code(x.dtype), _lib.stream_ptr(x.device)), "mf_swiglu_bwd")
        return dx.view(ctx.in_shape)


class FusedSwiGLU(nn.Module):
    def forward(self, x):
        return FusedSwiGLUFunction.apply(x)


def transition_forward(x, ln_weight, ln_bias, w1, w2, eps: float = 1e-5, flags: int = 0):
    """``w1`` [dim, 2*inner], ``w2`` [dim, inner].  Returns ``(y, mean, rstd)``."""
    _lib.require_cuda(x, ln_weight, ln_bias, w1, w2)
    dim = x.shape[-1]
    inner = w2.shape[1]
    if tuple(w1.shape) != (dim, 2 * inner) or w2.shape[0] != dim:
        raise ValueError(f"weight shapes {tuple(w1.shape)} / {tuple(w2.shape)} do not fit dim={dim}")
    x2 = x.reshape(-1, dim).contiguous()
    M, dt, dev = x2.shape[0], x2.dtype, x.device
    w1c, w2c = w1.to(dt).contiguous(), w2.to(dt).contiguous()
    lw = None if ln_weight is None else ln_weight.to(dt).contiguous()
    lb = None if ln_bias is None else ln_bias.to(dt).contiguous()
    y = torch.empty((M, dim), dtype=dt, device=dev)
    mean = torch.empty((M,), dtype=torch.float32, device=dev)
    rstd = torch.empty((M,), dtype=torch.float32, device=dev)
    a = _lib.TransitionFwdArgs()
    a.M, a.dim, a.inner, a.dtype, a.flags, a.eps = M, dim, inner, _lib.dtype_code(dt), flags, eps
    a.x, a.ln_w, a.ln_b, a.w1, a.w2 = x2.data_ptr(), _lib.ptr(lw), _lib.ptr(lb), w1c.data_ptr(), w2c.data_ptr()
    a.y, a.mean, a.rstd = y.data_ptr(), mean.data_ptr(), rstd.data_ptr()
    L_ = _lib.lib()
    with torch.cuda.device(dev):
        ws = _lib.workspace(L_.mf_transition_fwd_workspace_bytes(C.byref(a)), dev)
        a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
        _lib.check(L_.mf_transition_fwd(C.byref(a), _lib.stream_ptr(dev)), "mf_transition_fwd")
    return y.view(x.shape), mean, rstd


def transition_backward(dy, x, ln_weight, ln_bias, w1, w2, mean, rstd, flags: int = 0):
    """Returns ``(dx, d_ln_weight, d_ln_bias, dw1, dw2)``; parameter gradients fp32."""
    dim = x.shape[-1]
    inner = w2.shape[1]
    x2 = x.reshape(-1, dim).contiguous()
    M, dt, dev = x2.shape[0], x2.dtype, x.device
    dy2 = dy.reshape(-1, dim).to(dt).contiguous()
    w1c, w2c = w1.to(dt).contiguous(), w2.to(dt).contiguous()
    lw = None if ln_weight is None else ln_weight.to(dt).contiguous()
    lb = None if ln_bias is None else ln_bias.to(dt).contiguous()
    dx = torch.empty_like(x2)
    dw1 = torch.empty((dim, 2 * inner), dtype=torch.float32, device=dev)
    dw2 = torch.empty((dim, inner), dtype=torch.float32, device=dev)
    dlw = torch.empty((dim,), dtype=torch.float32, device=dev) if lw is not None else None
    dlb = torch.empty((dim,), dtype=torch.float32, device=dev) if lb is not None else None
    a = _lib.TransitionBwdArgs()
    a.M, a.dim, a.inner, a.dtype, a.flags = M, dim, inner, _lib.dtype_code(dt), flags
    a.x, a.ln_w, a.ln_b, a.w1, a.w2, a.dy = (x2.data_ptr(), _lib.ptr(lw), _lib.ptr(lb), w1c.data_ptr(),
                                             w2c.data_ptr(), dy2.data_ptr())
    a.mean, a.rstd = mean.data_ptr(), rstd.data_ptr()
    a.dx, a.dw1, a.dw2, a.d_ln_w, a.d_ln_b = dx.data_ptr(), dw1.data_ptr(), dw2.data_ptr(), _lib.ptr(dlw), _lib.ptr(dlb)
    L_ = _lib.lib()
    with torch.cuda.device(dev):
        ws = _lib.workspace(L_.mf_transition_bwd_workspace_bytes(C.byref(a)), dev)
        a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
        _lib.check(L_.mf_transition_bwd(C.byref(a), _lib.stream_ptr(dev)), "mf_transition_bwd")
    return dx.view(x.shape), dlw, dlb, dw1, dw2


class TransitionFunction(torch.autograd.Function):
    """``apply(x, ln_weight | None, ln_bias | None, w1 [dim, 2*inner], w2 [dim, inner])``."""

    @staticmethod
    @torch.amp.custom_fwd(device_type="cuda", cast_inputs=torch.bfloat16)
    def forward(ctx, x, ln_weight, ln_bias, w1, w2):
        y, mean, rstd = transition_forward(x, ln_weight, ln_bias, w1, w2)
        ctx.save_for_backward(x, ln_weight, ln_bias, w1, w2, mean, rstd)
        return y

    @staticmethod
    @torch.amp.custom_bwd(device_type="cuda")
    def backward(ctx, dy):
        x, ln_weight, ln_bias, w1, w2, mean, rstd = ctx.saved_tensors
        dx, dlw, dlb, dw1, dw2 = transition_backward(dy, x, ln_weight, ln_bias, w1, w2, mean, rstd)
        return (dx, None if dlw is None else dlw.to(ln_weight.dtype), None if dlb is None else dlb.to(ln_bias.dtype),
                dw1.to(w1.dtype), dw2.to(w2.dtype))


class FusedTransition(nn.Module):
    def __init__(self, dim, expansion_factor=4, include_ln=True, use_layernormlinear=True, device=None, dtype=None):
        factory_kwargs = {"device": device, "dtype": dtype}
        super().__init__()
        self.dim = dim
        dim_inner = int(dim * expansion_factor)
        self.dim_inner = dim_inner
        self.include_ln = include_ln
        self.use_layernormlinear = use_layernormlinear
        if include_ln:
            if use_layernormlinear:
                self.ff = nn.Sequential(
                    LayernormLinear(dim, dim_inner * 2, has_linear_bias=False, **factory_kwargs),
                    FusedSwiGLU(),
                    nn.Linear(dim_inner, dim, bias=False, **factory_kwargs),
                )
            else:
                self.ff = nn.Sequential(
                    nn.LayerNorm(dim, **factory_kwargs),
                    nn.Linear(dim, dim_inner * 2, bias=False, **factory_kwargs),
                    FusedSwiGLU(),
                    nn.Linear(dim_inner, dim, bias=False, **factory_kwargs),
                )
        else:
            self.ff = nn.Sequential(
                nn.Linear(dim, dim_inner * 2, bias=False, **factory_kwargs),
                FusedSwiGLU(),
                nn.Linear(dim_inner, dim, bias=False, **factory_kwargs),
            )

    def forward(self, input):
        if self.include_ln and self.use_layernormlinear:
            lnl = self.ff[0]
            return TransitionFunction.apply(input, lnl.WEIGHT, lnl.BIAS, lnl.linear_weight, self.ff[2].weight)
        if self.include_ln:
            ln, lin = self.ff[0], self.ff[1]
            return TransitionFunction.apply(input, ln.weight, ln.bias, lin.weight.t(), self.ff[3].weight)
        return TransitionFunction.apply(input, None, None, self.ff[0].weight.t(), self.ff[2].weight)

    def extra_repr(self):
        return f"dim={self.dim}, dim_inner={self.dim_inner}"
