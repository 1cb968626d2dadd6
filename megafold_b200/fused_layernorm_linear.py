"""LayerNorm fused into a linear layer, with the module and function interface of the reference.

Mirrors megafold/model/FusedLayernormLinear/fused_layernorm_linear.py: ``LayernormLinear`` (:498-545,
parameters ``WEIGHT[K]``, ``BIAS[K]``, ``linear_weight[K, N]``, ``linear_bias[N]``) and
``LayernormLinearFunction`` (:477-495).  Unlike the reference there is no shape table and no
fallback to torch (:538-541): every shape goes to the CUDA library (``mf_lnl_fwd`` / ``mf_lnl_bwd``).
Row statistics are kept in fp32 (the reference stores them in the input dtype, :361-362).
"""
from __future__ import annotations

import ctypes as C
import math

import torch
from torch import nn

from . import _lib

__all__ = ["LayernormLinear", "LayernormLinearFunction", "layernorm_linear_forward", "layernorm_linear_backward"]


def layernorm_linear_forward(x, linear_weight, linear_bias, ln_weight, ln_bias, eps: float = 1e-5, flags: int = 0):
    """Returns ``(y [..., N], mean fp32 [M], rstd fp32 [M])``."""
    _lib.require_cuda(x, linear_weight, linear_bias, ln_weight, ln_bias)
    K = x.shape[-1]
    if linear_weight.shape[0] != K:
        raise ValueError("Incompatible dimensions")
    N = linear_weight.shape[1]
    x2 = x.reshape(-1, K).contiguous()
    M = x2.shape[0]
    dt = x2.dtype
    w = linear_weight.to(dt).contiguous()
    lw = ln_weight.to(dt).contiguous()
    lb = None if ln_bias is None else ln_bias.to(dt).contiguous()
    b = None if linear_bias is None else linear_bias.to(dt).contiguous()
    y = torch.empty((M, N), dtype=dt, device=x.device)
    mean = torch.empty((M,), dtype=torch.float32, device=x.device)
    rstd = torch.empty((M,), dtype=torch.float32, device=x.device)
    a = _lib.LnlFwdArgs()
    a.M, a.K, a.N, a.dtype, a.flags, a.eps = M, K, N, _lib.dtype_code(dt), flags, eps
    a.x, a.ln_w, a.ln_b, a.w, a.b = x2.data_ptr(), lw.data_ptr(), _lib.ptr(lb), w.data_ptr(), _lib.ptr(b)
    a.y, a.mean, a.rstd = y.data_ptr(), mean.data_ptr(), rstd.data_ptr()
    with torch.cuda.device(x.device):
        _lib.check(_lib.lib().mf_lnl_fwd(C.byref(a), _lib.stream_ptr(x.device)), "mf_lnl_fwd")
    return y.view(*x.shape[:-1], N), mean, rstd


def layernorm_linear_backward(dy, x, linear_weight, ln_weight, ln_bias, mean, rstd, has_linear_bias, flags: int = 0):
    """Returns ``(dx, d_linear_weight, d_linear_bias, d_ln_weight, d_ln_bias)``; parameter gradients fp32."""
    K = x.shape[-1]
    N = linear_weight.shape[1]
    x2 = x.reshape(-1, K).contiguous()
    M = x2.shape[0]
    dt = x2.dtype
    dy2 = dy.reshape(-1, N).to(dt).contiguous()
    w = linear_weight.to(dt).contiguous()
    lw = ln_weight.to(dt).contiguous()
    lb = None if ln_bias is None else ln_bias.to(dt).contiguous()
    dev = x.device
    dx = torch.empty_like(x2)
    dw = torch.empty((K, N), dtype=torch.float32, device=dev)
    dlw = torch.empty((K,), dtype=torch.float32, device=dev)
    dlb = torch.empty((K,), dtype=torch.float32, device=dev) if ln_bias is not None else None
    db = torch.empty((N,), dtype=torch.float32, device=dev) if has_linear_bias else None
    a = _lib.LnlBwdArgs()
    a.M, a.K, a.N, a.dtype, a.flags = M, K, N, _lib.dtype_code(dt), flags
    a.x, a.ln_w, a.ln_b, a.w, a.dy = x2.data_ptr(), lw.data_ptr(), _lib.ptr(lb), w.data_ptr(), dy2.data_ptr()
    a.mean, a.rstd = mean.data_ptr(), rstd.data_ptr()
    a.dx, a.dw, a.db, a.d_ln_w, a.d_ln_b = dx.data_ptr(), dw.data_ptr(), _lib.ptr(db), dlw.data_ptr(), _lib.ptr(dlb)
    L_ = _lib.lib()
    with torch.cuda.device(dev):
        ws = _lib.workspace(L_.mf_lnl_bwd_workspace_bytes(C.byref(a)), dev)
        a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
        _lib.check(L_.mf_lnl_bwd(C.byref(a), _lib.stream_ptr(dev)), "mf_lnl_bwd")
    return dx.view(x.shape), dw, db, dlw, dlb


class LayernormLinearFunction(torch.autograd.Function):
    """``apply(X, linear_weight, linear_bias, WEIGHT, BIAS, has_layernorm_bias, has_linear_bias,
    supported_configs)``; the last argument (the reference's Triton tile configs) is ignored."""

    @staticmethod
    @torch.amp.custom_fwd(device_type="cuda", cast_inputs=torch.bfloat16)
    def forward(ctx, X, linear_weight, linear_bias, WEIGHT, BIAS, has_layernorm_bias=True, has_linear_bias=False,
                supported_configs=None):
        ln_b = BIAS if has_layernorm_bias else None
        lin_b = linear_bias if has_linear_bias else None
        y, mean, rstd = layernorm_linear_forward(X, linear_weight, lin_b, WEIGHT, ln_b)
        ctx.save_for_backward(X, linear_weight, mean, rstd, WEIGHT, ln_b)
        ctx.has_linear_bias = lin_b is not None
        ctx.dtypes = (linear_weight.dtype, None if lin_b is None else lin_b.dtype, WEIGHT.dtype,
                      None if ln_b is None else ln_b.dtype)
        return y

    @staticmethod
    @torch.amp.custom_bwd(device_type="cuda")
    def backward(ctx, dOUT):
        X, linear_weight, mean, rstd, WEIGHT, ln_b = ctx.saved_tensors
        dx, dw, db, dlw, dlb = layernorm_linear_backward(dOUT, X, linear_weight, WEIGHT, ln_b, mean, rstd,
                                                         ctx.has_linear_bias)
        wd, bd, lwd, lbd = ctx.dtypes
        return (dx, dw.to(wd), None if db is None else db.to(bd), dlw.to(lwd),
                None if dlb is None else dlb.to(lbd), None, None, None)


class LayernormLinear(nn.Module):
    """``LayerNorm(K)`` followed by ``Linear(K -> N)`` with the weight stored ``[K, N]``."""

    def __init__(self, K, N, has_layernorm_bias=True, has_linear_bias=True, device=None, dtype=None):
        factory_kwargs = {"device": device, "dtype": dtype}
        super().__init__()
        self.K, self.N = K, N
        self.has_layernorm_bias = has_layernorm_bias
        self.has_linear_bias = has_linear_bias
        self.WEIGHT = nn.Parameter(torch.empty(K, **factory_kwargs))
        self.BIAS = nn.Parameter(torch.empty(K, **factory_kwargs)) if has_layernorm_bias else None
        self.linear_weight = nn.Parameter(torch.empty((K, N), **factory_kwargs))
        self.linear_bias = nn.Parameter(torch.empty((N,), **factory_kwargs)) if has_linear_bias else None
        self.reset_parameters()

    def reset_parameters(self) -> None:
        # same distributions as nn.LayerNorm + nn.Linear (Kaiming-uniform on the [N, K] view)
        nn.init.ones_(self.WEIGHT)
        if self.BIAS is not None:
            nn.init.zeros_(self.BIAS)
        with torch.no_grad():
            as_linear = torch.empty((self.N, self.K), device=self.linear_weight.device, dtype=self.linear_weight.dtype)
            nn.init.kaiming_uniform_(as_linear, a=math.sqrt(5))
            self.linear_weight.copy_(as_linear.T)
        if self.linear_bias is not None:
            bound = 1 / math.sqrt(self.K) if self.K > 0 else 0
            nn.init.uniform_(self.linear_bias, -bound, bound)

    def forward(self, X):
        return LayernormLinearFunction.apply(X, self.linear_weight, self.linear_bias, self.WEIGHT, self.BIAS,
                                             self.has_layernorm_bias, self.has_linear_bias, None)

    def extra_repr(self):
        return f"K={self.K}, N={self.N}, has_linear_bias={self.has_linear_bias}"
