"""Parity of LayernormLinear, SwiGLU and Transition (through the C ABI) with the oracle and golden vectors."""
import os

import numpy as np
import pytest
import torch

import cases
import megafold_b200 as mfb
from megafold_b200 import _lib
from oracle import pairformer_oracle as orc
from util import assert_close_fp32, assert_close_lowp

# gradients that are sums over the M rows: their absolute floor grows like sqrt(M) (see util.assert_close_lowp)
SUMMED = {"dw", "db", "d_ln_w", "d_ln_b", "dw1", "dw2"}


def lowp(g_, r_, n, M):
    assert_close_lowp(g_, r_, n, summed_over=M if n.split()[0] in SUMMED else 1)

pytestmark = pytest.mark.gpu
G = os.path.join(os.path.dirname(__file__), "golden")
DEV = "cuda"


def run_lnl(x, ln_w, ln_b, w, b, dy, dtype):
    mod = mfb.LayernormLinear(w.shape[0], w.shape[1], has_layernorm_bias=ln_b is not None,
                              has_linear_bias=b is not None, device=DEV, dtype=dtype)
    with torch.no_grad():
        mod.WEIGHT.copy_(ln_w); mod.linear_weight.copy_(w)
        if ln_b is not None: mod.BIAS.copy_(ln_b)
        if b is not None: mod.linear_bias.copy_(b)
    xg = x.to(DEV, dtype).requires_grad_(True)
    y = mod(xg)
    y.backward(dy.to(DEV, dtype))
    torch.cuda.synchronize()
    return (y, xg.grad, mod.WEIGHT.grad, None if ln_b is None else mod.BIAS.grad, mod.linear_weight.grad,
            None if b is None else mod.linear_bias.grad)


LNL_NAMES = ("y", "dx", "d_ln_w", "d_ln_b", "dw", "db")


def test_lnl_matches_reference_vectors_fp32():
    g = np.load(os.path.join(G, "lnl.npz"))
    for i, _ in enumerate(cases.LNL_SHAPES):
        t = lambda n: torch.from_numpy(g[f"c{i}_{n}"])      # noqa: E731
        got = run_lnl(t("x"), t("ln_w"), t("ln_b"), t("w"), t("b"), t("dy"), torch.float32)
        for g_, n in zip(got, LNL_NAMES):
            assert_close_fp32(g_, t(n), f"case {i} {n}")


def _lnl_case(M, N, K, seed=42):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g) * 1.5 + 0.3
    ln_w = 1 + 0.1 * torch.randn(K, generator=g)
    ln_b = 0.1 * torch.randn(K, generator=g)
    w = torch.randn(K, N, generator=g) / K ** 0.5
    b = 0.1 * torch.randn(N, generator=g)
    dy = torch.randn(M, N, generator=g)
    return x, ln_w, ln_b, w, b, dy


@pytest.mark.parametrize("M,N,K", [(18, 31, 99), (1879, 18, 666), (300, 512, 128), (1000, 16, 128), (64, 3, 128),
                                   (513, 128, 64), (2, 1, 5)])
def test_lnl_ragged_fp32(M, N, K):
    x, ln_w, ln_b, w, b, dy = _lnl_case(M, N, K)
    got = run_lnl(x, ln_w, ln_b, w, b, dy, torch.float32)
    ref = orc.layernorm_linear_fwd_bwd(x, ln_w, ln_b, w, b, dy)
    y, dx, dlw, dlb, dw, db = ref
    for g_, r_, n in zip(got, (y, dx, dlw, dlb, dw, db), LNL_NAMES):
        assert_close_fp32(g_, r_, n)


def test_lnl_without_biases_fp32():
    x, ln_w, _, w, _, dy = _lnl_case(200, 48, 96)
    got = run_lnl(x, ln_w, None, w, None, dy, torch.float32)
    y, dx, dlw, _, dw, _ = orc.layernorm_linear_fwd_bwd(x, ln_w, None, w, None, dy)
    for g_, r_, n in zip((got[0], got[1], got[2], got[4]), (y, dx, dlw, dw), ("y", "dx", "d_ln_w", "dw")):
        assert_close_fp32(g_, r_, n)


@pytest.mark.parametrize("M,N,K", [(4096, 512, 128), (3000, 16, 128), (1024, 1024, 128), (777, 384, 384)])
def test_lnl_bf16_against_fp32_oracle(M, N, K):
    x, ln_w, ln_b, w, b, dy = _lnl_case(M, N, K)
    got = run_lnl(x, ln_w, ln_b, w, b, dy, torch.bfloat16)
    r = [t.to(torch.bfloat16).float() for t in (x, ln_w, ln_b, w, b, dy)]
    ref = orc.layernorm_linear_fwd_bwd(*r)
    for g_, r_, n in zip(got, ref, LNL_NAMES):
        lowp(g_, r_, n, M)


def test_swiglu_fp32_and_bf16():
    g = torch.Generator().manual_seed(1)
    x = torch.randn(37, 2 * 24, generator=g)
    dy = torch.randn(37, 24, generator=g)
    for dtype, check in ((torch.float32, assert_close_fp32), (torch.bfloat16, assert_close_lowp)):
        xr = x.to(dtype).float().detach().clone().requires_grad_(True)
        orc.swiglu(xr).backward(dy.to(dtype).float())
        xg = x.detach().to(DEV, dtype).clone().requires_grad_(True)
        saved = xg.detach().clone()
        y = mfb.FusedSwiGLU()(xg)
        y.backward(dy.to(DEV, dtype))
        check(y, orc.swiglu(xr).detach(), "y")
        check(xg.grad, xr.grad, "dx")
        assert torch.equal(xg.detach(), saved)          # the input is not overwritten


def run_transition(x, ln_w, ln_b, w1, w2, dy, dtype, variant="lnl"):
    dim, inner = w2.shape
    kw = dict(device=DEV, dtype=dtype)
    if variant == "lnl":
        mod = mfb.FusedTransition(dim, inner / dim, **kw)
        with torch.no_grad():
            mod.ff[0].WEIGHT.copy_(ln_w); mod.ff[0].BIAS.copy_(ln_b); mod.ff[0].linear_weight.copy_(w1)
            mod.ff[2].weight.copy_(w2)
        params = lambda: (mod.ff[0].WEIGHT.grad, mod.ff[0].BIAS.grad, mod.ff[0].linear_weight.grad, mod.ff[2].weight.grad)  # noqa: E731
    elif variant == "ln+linear":
        mod = mfb.FusedTransition(dim, inner / dim, use_layernormlinear=False, **kw)
        with torch.no_grad():
            mod.ff[0].weight.copy_(ln_w); mod.ff[0].bias.copy_(ln_b); mod.ff[1].weight.copy_(w1.T)
            mod.ff[3].weight.copy_(w2)
        params = lambda: (mod.ff[0].weight.grad, mod.ff[0].bias.grad, mod.ff[1].weight.grad.T, mod.ff[3].weight.grad)  # noqa: E731
    else:
        mod = mfb.FusedTransition(dim, inner / dim, include_ln=False, **kw)
        with torch.no_grad():
            mod.ff[0].weight.copy_(w1.T); mod.ff[2].weight.copy_(w2)
        params = lambda: (None, None, mod.ff[0].weight.grad.T, mod.ff[2].weight.grad)  # noqa: E731
    xg = x.to(DEV, dtype).requires_grad_(True)
    y = mod(xg)
    y.backward(dy.to(DEV, dtype))
    torch.cuda.synchronize()
    return (y, xg.grad) + params()


T_NAMES = ("y", "dx", "d_ln_w", "d_ln_b", "dw1", "dw2")


def test_transition_matches_reference_vectors_fp32():
    g = np.load(os.path.join(G, "transition.npz"))
    for i, _ in enumerate(cases.TRANSITION_SHAPES):
        t = lambda n: torch.from_numpy(g[f"c{i}_{n}"])      # noqa: E731
        got = run_transition(t("x"), t("ln_w"), t("ln_b"), t("w1_lin").T.contiguous(), t("w2"), t("dy"), torch.float32)
        want = (t("y"), t("dx"), t("d_ln_w"), t("d_ln_b"), t("dw1_lin").T, t("dw2"))
        for g_, r_, n in zip(got, want, T_NAMES):
            assert_close_fp32(g_, r_, f"case {i} {n}")


def _transition_case(M, dim, ef, seed=42):
    g = torch.Generator().manual_seed(seed)
    inner = int(dim * ef)
    x = torch.randn(M, dim, generator=g)
    ln_w = 1 + 0.1 * torch.randn(dim, generator=g)
    ln_b = 0.1 * torch.randn(dim, generator=g)
    w1 = torch.randn(dim, 2 * inner, generator=g) / dim ** 0.5
    w2 = torch.randn(dim, inner, generator=g) / inner ** 0.5
    dy = torch.randn(M, dim, generator=g)
    return x, ln_w, ln_b, w1, w2, dy


@pytest.mark.parametrize("variant", ["lnl", "ln+linear", "linear"])
@pytest.mark.parametrize("M,dim,ef", [(100, 64, 2), (333, 128, 4), (50, 24, 4)])
def test_transition_variants_fp32(variant, M, dim, ef):
    x, ln_w, ln_b, w1, w2, dy = _transition_case(M, dim, ef)
    got = run_transition(x, ln_w, ln_b, w1, w2, dy, torch.float32, variant)
    if variant == "linear":
        ref = orc.transition_fwd_bwd(x, None, None, w1, w2, dy)
    else:
        ref = orc.transition_fwd_bwd(x, ln_w, ln_b, w1, w2, dy)
    for g_, r_, n in zip(got, ref, T_NAMES):
        if r_ is not None:
            assert_close_fp32(g_, r_, n)


@pytest.mark.parametrize("M,dim,ef", [(2048, 128, 4), (1000, 384, 4), (515, 64, 2)])
def test_transition_bf16_against_fp32_oracle(M, dim, ef):
    x, ln_w, ln_b, w1, w2, dy = _transition_case(M, dim, ef)
    got = run_transition(x, ln_w, ln_b, w1, w2, dy, torch.bfloat16)
    r = [t.to(torch.bfloat16).float() for t in (x, ln_w, ln_b, w1, w2, dy)]
    ref = orc.transition_fwd_bwd(*r)
    for g_, r_, n in zip(got, ref, T_NAMES):
        lowp(g_, r_, n, M)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("M,N,K", [(20000, 512, 128), (1001, 72, 200), (9000, 1024, 128), (130, 8, 8)])
def test_lnl_backward_tensor_core_path(M, N, K, dtype):
    """Split reduction over many CTAs, ragged tiles in every dimension, both 16-bit types."""
    x, ln_w, ln_b, w, b, dy = [t.to(DEV, dtype) for t in _lnl_case(M, N, K, seed=7)]
    dy = dy / 8
    _, mean, rstd = mfb.layernorm_linear_forward(x, w, b, ln_w, ln_b)
    got = mfb.layernorm_linear_backward(dy, x, w, ln_w, ln_b, mean, rstd, True)
    assert _lib.last_path() == "tcgen05"
    ref = orc.layernorm_linear_fwd_bwd(*[t.float().cpu() for t in (x, ln_w, ln_b, w, b, dy)])
    _, dx, dlw, dlb, dw, db = ref
    for g_, r_, n in zip(got, (dx, dw, db, dlw, dlb), ("dx", "dw", "db", "d_ln_w", "d_ln_b")):
        lowp(g_, r_, n, M)
    simt = mfb.layernorm_linear_backward(dy, x, w, ln_w, ln_b, mean, rstd, True, flags=_lib.MF_FLAG_FORCE_SIMT)
    assert _lib.last_path() == "simt"
    for g_, r_, n in zip(got, simt, ("dx", "dw", "db", "d_ln_w", "d_ln_b")):
        lowp(g_, r_.float(), n + " vs CUDA cores", M)


@pytest.mark.parametrize("M,dim,ef,dtype", [(12000, 128, 4, torch.bfloat16), (777, 64, 2, torch.bfloat16),
                                            (300, 384, 4, torch.bfloat16), (1000, 128, 2, torch.float16),
                                            (129, 128, 0.25, torch.bfloat16)])
def test_transition_backward_tensor_core_path(M, dim, ef, dtype):
    """dim = 128 takes the fused backward core (hidden activation recomputed on chip), the other sizes the composition
    of tensor-core GEMMs and row passes; inner = 32 is a single hidden chunk."""
    x, ln_w, ln_b, w1, w2, dy = [t.to(DEV, dtype) for t in _transition_case(M, dim, ef, seed=3)]
    _, mean, rstd = mfb.transition_forward(x, ln_w, ln_b, w1, w2)
    got = mfb.transition_backward(dy, x, ln_w, ln_b, w1, w2, mean, rstd)
    assert _lib.last_path() == "tcgen05"
    ref = orc.transition_fwd_bwd(*[t.float().cpu() for t in (x, ln_w, ln_b, w1, w2, dy)])
    for g_, r_, n in zip(got, ref[1:], ("dx", "d_ln_w", "d_ln_b", "dw1", "dw2")):
        lowp(g_, r_, n, M)


def test_transition_backward_in_two_row_ranges():
    """More than 131072 rows: the fused backward goes through the rows in ranges that share one scratch area, the weight
    gradients accumulate over the ranges and the partial column sums of all ranges are reduced together.  M is chosen so
    that the second range is ragged (not a multiple of the 128-row tile).  Oracle: fp32 on the GPU, TF32 off."""
    M, dim, ef = 131072 + 4096 + 77, 128, 4
    x, ln_w, ln_b, w1, w2, dy = [t.to(DEV, torch.bfloat16) for t in _transition_case(M, dim, ef, seed=9)]
    _, mean, rstd = mfb.transition_forward(x, ln_w, ln_b, w1, w2)
    got = mfb.transition_backward(dy, x, ln_w, ln_b, w1, w2, mean, rstd)
    assert _lib.last_path() == "tcgen05"
    a, b = torch.backends.cuda.matmul.allow_tf32, torch.backends.cudnn.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    try:
        ref = orc.transition_fwd_bwd(*[t.float() for t in (x, ln_w, ln_b, w1, w2, dy)])
    finally:
        torch.backends.cuda.matmul.allow_tf32, torch.backends.cudnn.allow_tf32 = a, b
    for g_, r_, n in zip(got, ref[1:], ("dx", "d_ln_w", "d_ln_b", "dw1", "dw2")):
        lowp(g_, r_, n, M)
