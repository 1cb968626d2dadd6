"""The benchmark configurations at their own sizes, every output against the fp32 oracle.

Where the fp32 oracle would take minutes on host cores (the GEMM-heavy configurations) it is evaluated on the GPU in
fp32 with TF32 switched off: the same code, the same arithmetic, only a faster machine.  The attention oracle of
configuration 2 runs on the host (a few seconds).
"""
import contextlib

import pytest
import torch

import megafold_b200 as mfb
from megafold_b200 import _lib, workloads
from oracle import pairformer_oracle as orc
from util import assert_close_lowp

pytestmark = pytest.mark.gpu
DEV = "cuda"


@contextlib.contextmanager
def exact_fp32_matmul():
    """fp32 oracle on the GPU: no TF32 anywhere."""
    a, b = torch.backends.cuda.matmul.allow_tf32, torch.backends.cudnn.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    try:
        yield
    finally:
        torch.backends.cuda.matmul.allow_tf32, torch.backends.cudnn.allow_tf32 = a, b


def _gpu(c, rows=slice(None)):
    q, k, v, m, g = (c[n][:, rows].to(DEV) for n in ("q", "k", "v", "mask", "d_out"))
    bias = c["bias"].to(DEV)
    o, lse = mfb.evo_attention_forward(q, k, v, m, bias)
    dq, dk, dv, db = mfb.evo_attention_backward(g, q, k, v, m, bias, o, lse)
    torch.cuda.synchronize()
    return o, dq, dk, dv, db


def _oracle(c, rows=slice(None)):
    f = lambda t: t[:, rows].float()      # noqa: E731
    return orc.evo_attention_fwd_bwd(f(c["q"]), f(c["k"]), f(c["v"]), c["mask"][:, rows], c["bias"].float(), f(c["d_out"]))


def test_config3_single_attention_full_size():
    """B = 2, N = 1, L = 768, H = 16, D = 24 (head size padded to 32 inside the kernels), 10 % of the keys masked."""
    c = workloads.single_attention()
    got = _gpu(c)
    assert _lib.last_path() == "tcgen05"
    ref = _oracle(c)
    for g_, r_, n in zip(got, ref, ("o", "dq", "dk", "dv", "dbias")):
        assert_close_lowp(g_, r_, "cfg3 " + n)
    masked = ~c["mask"][:, 0, 0, 0]                       # [B, L]
    for b in range(2):
        assert float(got[2][b, 0, masked[b]].abs().max()) == 0.0        # dK rows of masked keys
        assert float(got[3][b, 0, masked[b]].abs().max()) == 0.0        # dV rows of masked keys
        assert float(got[4][b, 0, :, :, masked[b]].abs().max()) == 0.0  # dBias columns of masked keys


def test_config2_full_size_every_row_and_the_bias_gradient():
    """q/k/v [1, 384, 384, 4, 32] bf16: all 384 rows of o / dq / dk / dv and the d_pair_bias that sums over them, against
    the fp32 oracle of the whole problem (host cores, a few seconds)."""
    c = workloads.triangle_attention()
    full = _gpu(c)
    assert _lib.last_path() == "tcgen05"
    ref = _oracle(c)
    for g_, r_, n in zip(full[:4], ref[:4], ("o", "dq", "dk", "dv")):
        assert_close_lowp(g_, r_, "cfg2 " + n)
    assert_close_lowp(full[4], ref[4], "cfg2 d_pair_bias", summed_over=384)
    # rows are independent: a 12-row call reproduces its rows of o, dk, dv bit for bit (dQ: to rounding, a 12-row call
    # spreads the key tiles over CTAs and sums dQ in another order)
    rows = slice(372, 384)
    part = _gpu(c, rows)
    for g_, p_, n in zip(full[:4], part[:4], ("o", "dq", "dk", "dv")):
        if n == "dq":
            assert_close_lowp(g_[:, rows], p_.float(), "cfg2 dq rows vs 12-row call", tol=1e-2)
        else:
            assert torch.equal(g_[:, rows], p_), n
    # the bias gradient is bit-reproducible run to run (fixed summation order)
    again = _gpu(c)
    assert torch.equal(full[4], again[4])
    pad = slice(352, 384)                                  # the 32 padded tokens
    assert float(full[2][:, :, pad].abs().max()) == 0.0 and float(full[3][:, :, pad].abs().max()) == 0.0
    assert float(full[4][..., pad].abs().max()) == 0.0


def test_config2_layernorm_linear_full_size():
    """The projection around configuration 2: x [147456, 128] -> [147456, 512], forward and backward, at its own M (the
    weight gradient's split reduction runs with about two work items per SM).  Oracle: fp32 on the GPU, TF32 off."""
    c = workloads.layernorm_linear()
    d = {k: (v.to(DEV) if v is not None else None) for k, v in c.items()}
    y, mean, rstd = mfb.layernorm_linear_forward(d["x"], d["w"], d["b"], d["ln_w"], d["ln_b"])
    assert _lib.last_path() == "tcgen05"
    dx, dw, db, dlw, dlb = mfb.layernorm_linear_backward(d["d_out"], d["x"], d["w"], d["ln_w"], d["ln_b"], mean, rstd, True)
    assert _lib.last_path() == "tcgen05"
    with exact_fp32_matmul():
        ref = orc.layernorm_linear_fwd_bwd(*[d[k].float() if d[k] is not None else None for k in ("x", "ln_w", "ln_b", "w", "b")],
                                           d["d_out"].float())
    ry, rdx, rdlw, rdlb, rdw, rdb = ref
    M = c["x"].shape[0]
    assert_close_lowp(y, ry, "lnl y")
    assert_close_lowp(dx, rdx, "lnl dx")
    for g_, r_, n in ((dw, rdw, "dw"), (db, rdb, "db"), (dlw, rdlw, "d_ln_w"), (dlb, rdlb, "d_ln_b")):
        assert_close_lowp(g_, r_, "lnl " + n, summed_over=M)


def test_config4_transition_full_size():
    """x [262144, 128], inner 512: y, dx, dW1, dW2, dgamma, dbeta at the benchmark's M.  Oracle: fp32 on the GPU, TF32 off."""
    c = workloads.transition()
    d = {k: v.to(DEV) for k, v in c.items()}
    y, mean, rstd = mfb.transition_forward(d["x"], d["ln_w"], d["ln_b"], d["w1"], d["w2"])
    assert _lib.last_path() == "tcgen05"
    dx, dlw, dlb, dw1, dw2 = mfb.transition_backward(d["d_out"], d["x"], d["ln_w"], d["ln_b"], d["w1"], d["w2"], mean, rstd)
    assert _lib.last_path() == "tcgen05"
    with exact_fp32_matmul():
        ref = orc.transition_fwd_bwd(*[d[k].float() for k in ("x", "ln_w", "ln_b", "w1", "w2")], d["d_out"].float())
    ry, rdx, rdlw, rdlb, rdw1, rdw2 = ref
    M = c["x"].shape[0]
    assert_close_lowp(y, ry, "transition y")
    assert_close_lowp(dx, rdx, "transition dx")
    for g_, r_, n in ((dw1, rdw1, "dw1"), (dw2, rdw2, "dw2"), (dlw, rdlw, "d_ln_w"), (dlb, rdlb, "d_ln_b")):
        assert_close_lowp(g_, r_, "transition " + n, summed_over=M)
