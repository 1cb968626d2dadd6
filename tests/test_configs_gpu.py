"""The benchmark configurations at their own shapes: full size where the oracle finishes in seconds, otherwise
through properties that do not depend on the size (rows are independent; d_pair_bias is a sum over rows)."""
import pytest
import torch

import megafold_b200 as mfb
from megafold_b200 import _lib, workloads
from oracle import pairformer_oracle as orc
from util import assert_close_lowp

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _gpu(c, rows=slice(None)):
    q, k, v, m, g = (c[n][:, rows].to(DEV) for n in ("q", "k", "v", "mask", "d_out"))
    bias = c["bias"].to(DEV)
    o, lse = mfb.evo_attention_forward(q, k, v, m, bias)
    dq, dk, dv, db = mfb.evo_attention_backward(g, q, k, v, m, bias, o, lse)
    torch.cuda.synchronize()
    return o, dq, dk, dv, db


def _oracle(c, rows):
    f = lambda t: t[:, rows].float()      # noqa: E731
    return orc.evo_attention_fwd_bwd(f(c["q"]), f(c["k"]), f(c["v"]), c["mask"][:, rows], c["bias"].float(), f(c["d_out"]))


def test_config3_single_attention_full_size():
    """B = 2, N = 1, L = 768, H = 16, D = 24 (head size padded to 32 inside the kernels), 10 % of the keys masked."""
    c = workloads.single_attention()
    got = _gpu(c)
    assert _lib.last_path() == "tcgen05"
    ref = _oracle(c, slice(None))
    for g_, r_, n in zip(got, ref, ("o", "dq", "dk", "dv", "dbias")):
        assert_close_lowp(g_, r_, n)
    masked = ~c["mask"][:, 0, 0, 0]                       # [B, L]
    for b in range(2):
        assert float(got[2][b, 0, masked[b]].abs().max()) == 0.0        # dK rows of masked keys
        assert float(got[3][b, 0, masked[b]].abs().max()) == 0.0        # dV rows of masked keys
        assert float(got[4][b, 0, :, :, masked[b]].abs().max()) == 0.0  # dBias columns of masked keys


def test_config2_full_size_by_rows():
    """q/k/v [1, 384, 384, 4, 32]: the first and last 12 rows against the oracle; every row equal, bit for bit, to the
    same row computed in a 12-row call (dQ: to rounding); d_pair_bias equal to the sum of the d_pair_bias of four 96-row calls."""
    c = workloads.triangle_attention()
    full = _gpu(c)
    assert _lib.last_path() == "tcgen05"
    for rows in (slice(0, 12), slice(372, 384)):
        ref = _oracle(c, rows)
        for g_, r_, n in zip(full[:4], ref[:4], ("o", "dq", "dk", "dv")):
            assert_close_lowp(g_[:, rows], r_, f"{n} rows {rows.start}..{rows.stop}")
        part = _gpu(c, rows)
        for g_, p_, n in zip(full[:4], part[:4], ("o", "dq", "dk", "dv")):
            if n == "dq":       # a 12-row call spreads the key tiles over CTAs: dQ is then summed in another order
                assert_close_lowp(g_[:, rows], p_.float(), n, tol=1e-2)
            else:
                assert torch.equal(g_[:, rows], p_), n
    acc = torch.zeros_like(full[4], dtype=torch.float32)
    for s in range(0, 384, 96):
        acc += _gpu(c, slice(s, s + 96))[4].float()
    assert_close_lowp(full[4], acc, "d_pair_bias as a sum over row blocks", tol=1e-2)
    pad = slice(352, 384)                                  # the 32 padded tokens
    assert float(full[2][:, :, pad].abs().max()) == 0.0 and float(full[3][:, :, pad].abs().max()) == 0.0
    assert float(full[4][..., pad].abs().max()) == 0.0
