"""The shapes of the reference's own attention test sweep (`tests/test_evoattention.py:83-136`: ragged sequence lengths
with head sizes 8 / 16 / 32 / 64, one row with sixteen heads or 128 rows with four), in fp16 as the reference runs them,
through the autograd callable, against the fp32 oracle.

The reference compares its kernel with a torch implementation at `atol = 1e-2, rtol = 0` for fp16
(`tests/test_evoattention.py:73-80`).  The same absolute bound is applied here to o, dq, dk and dv; d_pair_bias is a
sum over the N rows, so its bound grows with sqrt(N) as in the other tests.  The row counts of the largest cases are
cut down (rows are independent) so that the fp32 oracle stays within seconds on host cores.
"""
import pytest
import torch

import megafold_b200 as mfb
from megafold_b200 import _lib
from oracle import pairformer_oracle as orc
from util import assert_close_lowp

pytestmark = pytest.mark.gpu
DEV = "cuda"

SWEEP = [
    # (B, H, N, L, D)
    (1, 16, 1, 23, 8), (1, 16, 1, 136, 8), (1, 16, 1, 341, 8), (1, 16, 1, 499, 8),
    (1, 4, 128, 23, 16), (1, 4, 128, 131, 16), (1, 4, 128, 241, 32), (1, 4, 128, 383, 32), (1, 4, 128, 476, 32),
    (1, 16, 1, 23, 64), (1, 16, 1, 99, 64), (1, 16, 1, 237, 64), (1, 16, 1, 389, 64), (1, 16, 1, 499, 64),
    (1, 16, 1, 128, 64), (1, 4, 128, 128, 32),
    (2, 10, 6, 384, 64), (1, 5, 8, 768, 64), (1, 1, 4, 1280, 64),          # rows cut down from 200 / 100 / 100
]


@pytest.mark.parametrize("B,H,N,L,D", SWEEP)
def test_reference_sweep_shape_fp16(B, H, N, L, D):
    g = torch.Generator().manual_seed(L * 131 + D)
    q, k, v, d_o = (torch.randn(B, N, L, H, D, generator=g).half() for _ in range(4))
    bias = torch.randn(B, 1, H, L, L, generator=g).half()
    mask = torch.rand(B, N, 1, 1, L, generator=g) > 0.2
    mask[..., 0] = True
    leaves = [t.to(DEV).requires_grad_(True) for t in (q, k, v, bias)]
    o = mfb.TritonEvoformer(leaves[0], leaves[1], leaves[2], mask.to(DEV), leaves[3])
    o.backward(d_o.to(DEV))
    torch.cuda.synchronize()
    assert _lib.last_path() == "tcgen05"
    assert _lib.lib().mf_async_status() == 0
    ref = orc.evo_attention_fwd_bwd(q.float(), k.float(), v.float(), mask, bias.float(), d_o.float())
    got = (o, leaves[0].grad, leaves[1].grad, leaves[2].grad, leaves[3].grad)
    for name, a, r in zip(("o", "dq", "dk", "dv"), got, ref):
        a, r = a.float().cpu(), r.float()
        err = float((a - r).abs().max())
        print(f"[parity] sweep {(B, H, N, L, D)} {name}: max_abs_err {err:.3e}")
        assert err <= 1e-2, f"{name}: max abs error {err:.3e} above the reference test's atol of 1e-2"
    assert_close_lowp(got[4], ref[4], f"sweep {(B, H, N, L, D)} d_pair_bias", tol=1e-2, summed_over=N)
