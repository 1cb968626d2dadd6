"""mf_evo_bwd_noalloc: the backward pass for hosts that cannot allocate.

Some users of this library run inside a process whose GPU memory was all claimed by an in-house pool at
start-up, or on a path where the device-wide synchronisation of cudaMalloc / cudaFree is not acceptable; they
cannot give mf_evo_bwd the workspace it asks for.  The variant tested here keeps its scratch inside the
library image.  The test calls it through the C ABI twice in a row (different inputs, so stale scratch from
the first call would show) and compares with the regular entry point running the same kernels.

This file sorts last on purpose: a run that stops at the first failure has then already run every other test.
"""
import ctypes as C

import pytest
import torch

from megafold_b200 import _lib
from megafold_b200.evoattention import _fill_common

pytestmark = pytest.mark.gpu


def _inputs(seed, B=1, N=3, L=70, H=2, D=32, dtype=torch.bfloat16):
    g = torch.Generator().manual_seed(seed)
    q, k, v, d_o = (torch.randn(B, N, L, H, D, generator=g).to("cuda", dtype) for _ in range(4))
    bias = torch.randn(B, 1, H, L, L, generator=g).to("cuda", dtype)
    mask = (torch.rand(B, N, 1, 1, L, generator=g) > 0.2).to("cuda")
    mask[..., 0] = True
    return q, k, v, mask, bias, d_o


def _backward(entry, q, k, v, mask, bias, d_o, o, lse, with_workspace):
    B, N, L, H, D = q.shape
    dq, dk, dv = (torch.empty_like(q) for _ in range(3))
    d_bias = torch.empty((B, 1, H, L, L), dtype=torch.float32, device=q.device)
    a = _lib.EvoBwdArgs()
    _fill_common(a, q, k, v, mask, bias, _lib.MF_FLAG_FORCE_SIMT)
    a.dbias_dtype = _lib.MF_F32
    a.o, a.d_o, a.lse = o.data_ptr(), d_o.data_ptr(), lse.data_ptr()
    a.dq, a.dk, a.dv, a.d_bias = dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), d_bias.data_ptr()
    ws = None
    if with_workspace:
        ws = _lib.workspace(_lib.lib().mf_evo_bwd_workspace_bytes(C.byref(a)), q.device)
        a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
    rc = entry(C.byref(a), _lib.stream_ptr(q.device))
    _lib.check(rc, "backward")
    torch.cuda.synchronize()
    return dq, dk, dv, d_bias


def test_noalloc_backward_matches_regular_entry_point_twice():
    import megafold_b200 as mfb
    L_ = _lib.lib()
    assert L_.mf_evo_bwd_noalloc_max_rows() == 1 << 20
    for seed in (0, 1):                      # two calls in a row through the same built-in scratch
        q, k, v, mask, bias, d_o = _inputs(seed)
        o, lse = mfb.evo_attention_forward(q, k, v, mask, bias, flags=_lib.MF_FLAG_FORCE_SIMT)
        ref = _backward(L_.mf_evo_bwd, q, k, v, mask, bias, d_o, o, lse, with_workspace=True)
        got = _backward(L_.mf_evo_bwd_noalloc, q, k, v, mask, bias, d_o, o, lse, with_workspace=False)
        # against the fp32 oracle on the inputs as stored (bf16), at the tolerance of the other low-precision tests
        from oracle import pairformer_oracle as orc
        f = lambda t: t.float().cpu()      # noqa: E731
        oracle = orc.evo_attention_fwd_bwd(f(q), f(k), f(v), mask.cpu(), f(bias), f(d_o))
        for name, g_, r_ in zip(("dq", "dk", "dv", "dbias"), got, oracle[1:]):
            torch.testing.assert_close(g_.float().cpu(), r_, rtol=2e-2, atol=2e-2 * (3 ** 0.5 if name == "dbias" else 1.0),
                                       msg=lambda m: f"seed {seed} {name} vs oracle: {m}")
        for name, g_, r_ in zip(("dq", "dk", "dv", "dbias"), got, ref):
            # same kernels, same summation order: 2e-2 is the bf16 tolerance of the other tests, equality is expected
            torch.testing.assert_close(g_.float(), r_.float(), rtol=2e-2, atol=2e-2, msg=lambda m: f"seed {seed} {name}: {m}")
            assert torch.equal(g_, r_), f"seed {seed} {name} differs bitwise"


def test_noalloc_rejects_sizes_beyond_the_built_in_scratch():
    q, k, v, mask, bias, d_o = _inputs(2, N=1, L=16, H=1, D=8)
    a = _lib.EvoBwdArgs()
    _fill_common(a, q, k, v, mask, bias, 0)
    a.N, a.L = 60000, 32                     # B*N*H*L = 1.92 Mi rows: beyond the limit; rejected before any launch
    a.dbias_dtype = _lib.MF_F32
    dummy = q.data_ptr()
    a.o = a.d_o = a.lse = a.dq = a.dk = a.dv = a.d_bias = dummy
    rc = _lib.lib().mf_evo_bwd_noalloc(C.byref(a), None)
    assert rc == -2
    assert b"built-in scratch" in _lib.lib().mf_last_error_string()
