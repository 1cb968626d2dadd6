"""Parity of the CUDA attention (through the C ABI) with the CPU oracle and the golden vectors."""
import os

import numpy as np
import pytest
import torch

import cases
import megafold_b200 as mfb
from megafold_b200 import _lib
from oracle import pairformer_oracle as orc
from util import assert_close_fp32, assert_close_lowp

pytestmark = pytest.mark.gpu
G = os.path.join(os.path.dirname(__file__), "golden")
DEV = "cuda"


def run_gpu(c, dtype=torch.float32, flags=0, bias_dtype=None):
    q, k, v = (c[n].to(DEV, dtype) for n in ("q", "k", "v"))
    bias = c["bias"].to(DEV, bias_dtype or dtype)
    mask = c["mask"].to(DEV)
    d_o = c["d_out"].to(DEV, dtype)
    o, lse = mfb.evo_attention_forward(q, k, v, mask, bias, flags=flags)
    dq, dk, dv, db = mfb.evo_attention_backward(d_o, q, k, v, mask, bias, o, lse, flags=flags)
    torch.cuda.synchronize()
    return o, dq, dk, dv, db


def rounded(c, dtype):
    """The inputs as the kernel sees them after storage rounding, back in fp32 for the oracle."""
    r = dict(c)
    for n in ("q", "k", "v", "bias", "d_out"):
        r[n] = c[n].to(dtype).float()
    return r


def make_case(B, N, L, H, D, seed, mask_p=0.25):
    g = torch.Generator().manual_seed(seed)
    q, k, v = (torch.randn(B, N, L, H, D, generator=g) for _ in range(3))
    bias = torch.randn(B, 1, H, L, L, generator=g)
    d_out = torch.randn(B, N, L, H, D, generator=g)
    mask = torch.rand(B, N, 1, 1, L, generator=g) > mask_p
    mask[..., 0] = True
    return dict(q=q, k=k, v=v, bias=bias, mask=mask, d_out=d_out)


NAMES = ("o", "dq", "dk", "dv", "dbias")


def test_cfg1_fp32_matches_oracle_and_reference_vectors():
    c = cases.evo_cfg1()
    got = run_gpu(c)
    assert _lib.last_path() == "simt"          # fp32 storage never takes the tensor-core path
    ref = orc.evo_attention_fwd_bwd(c["q"], c["k"], c["v"], c["mask"], c["bias"], c["d_out"])
    for g_, r_, n in zip(got, ref, NAMES):
        assert_close_fp32(g_, r_, n)
    gold = np.load(os.path.join(G, "evo_cfg1.npz"))
    for g_, n in zip(got, NAMES):
        assert_close_fp32(g_[cases.CFG1_SUB], torch.from_numpy(gold[n + "_sub"]), "golden " + n)
    # masked keys (the last 8 of every row): exactly zero gradient
    o, dq, dk, dv, db = got
    assert torch.all(dk[:, :, -8:] == 0) and torch.all(dv[:, :, -8:] == 0)
    assert torch.all(db[..., -8:] == 0)


def test_small_fp32_matches_reference_vectors():
    g = np.load(os.path.join(G, "evo_small.npz"))
    c = cases.evo_small()
    got = run_gpu(c)
    for g_, n in zip(got, NAMES):
        assert_close_fp32(g_, torch.from_numpy(g[n]), n)


@pytest.mark.parametrize("B,N,L,H,D", [(1, 2, 23, 2, 8), (2, 3, 77, 1, 16), (1, 2, 99, 3, 24), (1, 5, 130, 2, 32),
                                       (1, 2, 67, 2, 64), (1, 1, 200, 2, 40), (1, 3, 33, 1, 128)])
def test_ragged_shapes_fp32(B, N, L, H, D):
    c = make_case(B, N, L, H, D, seed=L + D)
    got = run_gpu(c)
    ref = orc.evo_attention_fwd_bwd(c["q"], c["k"], c["v"], c["mask"], c["bias"], c["d_out"])
    for g_, r_, n in zip(got, ref, NAMES):
        assert_close_fp32(g_, r_, n)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("flags", [0, _lib.MF_FLAG_FORCE_SIMT])
@pytest.mark.parametrize("B,N,L,H,D", [(1, 6, 64, 4, 32), (1, 3, 150, 2, 32), (2, 1, 96, 4, 24), (1, 2, 384, 2, 64),
                                       (1, 4, 257, 4, 16), (1, 2, 40, 2, 8)])
def test_low_precision_against_fp32_oracle(dtype, flags, B, N, L, H, D):
    c = make_case(B, N, L, H, D, seed=7 * L + D)
    got = run_gpu(c, dtype=dtype, flags=flags)
    r = rounded(c, dtype)
    ref = orc.evo_attention_fwd_bwd(r["q"], r["k"], r["v"], r["mask"], r["bias"], r["d_out"])
    for g_, r_, n in zip(got, ref, NAMES):
        assert_close_lowp(g_, r_, f"{n} ({_lib.last_path()})")
    # masked keys get exactly zero dK / dV, whatever the precision
    keep = c["mask"][:, :, 0, 0, :].to(DEV)
    assert torch.all(got[2][~keep] == 0) and torch.all(got[3][~keep] == 0)


def test_fp32_bias_with_bf16_qkv():
    """The reference benchmark passes an fp32 pair_bias next to bf16 q/k/v (benchmarks/evoattention_speed.py:68)."""
    c = make_case(1, 4, 128, 4, 32, seed=3)
    got = run_gpu(c, dtype=torch.bfloat16, bias_dtype=torch.float32)
    assert got[4].dtype == torch.float32
    r = rounded(c, torch.bfloat16)
    r["bias"] = c["bias"]
    ref = orc.evo_attention_fwd_bwd(r["q"], r["k"], r["v"], r["mask"], r["bias"], r["d_out"])
    for g_, r_, n in zip(got, ref, NAMES):
        assert_close_lowp(g_, r_, n)


def test_additive_float_mask_and_fully_masked_row():
    c = cases.evo_small()
    add = dict(c)
    add["mask"] = 1e9 * (c["mask"].float() - 1.0)
    a = run_gpu(c)
    b = run_gpu(add)
    for x, y, n in zip(a, b, NAMES):
        assert_close_fp32(x, y, "additive vs keep " + n)
    c["mask"] = c["mask"].clone()
    c["mask"][0, 1] = False                         # one row with every key masked -> uniform attention
    got = run_gpu(c)
    ref = orc.evo_attention_fwd_bwd(c["q"], c["k"], c["v"], c["mask"], c["bias"], c["d_out"])
    for g_, r_, n in zip(got, ref, NAMES):
        assert_close_fp32(g_, r_, "fully masked " + n)


def test_strided_inputs_and_autograd_function():
    """q, k, v as the model passes them: non-contiguous views of [(b n), h, l, d] (attention.py:469-471)."""
    B, N, L, H, D = 1, 4, 48, 2, 32
    c = make_case(B, N, L, H, D, seed=11)
    packed = {n: c[n].permute(0, 1, 3, 2, 4).contiguous() for n in ("q", "k", "v")}        # [B,N,H,L,D]
    leaves = {n: packed[n].to(DEV).requires_grad_(True) for n in packed}
    views = {n: leaves[n].permute(0, 1, 3, 2, 4) for n in leaves}                          # [B,N,L,H,D] strided
    assert not views["q"].is_contiguous()
    bias = c["bias"].to(DEV).requires_grad_(True)
    o = mfb.TritonEvoformer(views["q"], views["k"], views["v"], c["mask"].to(DEV), bias)
    o.backward(c["d_out"].to(DEV))
    ref = orc.evo_attention_fwd_bwd(c["q"], c["k"], c["v"], c["mask"], c["bias"], c["d_out"])
    assert_close_fp32(o, ref[0], "o")
    for n, r_ in zip(("q", "k", "v"), ref[1:4]):
        assert_close_fp32(leaves[n].grad.permute(0, 1, 3, 2, 4), r_, "d" + n)
    assert_close_fp32(bias.grad, ref[4], "dbias")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_bit_reproducible(dtype):
    c = make_case(1, 8, 96, 4, 32, seed=5)
    a = run_gpu(c, dtype=dtype)
    path = _lib.last_path()
    b = run_gpu(c, dtype=dtype)
    for x, y, n in zip(a, b, NAMES):
        if n == "dbias" and path == "tcgen05":
            # the tensor-core backward adds every row's dS into dBias with fp32 atomics, like the reference
            # (evoattention.py:465): the sum is exact to rounding but its order is not fixed
            assert_close_lowp(x, y.float(), n, tol=1e-2)
        else:
            assert torch.equal(x, y), n


@pytest.fixture(autouse=True)
def _no_bounded_wait_expired():
    yield
    assert _lib.lib().mf_async_status() == 0, "a kernel gave up on a bounded wait"


def test_host_pipeline_matches_device_call():
    """evoformer_fwd_bwd_host (row chunks over three streams; replayed as a CUDA graph from the second call with the
    same host buffers on) gives what the device-resident operator gives, also after the buffers' contents change."""
    c = make_case(1, 10, 96, 4, 32, seed=21)
    pin = {k: (v.bfloat16() if v.is_floating_point() else v).pin_memory() for k, v in c.items()}
    for rep in range(4):
        if rep:
            fresh = make_case(1, 10, 96, 4, 32, seed=21 + rep)
            for k in pin:                                                # same pinned buffers, new contents
                pin[k].copy_(fresh[k].bfloat16() if fresh[k].is_floating_point() else fresh[k])
            c = fresh
        out = mfb.evoformer_fwd_bwd_host(pin["q"], pin["k"], pin["v"], pin["mask"], pin["bias"], pin["d_out"], chunks=3)
        ref = run_gpu(c, dtype=torch.bfloat16)
        for n, r_ in zip(("o", "dq", "dk", "dv"), ref[:4]):
            assert torch.equal(out[n], r_.cpu()), (rep, n)               # rows are independent: chunking changes nothing
        assert_close_lowp(out["d_bias"].float(), ref[4].float().cpu(), f"d_bias (call {rep})", tol=1e-2)   # summed per chunk, then over chunks
    from megafold_b200 import host_pipeline
    pipe = next(iter(host_pipeline._cache.values()))
    assert pipe.graph is not None, "the three-stream schedule was not captured into a CUDA graph"


@pytest.mark.parametrize("B,N,L,H,D", [(1, 2, 1000, 2, 32), (1, 150, 800, 1, 32), (1, 3, 1024, 1, 24)])
def test_long_rows_stream_dq(B, N, L, H, D):
    """More than six query tiles: the backward kernel no longer keeps every dQ accumulator on chip but adds each block's
    product to an fp32 accumulator in global memory (with and without the key tiles spread over CTAs)."""
    c = make_case(B, N, L, H, D, seed=L + N)
    got = run_gpu(c, dtype=torch.bfloat16)
    assert _lib.last_path() == "tcgen05"
    r = rounded(c, torch.bfloat16)
    ref = orc.evo_attention_fwd_bwd(r["q"], r["k"], r["v"], r["mask"], r["bias"], r["d_out"])
    for g_, r_, n in zip(got, ref, NAMES):
        assert_close_lowp(g_, r_, n)
