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
    # the backward (the last call) took the path asked for: the tensor-core kernels cover every head size up to 64
    assert _lib.last_path() == ("simt" if flags else "tcgen05")
    # masked keys get exactly zero dK / dV, whatever the precision
    keep = c["mask"][:, :, 0, 0, :].to(DEV)
    assert torch.all(got[2][~keep] == 0) and torch.all(got[3][~keep] == 0)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,N,L,H,D", [(1, 2, 128, 2, 64), (1, 2, 256, 1, 64), (1, 3, 200, 2, 48), (1, 1, 768, 4, 64), (2, 1, 384, 8, 64),
                                       (1, 2, 1100, 1, 56)])
def test_head_sizes_above_32_on_the_tensor_cores(dtype, B, N, L, H, D):
    """Head sizes 33..64 (the reference's single-representation attention uses 64) run as two halves of 32 columns in
    the backward kernels: on-chip dQ accumulators for up to two query tiles, streamed dQ beyond; a head size that is not a
    multiple of 32 leaves the second half partly empty."""
    c = make_case(B, N, L, H, D, seed=3 * L + D)
    got = run_gpu(c, dtype=dtype)
    assert _lib.last_path() == "tcgen05"
    r = rounded(c, dtype)
    ref = orc.evo_attention_fwd_bwd(r["q"], r["k"], r["v"], r["mask"], r["bias"], r["d_out"])
    for g_, r_, n in zip(got, ref, NAMES):
        assert_close_lowp(g_, r_, n)
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


@pytest.mark.parametrize("L", [128, 150])
def test_bias_views_that_are_not_contiguous(L):
    """A pair bias shared by the batch elements (expanded view: batch stride 0) and one whose rows are slices of a wider
    buffer (row stride larger than L).  With L = 128 TMA can address both as they are (forward tiles, and the backward's
    MN-major operand); with L = 150 the rows are not 16-byte multiples and the backward makes its transposed copy."""
    B, N, H, D = 2, 3, 2, 32
    c = make_case(B, N, L, H, D, seed=11 + L)
    dt = torch.bfloat16
    q, k, v, d_o = (c[n].to(DEV, dt) for n in ("q", "k", "v", "d_out"))
    mask = c["mask"].to(DEV)
    shared = c["bias"][:1].to(DEV, dt)                                   # [1, 1, H, L, L]
    wide = torch.zeros(B, 1, H, L, L + 8, device=DEV, dtype=dt)
    wide[..., :L] = c["bias"].to(DEV, dt)
    for name, bias, ref_bias in (("expanded", shared.expand(B, 1, H, L, L), c["bias"][:1].expand(B, 1, H, L, L)),
                                 ("row-sliced", wide[..., :L], c["bias"])):
        assert not bias.is_contiguous()
        o, lse = mfb.evo_attention_forward(q, k, v, mask, bias)
        dq, dk, dv, db = mfb.evo_attention_backward(d_o, q, k, v, mask, bias, o, lse)
        torch.cuda.synchronize()
        assert _lib.last_path() == "tcgen05"
        r = rounded(c, dt)
        ref = orc.evo_attention_fwd_bwd(r["q"], r["k"], r["v"], r["mask"], ref_bias.to(dt).float(), r["d_out"])
        for g_, r_, n in zip((o, dq, dk, dv, db), ref, NAMES):
            assert_close_lowp(g_, r_, f"{name} bias, L={L}: {n}", summed_over=N if n == "dbias" else 1)


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
    """Every output, the row-summed d_pair_bias included, comes out the same bit for bit on both kernel families (the
    tensor-core path sums the rows in a separate kernel with a fixed order).  The shape keeps one work item per (b, n, h),
    so dQ has no cross-CTA partial sums either."""
    c = make_case(1, 40, 96, 4, 32, seed=5)
    a = run_gpu(c, dtype=dtype)
    b = run_gpu(c, dtype=dtype)
    for x, y, n in zip(a, b, NAMES):
        assert torch.equal(x, y), n


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("D,L", [(32, 200), (64, 150), (24, 384)])
def test_fully_masked_row_low_precision(dtype, D, L):
    """A row whose keys are all masked attends uniformly (masked_fill semantics): dV gets dO / L, nothing flows to q, k or
    the bias.  D = 32 / 24 run the tensor-core forward and backward; D = 64 feeds the tensor-core forward's log-sum-exp
    to the CUDA-core backward."""
    c = make_case(1, 4, L, 2, D, seed=D + L)
    c["mask"] = c["mask"].clone()
    c["mask"][0, 1] = False
    got = run_gpu(c, dtype=dtype)
    r = rounded(c, dtype)
    ref = orc.evo_attention_fwd_bwd(r["q"], r["k"], r["v"], r["mask"], r["bias"], r["d_out"])
    for g_, r_, n in zip(got, ref, NAMES):
        assert_close_lowp(g_, r_, f"fully masked {n} D={D}", summed_over=4 if n == "dbias" else 1)
    assert float(got[1][0, 1].abs().max()) == 0.0 and float(got[2][0, 1].abs().max()) == 0.0      # dQ, dK of the masked row


def test_fully_masked_row_noalloc_backward_reads_tensor_core_lse():
    """mf_evo_bwd_noalloc (CUDA cores) fed the log-sum-exp of the default (tensor-core) forward."""
    import ctypes as C
    from megafold_b200.evoattention import _fill_common
    c = make_case(1, 3, 70, 2, 32, seed=9)
    c["mask"] = c["mask"].clone()
    c["mask"][0, 2] = False
    dt = torch.bfloat16
    q, k, v, d_o = (c[n].to(DEV, dt) for n in ("q", "k", "v", "d_out"))
    bias, mask = c["bias"].to(DEV, dt), c["mask"].to(DEV)
    o, lse = mfb.evo_attention_forward(q, k, v, mask, bias)
    assert _lib.last_path() == "tcgen05"
    dq, dk, dv = (torch.empty_like(q) for _ in range(3))
    d_bias = torch.empty((1, 1, 2, 70, 70), dtype=torch.float32, device=DEV)
    a = _lib.EvoBwdArgs()
    _fill_common(a, q, k, v, mask, bias, 0)
    a.dbias_dtype = _lib.MF_F32
    a.o, a.d_o, a.lse = o.data_ptr(), d_o.data_ptr(), lse.data_ptr()
    a.dq, a.dk, a.dv, a.d_bias = dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), d_bias.data_ptr()
    _lib.check(_lib.lib().mf_evo_bwd_noalloc(C.byref(a), _lib.stream_ptr(q.device)), "mf_evo_bwd_noalloc")
    torch.cuda.synchronize()
    r = rounded(c, dt)
    ref = orc.evo_attention_fwd_bwd(r["q"], r["k"], r["v"], r["mask"], r["bias"], r["d_out"])
    for g_, r_, n in zip((dq, dk, dv, d_bias), ref[1:], NAMES[1:]):
        assert_close_lowp(g_, r_, "noalloc after tensor-core forward " + n, summed_over=3 if n == "dbias" else 1)


def test_bounded_wait_expiry_is_reported_and_later_calls_are_refused():
    """A wait that nobody satisfies runs into its cap: the kernel returns normally, the status word turns non-zero and the
    tensor-core entry points refuse further work.  Run in a throw-away process because the status is sticky."""
    import subprocess
    import sys
    code = r"""
import torch, megafold_b200 as mfb
from megafold_b200 import _lib
L = _lib.lib()
assert L.mf_async_status() == 0
assert L.mf_selftest_bounded_wait(None) == 0
torch.cuda.synchronize()
assert L.mf_async_status() != 0, "status word not raised"
t = torch.zeros(4, device="cuda") + 1          # the context is still usable
assert float(t.sum()) == 4.0
q = torch.randn(1, 2, 64, 2, 32, device="cuda", dtype=torch.bfloat16)
bias = torch.randn(1, 1, 2, 64, 64, device="cuda", dtype=torch.bfloat16)
mask = torch.ones(1, 2, 1, 1, 64, dtype=torch.bool, device="cuda")
try:
    mfb.evo_attention_forward(q, q, q, mask, bias)
except RuntimeError as e:
    assert "bounded wait" in str(e), str(e)
    print("REFUSED")
else:
    raise SystemExit("the call after an expired wait was not refused")
"""
    import os
    env = dict(os.environ, PYTHONPATH=os.pathsep.join([os.path.dirname(os.path.dirname(os.path.abspath(__file__)))] + sys.path))
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=300, env=env)
    assert out.returncode == 0 and "REFUSED" in out.stdout, out.stdout + out.stderr


def test_autocast_and_activation_checkpointing():
    """The operator under torch.autocast(bfloat16) and inside torch.utils.checkpoint (the reference wraps its fused
    modules in both, fused_layernorm_linear.py:480 and tensor_typing.py:81-88): same values and gradients as a plain call."""
    from torch.utils.checkpoint import checkpoint
    c = make_case(1, 4, 96, 2, 32, seed=13)
    dt = torch.bfloat16
    mask = c["mask"].to(DEV)

    def leaves():
        return [c[n].to(DEV, dt).requires_grad_(True) for n in ("q", "k", "v", "bias")]

    q, k, v, b = leaves()
    o = mfb.TritonEvoformer(q, k, v, mask, b)
    o.backward(c["d_out"].to(DEV, dt))
    plain = [o.detach()] + [t.grad for t in (q, k, v, b)]
    q, k, v, b = leaves()
    with torch.autocast("cuda", dtype=dt):
        o = checkpoint(lambda *a: mfb.TritonEvoformer(*a), q, k, v, mask, b, use_reentrant=False)
    o.backward(c["d_out"].to(DEV, dt))
    for x, y, n in zip(plain, [o.detach()] + [t.grad for t in (q, k, v, b)], NAMES):
        assert torch.equal(x, y), n
    # LayernormLinear and FusedTransition modules: fp32 parameters under bf16 autocast and a checkpoint, against the
    # same module held in bf16 and called directly
    import copy
    torch.manual_seed(0)
    lin = mfb.LayernormLinear(128, 256, device=DEV)
    tr = mfb.FusedTransition(dim=128, expansion_factor=2, device=DEV)
    x = torch.randn(300, 128, device=DEV)
    for mod in (lin, tr):
        xa = x.clone().requires_grad_(True)
        with torch.autocast("cuda", dtype=dt):
            y = checkpoint(mod, xa, use_reentrant=False)
        y.float().sum().backward()
        mod16 = copy.deepcopy(mod).to(dt)
        xb = x.to(dt).requires_grad_(True)
        yb = mod16(xb)
        yb.float().sum().backward()
        name = type(mod).__name__
        assert y.dtype == dt
        assert_close_lowp(y, yb.float(), name + " under autocast + checkpoint: y")
        assert_close_lowp(xa.grad, xb.grad.float(), name + " under autocast + checkpoint: dx")


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


@pytest.mark.parametrize("B,N,L,H,D", [(1, 2, 1000, 2, 32), (1, 150, 800, 1, 32), (1, 3, 1024, 1, 24), (1, 2, 1536, 2, 32),
                                       (1, 1, 2048, 2, 16)])
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
