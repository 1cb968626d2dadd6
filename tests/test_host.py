"""Host-side logic: shape checks, state_dict compatibility, row partition, sharded gradient (gloo)."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import cases
import megafold_b200 as mfb
from megafold_b200.evoattention import _check_shapes
from oracle import pairformer_oracle as orc


def test_shape_checks():
    q = torch.zeros(2, 3, 8, 2, 16)
    m = torch.ones(2, 3, 1, 1, 8, dtype=torch.bool)
    b = torch.zeros(2, 1, 2, 8, 8)
    assert _check_shapes(q, q, q, m, b) == (2, 3, 8, 2, 16)
    with pytest.raises(ValueError):
        _check_shapes(q, q[:, :2], q, m, b)
    with pytest.raises(ValueError):
        _check_shapes(q, q, q, m, torch.zeros(2, 3, 2, 8, 8))     # dim 1 of the bias must be 1
    with pytest.raises(ValueError):
        _check_shapes(q, q, q, torch.ones(2, 3, 8, dtype=torch.bool), b)
    with pytest.raises(ValueError):
        _check_shapes(q, q, q, m, None)
    with pytest.raises(TypeError):
        _check_shapes(q, q.half(), q, m, b)


def test_state_dict_keys_match_reference_modules():
    t = mfb.FusedTransition(16, expansion_factor=4)
    assert sorted(t.state_dict()) == ["ff.0.BIAS", "ff.0.WEIGHT", "ff.0.linear_weight", "ff.2.weight"]
    assert t.state_dict()["ff.0.linear_weight"].shape == (16, 128)
    assert t.state_dict()["ff.2.weight"].shape == (16, 64)
    l = mfb.LayernormLinear(16, 24)
    assert sorted(l.state_dict()) == ["BIAS", "WEIGHT", "linear_bias", "linear_weight"]
    assert l.linear_weight.shape == (16, 24)
    l2 = mfb.LayernormLinear(16, 24, has_layernorm_bias=False, has_linear_bias=False)
    assert sorted(l2.state_dict()) == ["WEIGHT", "linear_weight"]
    l3 = mfb.LayernormLinear(16, 24)
    l3.load_state_dict(l.state_dict(), strict=True)
    assert sorted(mfb.FusedTransition(16, include_ln=False).state_dict()) == ["ff.0.weight", "ff.2.weight"]
    assert sorted(mfb.FusedTransition(16, use_layernormlinear=False).state_dict()) == [
        "ff.0.bias", "ff.0.weight", "ff.1.weight", "ff.3.weight"]


def test_row_shard_covers_all_rows():
    for n, w in ((384, 8), (10, 4), (3, 8), (768, 3)):
        spans = [mfb.row_shard(n, r, w) for r in range(w)]
        assert spans[0][0] == 0 and spans[-1][1] == n
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        assert max(e - s for s, e in spans) - min(e - s for s, e in spans) <= 1
    with pytest.raises(ValueError):
        mfb.row_shard(8, 2, 2)


def _oracle_attention(q, k, v, m, b):
    return orc.evo_attention(q, k, v, m, b)


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        c = cases.evo_small()
        N = c["q"].shape[1]
        s, e = mfb.row_shard(N, rank, world)
        q, k, v = (c[n][:, s:e].clone().requires_grad_(True) for n in ("q", "k", "v"))
        bias = c["bias"].clone().requires_grad_(True)
        o = mfb.sharded_evoformer(q, k, v, c["mask"][:, s:e], bias, attention=_oracle_attention)
        o.backward(c["d_out"][:, s:e])
        torch.save(dict(o=o.detach(), dq=q.grad, dbias=bias.grad, span=(s, e)), os.path.join(out, f"r{rank}.pt"))
    finally:
        dist.destroy_process_group()


def test_row_sharded_bias_gradient_is_all_reduced(tmp_path):
    world = 2
    port = 29500 + os.getpid() % 2000
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    c = cases.evo_small()
    o, dq, dk, dv, db = orc.evo_attention_fwd_bwd(c["q"], c["k"], c["v"], c["mask"], c["bias"], c["d_out"])
    for r in range(world):
        got = torch.load(os.path.join(tmp_path, f"r{r}.pt"))
        s, e = got["span"]
        torch.testing.assert_close(got["o"], o[:, s:e], rtol=1e-5, atol=1e-6)
        torch.testing.assert_close(got["dq"], dq[:, s:e], rtol=1e-5, atol=1e-6)
        torch.testing.assert_close(got["dbias"], db, rtol=1e-5, atol=1e-5)     # full sum on every rank
