"""Row-sharded Pairformer block: communication and autograd plumbing on CPU ranks (gloo), with the operator oracle
standing in for the CUDA library."""
import os
from types import SimpleNamespace

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import megafold_b200 as mfb
from megafold_b200.pairformer_block import GatherRows, PairformerBlock, TransposeShards
from oracle import pairformer_block_oracle as blk
from oracle import pairformer_oracle as orc

L, C, CS = 20, 16, 24


def oracle_ops():
    return SimpleNamespace(lnl=lambda x, lw, lb, w, b: orc.layernorm_linear(x, lw, lb, w, b),
                           attention=orc.evo_attention, transition=orc.transition)


def make_block():
    torch.manual_seed(5)
    m = PairformerBlock(dim_pair=C, dim_single=CS, tri_heads=2, tri_dim_head=8, single_heads=3, single_dim_head=8,
                        expansion=2, ops=oracle_ops())
    with torch.no_grad():
        for p in m.parameters():
            p.add_(0.05 * torch.randn_like(p))
    return m


def make_inputs():
    g = torch.Generator().manual_seed(11)
    pair = torch.randn(L, L, C, generator=g)
    single = torch.randn(L, CS, generator=g)
    mask = torch.ones(L, dtype=torch.bool)
    mask[-3:] = False
    d_pair = torch.randn(L, L, C, generator=g)
    d_single = torch.randn(L, CS, generator=g)
    return pair, single, mask, d_pair, d_single


PAIR_TRACK = ("tri_start.", "tri_end.", "tr_", "single_attn.pair_ln", "single_attn.w_pair_bias")


def reference():
    m = make_block()
    pair, single, mask, d_pair, d_single = make_inputs()
    params = blk.params_of(m)
    pair = pair.clone().requires_grad_(True)
    x, s = blk.block(pair, single, mask, params)
    (x * d_pair).sum().add((s * d_single).sum()).backward()
    grads = {}
    for name, a in (("tri_start", params["tri_start"]), ("tri_end", params["tri_end"]), ("single_attn", params["single_attn"])):
        for k, v in a.items():
            if torch.is_tensor(v):
                grads[f"{name}.{k}"] = v.grad
    for k, v in params["transition"].items():
        grads[f"tr_{k}"] = v.grad
    return x.detach(), s.detach(), pair.grad, grads


def test_block_unsharded_matches_the_plain_torch_block():
    m = make_block()
    pair, single, mask, d_pair, d_single = make_inputs()
    pair = pair.clone().requires_grad_(True)
    x, s = m(pair, single, mask)
    (x * d_pair).sum().add((s * d_single).sum()).backward()
    rx, rs, rdpair, rgrads = reference()
    torch.testing.assert_close(x, rx, rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(s, rs, rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(pair.grad, rdpair, rtol=1e-4, atol=1e-5)
    for name, p in m.named_parameters():
        torch.testing.assert_close(p.grad, rgrads[name], rtol=1e-4, atol=1e-4, msg=name)


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # the two communication primitives on their own
        a, b = mfb.row_shard(7, rank, world)
        full = torch.arange(7 * 7 * 2, dtype=torch.float32).view(7, 7, 2)
        got = TransposeShards.apply(full[a:b].clone())
        assert torch.equal(got, full.transpose(0, 1)[a:b])
        assert torch.equal(GatherRows.apply(full[a:b].clone(), 7), full)
        # the block on this rank's rows
        m = make_block()
        pair, single, mask, d_pair, d_single = make_inputs()
        a, b = mfb.row_shard(L, rank, world)
        rows = pair[a:b].clone().requires_grad_(True)
        x, s = m(rows, single, mask)
        (x * d_pair[a:b]).sum().add((s * d_single).sum()).backward()
        grads = {}
        for name, p in m.named_parameters():
            g = p.grad.clone()
            if name.startswith(PAIR_TRACK):
                dist.all_reduce(g)          # what data-parallel training does with the partial sums over rows
            grads[name] = g
        torch.save(dict(x=x.detach(), s=s.detach(), dpair=rows.grad, grads=grads, span=(a, b)), os.path.join(out, f"r{rank}.pt"))
    finally:
        dist.destroy_process_group()


def test_block_sharded_over_two_ranks(tmp_path):
    world = 2
    port = 31500 + os.getpid() % 2000
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    rx, rs, rdpair, rgrads = reference()
    for r in range(world):
        got = torch.load(os.path.join(tmp_path, f"r{r}.pt"))
        a, b = got["span"]
        torch.testing.assert_close(got["x"], rx[a:b], rtol=1e-4, atol=1e-5)
        torch.testing.assert_close(got["s"], rs, rtol=1e-4, atol=1e-5)
        torch.testing.assert_close(got["dpair"], rdpair[a:b], rtol=1e-4, atol=1e-5)
        for name, g in got["grads"].items():
            torch.testing.assert_close(g, rgrads[name], rtol=1e-4, atol=1e-4, msg=name)
