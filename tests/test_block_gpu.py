"""The Pairformer block of the long-crop configuration on the CUDA operators (one GPU) against the plain-torch block."""
import pytest
import torch

from megafold_b200.pairformer_block import PairformerBlock
from oracle import pairformer_block_oracle as blk
from util import assert_close_lowp

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("L", [64, 200, 768])
def test_block_bf16_matches_plain_torch_block(L):
    """L = 768 is the benchmark's size: the plain-torch fp32 block is then evaluated on the GPU with TF32 off (minutes on
    host cores), the small sizes on the host."""
    torch.manual_seed(3)
    dev, dt = "cuda", torch.bfloat16
    odev = "cuda" if L > 256 else "cpu"
    tf32 = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    m = PairformerBlock(device=dev, dtype=dt)
    g = torch.Generator().manual_seed(L)
    pair = torch.randn(L, L, 128, generator=g).to(dt)
    single = torch.randn(L, 384, generator=g).to(dt)
    mask = torch.ones(L, dtype=torch.bool)
    mask[-max(1, L // 20):] = False
    d_pair = (torch.randn(L, L, 128, generator=g) / 4).to(dt)
    d_single = (torch.randn(L, 384, generator=g) / 4).to(dt)

    rows = pair.to(dev).requires_grad_(True)
    sg = single.to(dev).requires_grad_(True)
    x, s = m(rows, sg, mask.to(dev))
    torch.autograd.backward([x, s], [d_pair.to(dev), d_single.to(dev)])
    torch.cuda.synchronize()

    params = blk.params_of(m, device=odev)
    rp = pair.float().to(odev).requires_grad_(True)
    rsg = single.float().to(odev).requires_grad_(True)
    rx, rs = blk.block(rp, rsg, mask.to(odev), params)
    torch.autograd.backward([rx, rs], [d_pair.float().to(odev), d_single.float().to(odev)])
    torch.backends.cuda.matmul.allow_tf32 = tf32
    # The block chains four 16-bit operators, each within 2e-2 of its own oracle, through three residual additions that
    # are themselves rounded to bf16: the absolute floor of the block's outputs is that of four accumulated errors.
    assert_close_lowp(x, rx.detach(), f"block L={L} pair out", summed_over=4)
    assert_close_lowp(s, rs.detach(), f"block L={L} single out", summed_over=4)
    assert_close_lowp(rows.grad, rp.grad, f"block L={L} d pair", summed_over=4)
    # d single sums the bias-projection gradient over the L rows of the pair representation
    assert_close_lowp(sg.grad, rsg.grad, f"block L={L} d single", summed_over=L)
    # Parameter gradients are sums over up to L*L rows of 16-bit-rounded terms that largely cancel (some are zero in
    # exact arithmetic: a LayerNorm shift in front of the bias projection moves every logit of a head alike), so they
    # are held to 3e-2 of the gradient's norm plus 0.05 per element (RMS) rather than element by element.
    for name, p in m.named_parameters():
        head, _, leaf = name.partition(".")
        ref = params["transition"][name[3:]].grad if name.startswith("tr_") else params[head][leaf].grad
        err = (p.grad.float().cpu() - ref.cpu()).norm()
        ref = ref.cpu()
        assert err <= 3e-2 * ref.norm() + 0.05 * ref.numel() ** 0.5, f"{name}: error norm {float(err):.3g} vs {float(ref.norm()):.3g}"


def _nccl_worker(rank, world, port, L, out):
    import os
    import torch.distributed as dist
    from megafold_b200 import row_shard
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        torch.manual_seed(3)
        m = PairformerBlock(device=dev, dtype=torch.bfloat16)
        g = torch.Generator().manual_seed(L)
        pair = torch.randn(L, L, 128, generator=g).to(torch.bfloat16)
        single = torch.randn(L, 384, generator=g).to(torch.bfloat16)
        mask = torch.ones(L, dtype=torch.bool)
        mask[-3:] = False
        d_pair = (torch.randn(L, L, 128, generator=g) / 4).to(torch.bfloat16)
        d_single = (torch.randn(L, 384, generator=g) / 4).to(torch.bfloat16)
        a, b = row_shard(L, rank, world)
        rows = pair[a:b].to(dev).requires_grad_(True)
        sg = single.to(dev).requires_grad_(True)
        x, s = m(rows, sg, mask.to(dev))
        torch.autograd.backward([x, s], [d_pair[a:b].to(dev), d_single.to(dev)])
        torch.cuda.synchronize()
        torch.save(dict(x=x.detach().cpu(), s=s.detach().cpu(), dpair=rows.grad.cpu(), dsingle=sg.grad.cpu(), span=(a, b)),
                   f"{out}/r{rank}.pt")
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_block_sharded_over_two_gpus_matches_one_gpu(tmp_path):
    """Rows of the pair representation over two GPUs (NCCL all-gather, all-to-all, all-reduce) against the same block on
    one GPU: outputs and input gradients of every row."""
    import os
    import torch.multiprocessing as mp
    L = 160
    torch.manual_seed(3)
    dev = "cuda"
    m = PairformerBlock(device=dev, dtype=torch.bfloat16)
    g = torch.Generator().manual_seed(L)
    pair = torch.randn(L, L, 128, generator=g).to(torch.bfloat16)
    single = torch.randn(L, 384, generator=g).to(torch.bfloat16)
    mask = torch.ones(L, dtype=torch.bool)
    mask[-3:] = False
    d_pair = (torch.randn(L, L, 128, generator=g) / 4).to(torch.bfloat16)
    d_single = (torch.randn(L, 384, generator=g) / 4).to(torch.bfloat16)
    rows = pair.to(dev).requires_grad_(True)
    sg = single.to(dev).requires_grad_(True)
    x, s = m(rows, sg, mask.to(dev))
    torch.autograd.backward([x, s], [d_pair.to(dev), d_single.to(dev)])
    torch.cuda.synchronize()
    port = 32500 + os.getpid() % 2000
    mp.spawn(_nccl_worker, args=(2, port, L, str(tmp_path)), nprocs=2, join=True)
    for r in range(2):
        got = torch.load(os.path.join(tmp_path, f"r{r}.pt"))
        a, b = got["span"]
        assert_close_lowp(got["x"], x[a:b].detach().float().cpu(), f"pair out rank {r}")
        assert_close_lowp(got["s"], s.detach().float().cpu(), f"single out rank {r}")
        assert_close_lowp(got["dpair"], rows.grad[a:b].float().cpu(), f"d pair rank {r}")
    # the single-track gradient is complete on every rank only for its own path; the contribution through the pair bias of the
    # single attention flows into the pair rows, so d single is identical on both ranks and equals the one-GPU value
    got0 = torch.load(os.path.join(tmp_path, "r0.pt"))
    assert_close_lowp(got0["dsingle"], sg.grad.float().cpu(), "d single")
