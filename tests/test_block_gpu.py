"""The Pairformer block of the long-crop configuration on the CUDA operators (one GPU) against the plain-torch block."""
import pytest
import torch

from megafold_b200.pairformer_block import PairformerBlock
from oracle import pairformer_block_oracle as blk
from util import assert_close_lowp

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("L", [64, 200])
def test_block_bf16_matches_plain_torch_block(L):
    torch.manual_seed(3)
    dev, dt = "cuda", torch.bfloat16
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

    params = blk.params_of(m)
    rp = pair.float().requires_grad_(True)
    rsg = single.float().requires_grad_(True)
    rx, rs = blk.block(rp, rsg, mask, params)
    torch.autograd.backward([rx, rs], [d_pair.float(), d_single.float()])
    assert_close_lowp(x, rx.detach(), "pair out")
    assert_close_lowp(s, rs.detach(), "single out")
    assert_close_lowp(rows.grad, rp.grad, "d pair")
    assert_close_lowp(sg.grad, rsg.grad, "d single")
    # Parameter gradients are sums over up to L*L rows of 16-bit-rounded terms that largely cancel (some are zero in
    # exact arithmetic: a LayerNorm shift in front of the bias projection moves every logit of a head alike), so they
    # are held to 3e-2 of the gradient's norm plus 0.05 per element (RMS) rather than element by element.
    for name, p in m.named_parameters():
        head, _, leaf = name.partition(".")
        ref = params["transition"][name[3:]].grad if name.startswith("tr_") else params[head][leaf].grad
        err = (p.grad.float().cpu() - ref).norm()
        assert err <= 3e-2 * ref.norm() + 0.05 * ref.numel() ** 0.5, f"{name}: error norm {float(err):.3g} vs {float(ref.norm()):.3g}"
