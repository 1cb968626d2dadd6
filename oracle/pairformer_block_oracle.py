"""CPU restatement of the long-crop benchmark block, unsharded and in plain torch.  TEST INFRASTRUCTURE ONLY:
nothing in the product imports this file.

Composition (benchmark configuration 5, the long-crop block): pair += TriangleAttention(starting node); pair += TriangleAttention(ending
node); pair += Transition; single += AttentionPairBias - each attention following the reference's
``Attention.forward`` (megafold/model/attention.py:158-210: q/k/v/gate projections of the normalised input, the
default branch of ``Attend.forward`` :500-539 with the pair bias added and masked keys filled with -finfo.max,
sigmoid gate, bias-free output projection) and ``TriangleAttention`` (megafold/model/megafold.py:635-648: bias
projected from the normalised pair representation, ending node = the same on the transposed representation).
Parity unpinned for the composition itself (the reference has no test vectors for a block and cannot be imported
whole); its three operators are pinned separately by the golden vectors of the operator oracle.
"""
import torch
import torch.nn.functional as F


def _attention(x, mask, bias, a, eps=1e-5):
    """x [n, L, dim]; mask bool [L]; bias [H, L, L]; a: dict of parameters of one attention."""
    n, L, C = x.shape
    H, D = a["heads"], a["dim_head"]
    xn = F.layer_norm(x, (C,), a["ln_w"], a["ln_b"], eps)
    y = xn @ a["w_qkvg"] + a["b_qkvg"]
    q, k, v, g = y.view(n, L, 4, H, D).unbind(dim=2)                 # [n, L, H, D]
    sim = torch.einsum("nihd,njhd->nhij", q * D ** -0.5, k) + bias[None]
    sim = sim.masked_fill(~mask.view(1, 1, 1, L), -torch.finfo(sim.dtype).max)
    o = torch.einsum("nhij,njhd->nihd", sim.softmax(dim=-1), v).reshape(n, L, H * D)
    return (o * torch.sigmoid(g.reshape(n, L, H * D))) @ a["w_out"].T


def _pair_bias(pair, a, eps=1e-5):
    xn = F.layer_norm(pair, (pair.shape[-1],), a["pair_ln_w"], a["pair_ln_b"], eps)
    return (xn @ a["w_pair_bias"])[..., : a["heads"]].permute(2, 0, 1)   # [H, L, L]; columns beyond H are padding


def _transition(x, t, eps=1e-5):
    h = F.layer_norm(x, (x.shape[-1],), t["ln_w"], t["ln_b"], eps) @ t["w1"]
    a, b = h.chunk(2, dim=-1)
    return (F.silu(b) * a) @ t["w2"].T


def block(pair, single, mask, params):
    """pair [L, L, C], single [L, Cs], mask bool [L]; params = {"tri_start", "tri_end", "single_attn": attention
    dicts, "transition": dict}.  Returns (pair, single)."""
    x = pair
    x = x + _attention(x, mask, _pair_bias(x, params["tri_start"]), params["tri_start"])
    xt = x.transpose(0, 1)
    x = x + _attention(xt, mask, _pair_bias(xt, params["tri_end"]), params["tri_end"]).transpose(0, 1)
    x = x + _transition(x, params["transition"])
    s = single + _attention(single[None], mask, _pair_bias(x, params["single_attn"]), params["single_attn"])[0]
    return x, s


def params_of(module, device="cpu"):
    """The parameter dictionaries of a ``megafold_b200.pairformer_block.PairformerBlock`` as fp32 leaf tensors on
    ``device`` (the fp32 block is evaluated on the GPU for the benchmark-sized test, on the host otherwise)."""
    def attn(a):
        d = {k: getattr(a, k).detach().float().to(device).clone().requires_grad_(True)
             for k in ("ln_w", "ln_b", "w_qkvg", "b_qkvg", "pair_ln_w", "pair_ln_b", "w_pair_bias", "w_out")}
        d["heads"], d["dim_head"] = a.heads, a.dim_head
        return d
    tr = {k: getattr(module, "tr_" + k).detach().float().to(device).clone().requires_grad_(True) for k in ("ln_w", "ln_b", "w1", "w2")}
    return {"tri_start": attn(module.tri_start), "tri_end": attn(module.tri_end), "single_attn": attn(module.single_attn),
            "transition": tr}
