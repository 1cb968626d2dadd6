"""Generate tests/golden/*.npz by running the reference's OWN PyTorch classes on CPU.

Run once, in a container that has the reference checkout:

    python tests/golden/make_golden.py /path/to/reference

The reference package cannot be imported whole here (its __init__ pulls in
biology, CLI and trainer dependencies that are not installed), so this script
  * registers empty namespace packages for ``megafold``, ``megafold.model`` and
    ``megafold.utils`` whose __path__ points into the checkout,
  * stubs the absent third-party modules that ``megafold/tensor_typing.py``
    imports but the attention math never touches (sh, environs, loguru, Bio.PDB),
  * imports ``megafold.model.attention.Attend`` (the reference's PyTorch attention),
  * lifts the class definitions ``LayernormLinear`` (whose forward falls back to
    torch for shapes outside its tuning table) and ``Transition``/``SwiGLU``
    (benchmarks/transition_speed.py) out of their source files by AST, because
    those files need a live GPU driver / Triton launch at import time.
No reference source is copied into this repository: only tensors it computed.
"""
import ast
import importlib
import math
import os
import sys
import types

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import cases  # noqa: E402

OUT = os.path.dirname(os.path.abspath(__file__))


def _stub(name, **attrs):
    m = types.ModuleType(name)
    m.__dict__.update(attrs)
    sys.modules[name] = m
    return m


class _Any:
    def __init__(self, *a, **k):
        pass

    def __call__(self, *a, **k):
        return _Any()

    def __getattr__(self, n):
        return _Any()


class _Env:
    def read_env(self, *a, **k):
        pass

    def bool(self, name, default=False):
        return default


class _ErrorReturnCode_1(Exception):
    pass


def _which(*a, **k):
    raise _ErrorReturnCode_1()


def import_reference(ref):
    _stub("sh", which=_which, ErrorReturnCode_1=_ErrorReturnCode_1)
    _stub("environs", Env=_Env)
    _stub("loguru", logger=_Any())
    _stub("Bio")
    _stub("Bio.PDB")
    _stub("Bio.PDB.Atom", Atom=_Any, DisorderedAtom=_Any)
    _stub("Bio.PDB.Chain", Chain=_Any)
    _stub("Bio.PDB.Residue", DisorderedResidue=_Any, Residue=_Any)
    for pkg, sub in (("megafold", "megafold"), ("megafold.model", "megafold/model"),
                     ("megafold.utils", "megafold/utils")):
        _stub(pkg).__path__ = [os.path.join(ref, sub)]
    return importlib.import_module("megafold.model.attention")


def lift_classes(path, names, namespace):
    """exec only the named top-level class definitions of a reference source file."""
    tree = ast.parse(open(path).read())
    body = [n for n in tree.body if isinstance(n, ast.ClassDef) and n.name in names]
    assert len(body) == len(names), (path, names)
    mod = ast.Module(body=body, type_ignores=[])
    exec(compile(mod, path, "exec"), namespace)
    return namespace


def run_attend(att, c):
    """Reference PyTorch attention (attention.py:500-539) on [B,N,L,H,D] inputs."""
    B, N, L, H, D = c["q"].shape
    attend = att.Attend()
    leaves = {n: c[n].clone().requires_grad_(True) for n in ("q", "k", "v", "bias")}
    to_bh = lambda t: t.permute(0, 1, 3, 2, 4).reshape(B * N, H, L, D)      # noqa: E731
    bias = leaves["bias"].expand(B, N, H, L, L).reshape(B * N, H, L, L)
    out = attend(to_bh(leaves["q"]), to_bh(leaves["k"]), to_bh(leaves["v"]),
                 mask=c["mask"].reshape(B * N, L), attn_bias=bias)
    out = out.reshape(B, N, H, L, D).permute(0, 1, 3, 2, 4).contiguous()
    out.backward(c["d_out"])
    return dict(o=out.detach(), dq=leaves["q"].grad, dk=leaves["k"].grad, dv=leaves["v"].grad,
                dbias=leaves["bias"].grad)


def main(ref):
    att = import_reference(ref)
    torch.set_num_threads(1)          # fixed summation order

    # --- attention -----------------------------------------------------------------
    c = cases.evo_small()
    r = run_attend(att, c)
    np.savez_compressed(os.path.join(OUT, "evo_small.npz"),
                        **{k: v.numpy() for k, v in c.items()}, **{k: v.numpy() for k, v in r.items()})
    c = cases.evo_cfg1()
    r = run_attend(att, c)
    sub = cases.CFG1_SUB
    keep = {}
    for name, t in r.items():
        keep[name + "_sub"] = t[sub].numpy()
        keep[name + "_sum"] = np.float64(t.double().sum().item())
        keep[name + "_abssum"] = np.float64(t.double().abs().sum().item())
    keep["input_sum"] = np.float64(sum(c[n].double().sum().item() for n in ("q", "k", "v", "bias", "d_out")))
    np.savez_compressed(os.path.join(OUT, "evo_cfg1.npz"), **keep)

    # --- LayernormLinear (reference class, torch fallback branch, :538-541) ---------
    helper = importlib.import_module("megafold.model.FusedLayernormLinear.helper")
    ns = dict(torch=torch, nn=torch.nn, F=torch.nn.functional, math=math,
              calculate_config_layernorm_linear=helper.calculate_config_layernorm_linear,
              LayernormLinearFunction=None)
    lift_classes(os.path.join(ref, "megafold/model/FusedLayernormLinear/fused_layernorm_linear.py"),
                 ["LayernormLinear"], ns)
    LayernormLinear = ns["LayernormLinear"]
    blob = {}
    for i, (M, N, K) in enumerate(cases.LNL_SHAPES):
        torch.manual_seed(42)
        mod = LayernormLinear(K, N)
        with torch.no_grad():            # non-trivial gamma / beta
            mod.WEIGHT.add_(0.1 * torch.randn(K))
            mod.BIAS.add_(0.1 * torch.randn(K))
        assert helper.calculate_config_layernorm_linear(M, N, K, 2) is None
        x = torch.randn(M, K, requires_grad=True)
        dy = torch.randn(M, N)
        y = mod(x)
        y.backward(dy)
        for n, t in dict(x=x, dy=dy, y=y, dx=x.grad, ln_w=mod.WEIGHT, ln_b=mod.BIAS, w=mod.linear_weight,
                         b=mod.linear_bias, d_ln_w=mod.WEIGHT.grad, d_ln_b=mod.BIAS.grad,
                         dw=mod.linear_weight.grad, db=mod.linear_bias.grad).items():
            blob[f"c{i}_{n}"] = t.detach().numpy()
    np.savez_compressed(os.path.join(OUT, "lnl.npz"), **blob)

    # --- Transition (benchmarks/transition_speed.py:8-39) ---------------------------
    ns = dict(torch=torch, nn=torch.nn)
    lift_classes(os.path.join(ref, "benchmarks/transition_speed.py"), ["Transition", "SwiGLU"], ns)
    blob = {}
    for i, (M, dim, ef) in enumerate(cases.TRANSITION_SHAPES):
        torch.manual_seed(42)
        mod = ns["Transition"](dim=dim, expansion_factor=ef)
        with torch.no_grad():
            mod.ff[0].weight.add_(0.1 * torch.randn(dim))
            mod.ff[0].bias.add_(0.1 * torch.randn(dim))
        x = torch.randn(M, dim, requires_grad=True)
        dy = torch.randn(M, dim)
        y = mod(x)
        y.backward(dy)
        for n, t in dict(x=x, dy=dy, y=y, dx=x.grad, ln_w=mod.ff[0].weight, ln_b=mod.ff[0].bias,
                         w1_lin=mod.ff[1].weight, w2=mod.ff[3].weight, d_ln_w=mod.ff[0].weight.grad,
                         d_ln_b=mod.ff[0].bias.grad, dw1_lin=mod.ff[1].weight.grad,
                         dw2=mod.ff[3].weight.grad).items():
            blob[f"c{i}_{n}"] = t.detach().numpy()
    np.savez_compressed(os.path.join(OUT, "transition.npz"), **blob)
    print("golden vectors written to", OUT)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py /path/to/reference   (the reference checkout is not looked for anywhere else)")
    main(sys.argv[1])
