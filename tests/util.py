"""Tolerance helpers shared by the GPU parity tests.

Every comparison also records the largest absolute and relative error it saw (``ERRORS``); the tests print them with
``report()`` so that a run shows how far inside the tolerance each tensor is.
"""
import torch

ERRORS = {}


def _record(what, got, ref):
    err = (got - ref).abs()
    max_abs = float(err.max()) if err.numel() else 0.0
    big = ref.abs() > 0.1 * float(ref.abs().max()) if ref.numel() else ref.abs() > 0
    max_rel = float((err[big] / ref.abs()[big]).max()) if bool(big.any()) else 0.0
    ERRORS[what] = (max_abs, max_rel)
    print(f"[parity] {what}: max_abs_err {max_abs:.3e}  max_rel_err(|ref| > 0.1 max) {max_rel:.3e}  max|ref| {float(ref.abs().max()) if ref.numel() else 0:.3e}")


def assert_close_fp32(got, ref, what=""):
    """fp32 storage: 1e-4 relative (plus 1e-5 of the tensor's scale as the absolute floor)."""
    ref = ref.to(torch.float32).cpu()
    got = got.detach().float().cpu()
    _record(what, got, ref)
    scale = max(float(ref.abs().max()), 1e-6)
    torch.testing.assert_close(got, ref, rtol=1e-4, atol=1e-5 * scale, msg=lambda m: f"{what}: {m}")


def assert_close_lowp(got, ref, what="", tol=2e-2, summed_over=1):
    """bf16 / fp16 storage against the fp32 oracle: rtol = atol = 2e-2, as stated for this operator family.

    ``summed_over``: for a gradient that is a sum over that many independent rows (d_pair_bias over the N rows, weight
    gradients over the M rows) the absolute floor grows like the random walk of the terms' rounding errors,
    ``atol = tol * sqrt(summed_over)``; every other tensor is held to the plain bound."""
    ref = ref.to(torch.float32).cpu()
    got = got.detach().float().cpu()
    _record(what, got, ref)
    torch.testing.assert_close(got, ref, rtol=tol, atol=tol * max(1.0, float(summed_over)) ** 0.5,
                               msg=lambda m: f"{what}: {m}")
