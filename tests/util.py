"""Tolerance helpers shared by the GPU parity tests."""
import torch


def assert_close_fp32(got, ref, what=""):
    """fp32 storage: 1e-4 relative (plus 1e-5 of the tensor's scale as the absolute floor)."""
    ref = ref.to(torch.float32)
    scale = max(float(ref.abs().max()), 1e-6)
    torch.testing.assert_close(got.detach().float().cpu(), ref.cpu(), rtol=1e-4, atol=1e-5 * scale,
                               msg=lambda m: f"{what}: {m}")


def assert_close_lowp(got, ref, what="", tol=2e-2):
    """bf16 / fp16 storage against the fp32 oracle: rtol = atol = 2e-2 (atol scaled by the tensor's
    largest magnitude when that exceeds 1, since sums over many rows grow with the row count)."""
    ref = ref.to(torch.float32).cpu()
    scale = max(float(ref.abs().max()), 1.0)
    torch.testing.assert_close(got.detach().float().cpu(), ref, rtol=tol, atol=tol * scale,
                               msg=lambda m: f"{what}: {m}")
