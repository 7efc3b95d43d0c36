"""Helpers for the GPU parity tests: the package import (fails loudly if the C-ABI library is
missing on a GPU box) and seeded input makers."""
import torch


def ops():
    import ramnet_ops  # noqa: F401  (registers torch.ops.ramnet_ops.*)
    import ramnet_ops._C as C
    return C


def randn(shape, seed, dtype=torch.float32, std=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * std).to(dtype)


def quantised(t, dtype):
    """Round to the low-precision dtype and return (low, fp32 copy of the same values)."""
    low = t.to(dtype)
    return low, low.to(torch.float32)
