"""Shared checks for the parity tests."""

from __future__ import annotations

import torch

# tolerance the path states for bf16 outputs against the reference arithmetic
REL, ABS = 1e-2, 1e-3


def bits(t: torch.Tensor) -> torch.Tensor:
    """Raw bits of a bf16/fp32 tensor, for exact comparison (NaN-safe, -0 != +0)."""

    if t.dtype == torch.bfloat16:
        return t.contiguous().view(torch.int16)
    if t.dtype == torch.float32:
        return t.contiguous().view(torch.int32)
    return t


def assert_same_bits(a: torch.Tensor, b: torch.Tensor, what: str = "") -> None:
    assert a.shape == b.shape and a.dtype == b.dtype, f"{what}: {a.shape}/{a.dtype} vs {b.shape}/{b.dtype}"
    diff = bits(a) != bits(b)
    assert not bool(diff.any()), f"{what}: {int(diff.sum())} of {diff.numel()} elements differ in bits"


def assert_close(got: torch.Tensor, want: torch.Tensor, what: str = "", rel: float = REL, abs_: float = ABS) -> None:
    """|got - want| <= abs + rel * |want| elementwise (the path's stated bf16 tolerance)."""

    g, w = got.float().cpu(), want.float().cpu()
    err = (g - w).abs()
    bound = abs_ + rel * w.abs()
    bad = err > bound
    assert not bool(bad.any()), (f"{what}: {int(bad.sum())} of {bad.numel()} outside rel {rel} / abs {abs_}; "
                                 f"worst err {float(err.max()):.4g} at want {float(w.flatten()[err.argmax()]):.4g}")
