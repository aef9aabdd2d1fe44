"""Top-k over vocabulary rows, exact and deterministic: radix select on bf16 keys.

Mirror of the reference's ``engine/topk.py:130-146`` (``topk_rows``): value descending, ties to the
lower token id, k <= ``MAX_K``. A row is cut into slices (one CTA each) whose candidates a second
kernel ranks; a row's result depends on that row alone.
"""

from __future__ import annotations

import torch

from . import _lib

MAX_K = 64


def topk_rows(x: torch.Tensor, k: int, scratch: torch.Tensor | None = None) -> tuple[torch.Tensor, torch.Tensor]:
    """(indices [R, k] int32, values [R, k] float32) of each row's k largest, value desc then id asc."""

    _lib.need_cuda(x)
    if x.dtype != torch.bfloat16:
        x = x.to(torch.bfloat16)
    x2 = x.reshape(-1, x.shape[-1])
    if x2.stride(1) != 1:
        x2 = x2.contiguous()
    rows, vocab = x2.shape
    k = int(k)
    if not 1 <= k <= MAX_K or k > vocab:
        raise ValueError(f"topk_rows: k must be in [1, {MAX_K}] and at most the row length")
    idx = torch.empty((rows, k), dtype=torch.int32, device=x.device)
    val = torch.empty((rows, k), dtype=torch.float32, device=x.device)
    lib = _lib.load()
    need = lib.tf_topk_scratch_bytes(rows, vocab, k)
    if scratch is None or scratch.numel() * scratch.element_size() < need:
        scratch = torch.empty(need, dtype=torch.uint8, device=x.device)
    with torch.cuda.device(x.device):
        _lib.check(lib.tf_topk_rows(x2.data_ptr(), x2.stride(0), rows, vocab, k, idx.data_ptr(), val.data_ptr(),
                                    scratch.data_ptr(), scratch.numel() * scratch.element_size(), _lib.stream()), "topk_rows")
    return idx, val


__all__ = ["MAX_K", "topk_rows"]
