"""Sampling that is byte exact to serial decoding: every token a fixed function of its position.

Mirror of the reference's ``engine/exact_sampling.py`` (``Sampling``, ``uniform_rows``, ``choose_rows``,
``sample_rows``, ``MARGIN``) and of its CUDA ``sample_rows`` (``families/qwen3_5/cuda/sampling.py:13-34``).
The token at absolute position p is the argmax over the kept candidates of ``logit/T + Gumbel(hash(seed,
p, id))``: it depends only on the row's own logits and position, so a window row draws the token the
serial step at that position draws. Candidates come from the GPU radix top-k; the draw runs on the
GPU too (``tf_sample_rows``); ``choose_rows`` takes candidates in any order (merged vocabulary shards of a
tensor-parallel head) and draws with the same kernel; there is no host-side draw in this package.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Sequence

import numpy as np
import torch

from . import _lib
from .topk import MAX_K, topk_rows

MARGIN = 8     # candidates beyond top_k read from the top-k kernel, so tied values resolve by id


@dataclass(frozen=True)
class Sampling:
    seed: int
    temperature: float = 1.0
    top_k: int = 20
    top_p: float = 0.95


def choose_rows(values, ids, positions: Sequence[int], s: Sampling) -> list[int]:
    """The draw for rows of candidate (value, id) pairs in any order (reference:
    ``exact_sampling.choose_rows``), run on the GPU: the candidates are put in the order the radix top-k
    writes them, (value descending, id ascending), and handed to the keyed draw kernel."""

    dev = torch.device("cuda")
    val = torch.as_tensor(np.asarray(values), dtype=torch.float32).to(dev)
    idx = torch.as_tensor(np.asarray(ids).astype(np.int32)).to(dev)
    rows, width = idx.shape
    by_id = torch.argsort(idx, dim=-1, stable=True)
    by_val = torch.argsort(torch.gather(val, 1, by_id), dim=-1, descending=True, stable=True)
    order = torch.gather(by_id, 1, by_val)
    idx, val = torch.gather(idx, 1, order).contiguous(), torch.gather(val, 1, order).contiguous()
    pos = torch.as_tensor(list(positions), dtype=torch.int64).to(dev)
    tokens = torch.empty(rows, dtype=torch.int32, device=dev)
    k = max(1, min(int(s.top_k) if s.top_k else width, width))
    with torch.cuda.device(dev):
        _lib.check(_lib.load().tf_sample_rows(idx.data_ptr(), val.data_ptr(), width, pos.data_ptr(), int(s.seed) & 0xFFFFFFFFFFFFFFFF,
                                              max(float(s.temperature), 1e-6), k, float(s.top_p), tokens.data_ptr(), rows,
                                              _lib.stream()), "choose_rows")
    return [int(t) for t in tokens.cpu()]


def top_candidates(logits: torch.Tensor, s: Sampling) -> tuple[torch.Tensor, torch.Tensor]:
    """The rows' top ``top_k + MARGIN`` (ids, values), ordered by (value desc, id asc)."""

    vocab = logits.shape[-1]
    count = min(vocab, (int(s.top_k) if s.top_k else MAX_K - MARGIN) + MARGIN, MAX_K)
    return topk_rows(logits.reshape(-1, vocab), count)


def sample_rows(logits: torch.Tensor, positions, s: Sampling | None, *, top: tuple | None = None) -> torch.Tensor:
    """Rows of ``logits`` [W, V] bf16 at absolute ``positions`` -> one token each (int32 on the device).

    Greedy (``s`` None or temperature <= 0) is the first maximum. ``positions``: int64 tensor or a list.
    """

    _lib.need_cuda(logits)
    rows = logits.shape[0]
    if s is None or s.temperature <= 0:
        return topk_rows(logits, 1)[0].reshape(rows)
    if not 0 < int(s.top_k) <= MAX_K - MARGIN:
        raise ValueError(f"sample_rows: top_k must be in 1..{MAX_K - MARGIN} (the radix top-k holds {MAX_K} candidates)")
    idx, val = top if top is not None else top_candidates(logits, s)
    if not torch.is_tensor(positions):
        positions = torch.tensor(list(positions), dtype=torch.int64)
    positions = positions.to(device=logits.device, dtype=torch.int64)
    if positions.shape != (rows,):
        raise ValueError("sample_rows: one position per row")
    tokens = torch.empty(rows, dtype=torch.int32, device=logits.device)
    with torch.cuda.device(logits.device):
        _lib.check(_lib.load().tf_sample_rows(idx.data_ptr(), val.data_ptr(), idx.shape[1], positions.data_ptr(),
                                              int(s.seed) & 0xFFFFFFFFFFFFFFFF, float(s.temperature), int(s.top_k),
                                              float(s.top_p), tokens.data_ptr(), rows, _lib.stream()), "sample_rows")
    return tokens


__all__ = ["MARGIN", "Sampling", "choose_rows", "sample_rows", "top_candidates"]
