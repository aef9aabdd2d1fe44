"""Sampling that is byte exact to serial decoding: every token a fixed function of its position.

Mirror of the reference's ``engine/exact_sampling.py`` (``Sampling``, ``uniform_rows``, ``choose_rows``,
``sample_rows``, ``MARGIN``) and of its CUDA ``sample_rows`` (``families/qwen3_5/cuda/sampling.py:13-34``).
The token at absolute position p is the argmax over the kept candidates of ``logit/T + Gumbel(hash(seed,
p, id))``: it depends only on the row's own logits and position, so a window row draws the token the
serial step at that position draws. Candidates come from the GPU radix top-k; the draw runs on the
GPU too (``tf_sample_rows``). ``choose_rows`` is the same rule on the host in numpy, used where
candidates from several vocabulary shards are merged (tensor-parallel head).
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


def _mix(x: np.ndarray) -> np.ndarray:
    x = x ^ (x >> np.uint64(30))
    x = x * np.uint64(0xBF58476D1CE4E5B9)
    x = x ^ (x >> np.uint64(27))
    x = x * np.uint64(0x94D049BB133111EB)
    return x ^ (x >> np.uint64(31))


def uniform_rows(seed: int, positions: np.ndarray, ids: np.ndarray) -> np.ndarray:
    """Uniform (0, 1) doubles from a splitmix64 hash of (seed, position, token id), one row per position."""

    with np.errstate(over="ignore"):
        x = _mix(np.uint64(seed & 0xFFFFFFFFFFFFFFFF) + np.uint64(0x9E3779B97F4A7C15))
        x = _mix(x ^ (np.asarray(positions).astype(np.uint64)[:, None] * np.uint64(0xD1B54A32D192ED03)))
        x = _mix(x ^ ids.astype(np.uint64))
    return (x >> np.uint64(11)).astype(np.float64) * 2.0 ** -53 + 2.0 ** -54


def choose_rows(values: np.ndarray, ids: np.ndarray, positions: Sequence[int], s: Sampling) -> list[int]:
    """Host form of the draw for rows of candidate (value, id) pairs in any order."""

    rows, width = ids.shape
    order = np.lexsort((ids, -values), axis=-1)
    k = max(1, min(int(s.top_k) if s.top_k else width, width))
    ids = np.take_along_axis(ids, order, axis=-1)[:, :k]
    scaled = np.take_along_axis(values, order, axis=-1)[:, :k].astype(np.float64) / max(float(s.temperature), 1e-6)
    score = scaled - np.log(-np.log(uniform_rows(s.seed, np.asarray(positions), ids)))
    if 0.0 < s.top_p < 1.0:
        probs = np.exp(scaled - scaled.max(axis=-1, keepdims=True))
        probs /= probs.sum(axis=-1, keepdims=True)
        keep = (np.cumsum(probs, axis=-1) < s.top_p).sum(axis=-1) + 1
        score[np.arange(k)[None, :] >= keep[:, None]] = -np.inf
    return [int(t) for t in ids[np.arange(rows), np.argmax(score, axis=-1)]]


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


__all__ = ["MARGIN", "Sampling", "choose_rows", "sample_rows", "top_candidates", "uniform_rows"]
