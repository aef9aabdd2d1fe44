"""Token choice when the head is split over the vocabulary (tensor-parallel ranks).

Mirror of the reference's ``split_candidates`` / ``choose_merged`` (``families/qwen3_5/cuda/decode_tp.py:53-89``):
each rank takes the top ``top_k + MARGIN`` candidates of its own vocabulary slice (ids shifted to
global), every rank gathers all candidates, and the draw runs over the union — the global top-k,
ties by id included, is always inside it, so the token equals the whole-vocabulary draw.
"""

from __future__ import annotations

import torch

from . import _lib, exact_sampling
from .topk import topk_rows


def split_candidates(logits: torch.Tensor, sampling, offset: int):
    """This rank's candidates (global ids int32 [R, k], values fp32 [R, k]) from its vocabulary slice."""

    if sampling is None or sampling.temperature <= 0:
        idx, val = topk_rows(logits, 1)
    else:
        idx, val = exact_sampling.top_candidates(logits, sampling)
    return idx + offset, val


def merge_candidates(all_idx: torch.Tensor, all_val: torch.Tensor, k: int):
    """(world, R, c) candidates -> each row's best k by (value desc, id asc), as the radix top-k orders them."""

    world, rows, c = all_idx.shape
    idx = all_idx.permute(1, 0, 2).reshape(rows, world * c)
    val = all_val.permute(1, 0, 2).reshape(rows, world * c)
    # stable sorts: by id ascending, then by value descending keeps id order among equal values
    order = torch.argsort(idx, dim=1, stable=True)
    idx, val = torch.gather(idx, 1, order), torch.gather(val, 1, order)
    order = torch.argsort(val, dim=1, descending=True, stable=True)
    return torch.gather(idx, 1, order)[:, :k].contiguous(), torch.gather(val, 1, order)[:, :k].contiguous()


def choose_split(logits: torch.Tensor, positions: torch.Tensor, sampling, tp, local_vocab: int) -> torch.Tensor:
    """Every rank calls this with its slice of the logits; every rank returns the same tokens."""

    idx, val = split_candidates(logits, sampling, tp.rank * local_vocab)
    all_idx = torch.empty((tp.world, *idx.shape), dtype=idx.dtype, device=idx.device)
    all_val = torch.empty((tp.world, *val.shape), dtype=val.dtype, device=val.device)
    tp.dist.all_gather_into_tensor(all_idx.view(-1, idx.shape[1]), idx.contiguous(), group=tp.group)
    tp.dist.all_gather_into_tensor(all_val.view(-1, val.shape[1]), val.contiguous(), group=tp.group)
    k = idx.shape[1]
    midx, mval = merge_candidates(all_idx, all_val, k)
    if sampling is None or sampling.temperature <= 0:
        return midx[:, 0].contiguous()
    rows = midx.shape[0]
    tokens = torch.empty(rows, dtype=torch.int32, device=midx.device)
    with torch.cuda.device(midx.device):
        _lib.check(_lib.load().tf_sample_rows(midx.data_ptr(), mval.data_ptr(), k, positions.data_ptr(),
                                              int(sampling.seed) & 0xFFFFFFFFFFFFFFFF, float(sampling.temperature),
                                              int(sampling.top_k), float(sampling.top_p), tokens.data_ptr(), rows,
                                              _lib.stream()), "sample_rows")
    return tokens


__all__ = ["choose_split", "merge_candidates", "split_candidates"]
