"""Tensor-parallel sharding of the dense hybrid decoder and the rank-ordered partial sum.

Mirror of the reference's partition map (``families/qwen3_5/cuda/distributed.py:32-171``): heads and
MLP width are split by whole output rows (column-parallel), the output/down projections by whole
input groups (row-parallel) and return fp32 partials; every rank then holds all ranks' partials
(all-gather) and adds them in rank order 0..n-1 with ONE rounding (``distributed.py:267-289``) — never
an all-reduce, whose summation order is the library's choice. The ordered sum is fused into the next
``norm_xs`` kernel. Unlike the reference (two ranks only) any world size dividing the head counts
works; KV heads are replicated when there are more ranks than KV heads.
"""

from __future__ import annotations

from dataclasses import replace

import torch

from .forward import Config


def shard_config(cfg: Config, rank: int, world: int) -> Config:
    """The per-rank architecture: local head counts, MLP width and vocabulary slice."""

    if world == 1:
        return cfg
    if not 0 <= rank < world:
        raise ValueError("rank outside the world")
    for name in ("heads", "k_heads", "v_heads", "intermediate", "vocab"):
        if getattr(cfg, name) % world:
            raise ValueError(f"{name}={getattr(cfg, name)} does not split over {world} ranks")
    if (cfg.intermediate // world) % 64 or (cfg.v_heads // world * 128) % 64:
        raise ValueError("row-parallel shards must be whole 64-input groups")
    if cfg.kv_heads % world and world % cfg.kv_heads:
        raise ValueError(f"kv_heads={cfg.kv_heads} neither splits over nor replicates across {world} ranks")
    kv = max(1, cfg.kv_heads // world)          # more ranks than KV heads: each head lives on world/kv_heads ranks
    if (cfg.heads // world) % kv:
        raise ValueError("local query heads must be a multiple of local KV heads")
    return replace(cfg, heads=cfg.heads // world, kv_heads=kv, k_heads=cfg.k_heads // world, v_heads=cfg.v_heads // world,
                   intermediate=cfg.intermediate // world, vocab=cfg.vocab // world)


def kv_head_of_rank(cfg: Config, rank: int, world: int) -> range:
    """Global KV heads a rank holds (a slice when they split, one replicated head otherwise)."""

    if cfg.kv_heads % world == 0:
        per = cfg.kv_heads // world
        return range(rank * per, (rank + 1) * per)
    return range(rank * cfg.kv_heads // world, rank * cfg.kv_heads // world + 1)


class RankGroup:
    """The collective a row-parallel projection needs: every rank ends up with all ranks' fp32
    partials, stacked in rank order. NCCL all-gather on the current stream (gloo on CPU in tests)."""

    def __init__(self, group=None):
        import torch.distributed as dist

        self.dist = dist
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)

    def gather_partials(self, local: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        """(M, D) fp32 -> (world, M, D) fp32, rank order."""

        if local.dtype != torch.float32 or local.dim() != 2:
            raise ValueError("local partial must be a 2-D fp32 tensor")
        if out is None:
            out = torch.empty((self.world, *local.shape), dtype=torch.float32, device=local.device)
        # the collective wants the ranks' blocks concatenated along dim 0
        self.dist.all_gather_into_tensor(out.view(-1, local.shape[1]), local.contiguous(), group=self.group)
        return out


def sum_rank_partials(partials: torch.Tensor, dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """Host-visible statement of the rule the fused kernel implements: add in rank order, round once."""

    acc = partials[0].clone()
    for p in partials[1:]:
        acc = acc + p
    return acc.to(dtype)


__all__ = ["RankGroup", "kv_head_of_rank", "shard_config", "sum_rank_partials"]
