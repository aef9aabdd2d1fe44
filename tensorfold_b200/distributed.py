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
from types import SimpleNamespace

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
    """The exchange a row-parallel projection needs: every rank ends up with all ranks' fp32 partials,
    stacked in rank order.

    ``exchange="peer"`` (GPUs): the library's own kernel stores the partial into every rank's buffer in
    symmetric memory over NVLink and the ranks signal one another through flag words
    (``tf_peer_exchange``) - a few microseconds per exchange, capturable in a CUDA graph as an ordinary
    kernel. ``exchange="nccl"``: ``all_gather_into_tensor`` on the current stream (gloo on CPU in
    tests). Never an all-reduce: the sum is done in rank order by the consuming kernel."""

    def __init__(self, group=None, exchange: str = "nccl", max_rows: int = 128, hidden: int = 0, device=None,
                 fused: bool = False):
        import torch.distributed as dist

        self.dist = dist
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.exchange = exchange
        self.count = 0                      # exchanges issued so far (slots alternate)
        self.fuse = bool(fused)
        if exchange == "peer":
            import os

            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")     # plain peer stores only
            import torch.distributed._symmetric_memory as symm_mem

            if hidden <= 0 or device is None:
                raise ValueError("peer exchange needs the hidden size and the device")
            from . import _lib

            self.slot_bytes = (_lib.load().tf_peer_slot_bytes(max_rows, hidden, self.world) + 255) // 256 * 256
            self.buf = symm_mem.empty(2 * self.slot_bytes, dtype=torch.uint8, device=device)
            self.buf.zero_()
            self.handle = symm_mem.rendezvous(self.buf, group=group if group is not None else dist.group.WORLD)
            self.state = torch.zeros(2, dtype=torch.int32, device=device)       # exchange number, CTA tickets
            torch.cuda.synchronize(device)
            dist.barrier(group)
        elif exchange != "nccl":
            raise ValueError("exchange must be 'peer' or 'nccl'")

    def check_settings(self, settings: dict) -> None:
        """Refuse to start when the ranks were given different settings: every rank must issue the same
        kernels and exchanges in the same order (reference: ``families/qwen3_5/cuda/engine.py:54-62``). The
        settings travel as one int64 digest per key, gathered by the group's collective."""

        import hashlib

        keys = sorted(settings)
        mine = torch.tensor([int.from_bytes(hashlib.sha256(f"{k}={settings[k]!r}".encode()).digest()[:7], "big") for k in keys] +
                            [int.from_bytes(hashlib.sha256(",".join(keys).encode()).digest()[:7], "big")], dtype=torch.int64)
        dev = self.state.device if self.exchange == "peer" else (torch.device("cuda", torch.cuda.current_device())
                                                                 if self.dist.get_backend(self.group) == "nccl" else torch.device("cpu"))
        mine = mine.to(dev)
        everyone = torch.empty(self.world * mine.numel(), dtype=torch.int64, device=dev)
        self.dist.all_gather_into_tensor(everyone, mine, group=self.group)
        everyone = everyone.cpu().reshape(self.world, -1)
        for r in range(self.world):
            if not torch.equal(everyone[r], everyone[0]):
                diff = [k for i, k in enumerate(keys) if everyone[r, i] != everyone[0, i]] or ["the set of settings"]
                raise RuntimeError(f"ranks were started with different settings: rank {r} differs from rank 0 in {diff}; "
                                   "every rank must run the same calls in the same order")

    @property
    def fused(self) -> bool:
        """Whether the exchange rides inside the row-parallel matmul's epilogue and the next norm kernel
        (``tf_qmm_peer`` / ``tf_norm_xs_peer``) instead of being a step of its own."""

        return self.exchange == "peer" and self.fuse

    def peer_args(self):
        """(buffer pointer table, slot bytes, exchange-number word, ticket word, this rank's buffer) for the fused form."""

        return (self.handle.buffer_ptrs_dev, self.slot_bytes, self.state[0:1].data_ptr(), self.state[1:2].data_ptr(),
                self.buf.data_ptr())

    def gather_partials(self, local: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        """(M, D) fp32 -> (world, M, D) fp32, rank order."""

        if local.dtype != torch.float32 or local.dim() != 2:
            raise ValueError("local partial must be a 2-D fp32 tensor")
        if self.exchange == "peer":
            from . import _lib

            m, d = local.shape
            lib = _lib.load()
            if lib.tf_peer_slot_bytes(m, d, self.world) > self.slot_bytes:
                raise ValueError("partial larger than the exchange buffer")
            self.count += 1
            local = local.contiguous()
            if out is None:
                out = torch.empty((self.world, m, d), dtype=torch.float32, device=local.device)
            with torch.cuda.device(local.device):
                _lib.check(lib.tf_peer_exchange(local.data_ptr(), m, d, self.handle.buffer_ptrs_dev, self.slot_bytes, out.data_ptr(), self.rank,
                                                self.world, self.state[0:1].data_ptr(), self.state[1:2].data_ptr(),
                                                _lib.status(local.device).word.data_ptr(), _lib.stream()), "peer exchange")
            return out
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


def split_output(q, r0: int, r1: int):
    """Column-parallel shard of a stored 4-bit projection: whole output rows r0..r1 (packed rows are
    never cut, so nothing is repacked). Reference: ``distributed.py:32-60`` (``split_output``)."""

    return SimpleNamespace(words=q.words[r0:r1].contiguous(), scales=q.scales[r0:r1].contiguous(),
                           biases=q.biases[r0:r1].contiguous())


def split_input(q, c0: int, c1: int, group: int = 64):
    """Row-parallel shard: inputs c0..c1, whole groups (words ``[:, c0/8:c1/8]``, scales and biases
    ``[:, c0/group:c1/group]``). Reference: ``distributed.py:62-98`` (``split_input``)."""

    if c0 % group or c1 % group:
        raise ValueError("row-parallel shards must be whole input groups")
    return SimpleNamespace(words=q.words[:, c0 // 8:c1 // 8].contiguous(), scales=q.scales[:, c0 // group:c1 // group].contiguous(),
                           biases=q.biases[:, c0 // group:c1 // group].contiguous())


def _cat(parts):
    return SimpleNamespace(words=torch.cat([p.words for p in parts]), scales=torch.cat([p.scales for p in parts]),
                           biases=torch.cat([p.biases for p in parts]))


def split_model(model: dict, rank: int, world: int) -> dict:
    """The tensor-parallel shard of a stored model (the dict ``forward.load_weights`` reads): heads and
    MLP width by output rows, output/down projections by input groups, vocabulary rows for the head;
    norms and the embedding are replicated. Reference: ``distributed.py:100-171`` (``split_layer``,
    ``split_weights``)."""

    cfg = model["config"]
    if world == 1:
        return model
    sc = shard_config(cfg, rank, world)
    g = cfg.group
    kd, vd = cfg.k_heads * cfg.dk, cfg.v_heads * cfg.dv
    kdl, vdl = sc.k_heads * cfg.dk, sc.v_heads * cfg.dv
    il = sc.intermediate
    kv0 = kv_head_of_rank(cfg, rank, world).start
    hd = cfg.head_dim
    layers = []
    for src in model["layers"]:
        out = {"linear": src["linear"], "input_norm": src["input_norm"], "post_norm": src["post_norm"],
               "gate": split_output(src["gate"], rank * il, (rank + 1) * il), "up": split_output(src["up"], rank * il, (rank + 1) * il),
               "down": split_input(src["down"], rank * il, (rank + 1) * il, g)}
        if src["linear"]:
            def seg(t):
                return (t[rank * kdl:(rank + 1) * kdl], t[kd + rank * kdl:kd + (rank + 1) * kdl],
                        t[2 * kd + rank * vdl:2 * kd + (rank + 1) * vdl])
            qkv = src["qkv"]
            out["qkv"] = _cat([split_output(qkv, rank * kdl, (rank + 1) * kdl), split_output(qkv, kd + rank * kdl, kd + (rank + 1) * kdl),
                               split_output(qkv, 2 * kd + rank * vdl, 2 * kd + (rank + 1) * vdl)])
            out["z"] = split_output(src["z"], rank * vdl, (rank + 1) * vdl)
            out["b"] = split_output(src["b"], rank * sc.v_heads, (rank + 1) * sc.v_heads)
            out["a"] = split_output(src["a"], rank * sc.v_heads, (rank + 1) * sc.v_heads)
            out["out"] = split_input(src["out"], rank * vdl, (rank + 1) * vdl, g)
            out["conv"] = torch.cat(seg(src["conv"]))
            out["A_log"] = src["A_log"][rank * sc.v_heads:(rank + 1) * sc.v_heads]
            out["dt_bias"] = src["dt_bias"][rank * sc.v_heads:(rank + 1) * sc.v_heads]
            out["norm"] = src["norm"]
        else:
            h0, h1 = rank * sc.heads, (rank + 1) * sc.heads
            out["q"] = split_output(src["q"], h0 * 2 * hd, h1 * 2 * hd)            # per-head [q_h ; gate_h] blocks
            out["k"] = split_output(src["k"], kv0 * hd, (kv0 + sc.kv_heads) * hd)
            out["v"] = split_output(src["v"], kv0 * hd, (kv0 + sc.kv_heads) * hd)
            out["o"] = split_input(src["o"], h0 * hd, h1 * hd, g)
            out["q_norm"], out["k_norm"] = src["q_norm"], src["k_norm"]
        layers.append(out)
    vl = sc.vocab
    return {"config": sc, "layers": layers, "embed": model["embed"], "norm": model["norm"],
            "head": split_output(model["head"], rank * vl, (rank + 1) * vl)}


__all__ = ["RankGroup", "kv_head_of_rank", "shard_config", "split_input", "split_model", "split_output", "sum_rank_partials"]
