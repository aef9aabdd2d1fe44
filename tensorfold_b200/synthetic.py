"""Random-initialised weights of the dense hybrid architecture, generated on the device.

For benchmarks and large-shape tests, where no checkpoint exists: packed 4-bit words are uniform
random, scales are positive and small with biases = -7.5 * scales (codes centred on zero), norm
weights near one — the recipe the reference's own forward tests use
(``tests/cuda/test_flashnext_forward.py:35-53``), scaled by 1/sqrt(K) so activations stay O(1)
through many layers.
"""

from __future__ import annotations

import torch

from .forward import Config, LayerWeights, Weights
from .lane_moe import Experts
from .lane_qmm import QWeight, tile_weight


def random_q4(gen: torch.Generator, n: int, k: int, group: int, device, spread: float = 1.0) -> QWeight:
    words = torch.randint(-2 ** 31, 2 ** 31 - 1, (n, k // 8), generator=gen, dtype=torch.int64, device=device).to(torch.int32)
    s = (torch.rand((n, k // group), generator=gen, device=device) / 8 + 1 / 64) * (spread * 4.0 / k ** 0.5)
    scales = s.to(torch.bfloat16)
    biases = (-7.5 * scales.float()).to(torch.bfloat16)
    return tile_weight(words, scales, biases, group)


def random_weights(cfg: Config, seed: int = 0, device="cuda", rank: int = 0, world: int = 1, expert_ids=None) -> Weights:
    """Weights of ``cfg`` from ``seed``; with ``world`` > 1, the tensor-parallel shard of ``rank``
    (heads and MLP width split; see ``distributed.shard_config``). ``expert_ids``: for expert
    parallelism, the global ids of the experts to create (``ExpertGroup.local_experts``); an expert's
    weights depend on (seed, layer, id) only, so every world size sees the same experts."""

    from .distributed import shard_config

    gen = torch.Generator(device=device).manual_seed(seed * 1000 + rank)
    sc = shard_config(cfg, rank, world)
    g = cfg.group
    bf = torch.bfloat16

    def norm(n):
        # replicated tensors must be identical on every rank: draw them from a rank-independent stream
        return (1 + 0.05 * torch.randn(n, generator=rgen, device=device)).to(bf)

    rgen = torch.Generator(device=device).manual_seed(seed * 1000 + 999)
    kd, vd = sc.k_heads * 128, sc.v_heads * 128
    layers = []
    for i in range(cfg.layers):
        linear = cfg.is_linear(i)
        inorm, pnorm = norm(cfg.hidden), norm(cfg.hidden)
        extra = {}
        if cfg.experts:
            ne = cfg.experts + (1 if cfg.shared_expert else 0)
            gate_up = down = None
            ids = list(range(ne)) if expert_ids is None else list(expert_ids)
            gu, dn = [], []
            egen = torch.Generator(device=device)
            for e in ids:
                egen.manual_seed((seed * 1000 + i) * 4096 + e + 1)
                gu.append(random_q4(egen, 2 * cfg.moe_intermediate, cfg.hidden, g, device).tiled)
                dn.append(random_q4(egen, cfg.hidden, cfg.moe_intermediate, g, device).tiled)
            extra = dict(router=(0.05 * torch.randn((ne, cfg.hidden), generator=rgen, device=device)).to(bf),
                         experts=Experts(torch.cat(gu), torch.cat(dn), len(ids), cfg.hidden, cfg.moe_intermediate, g))
        else:
            gate_up = random_q4(gen, 2 * sc.intermediate, cfg.hidden, g, device)
            down = random_q4(gen, cfg.hidden, sc.intermediate, g, device)
        if linear:
            lw = LayerWeights(True, inorm, pnorm, random_q4(gen, -(-(2 * kd + 2 * vd + 2 * sc.v_heads) // 8) * 8, cfg.hidden, g, device),
                              random_q4(gen, cfg.hidden, vd, g, device), gate_up, down,
                              conv=(0.3 * torch.randn((2 * kd + vd, 4), generator=gen, device=device)).to(bf),
                              A_log=0.5 * torch.randn(sc.v_heads, generator=gen, device=device),
                              dt_bias=0.5 * torch.randn(sc.v_heads, generator=gen, device=device), norm=norm(128), **extra)
        else:
            nq = sc.heads * 2 * cfg.head_dim + 2 * sc.kv_heads * cfg.head_dim
            lw = LayerWeights(False, inorm, pnorm, random_q4(gen, nq, cfg.hidden, g, device),
                              random_q4(gen, cfg.hidden, sc.heads * cfg.head_dim, g, device), gate_up, down,
                              q_norm=norm(cfg.head_dim), k_norm=norm(cfg.head_dim), **extra)
        layers.append(lw)
    words = torch.randint(-2 ** 31, 2 ** 31 - 1, (cfg.vocab, cfg.hidden // 8), generator=rgen, dtype=torch.int64, device=device).to(torch.int32)
    s = ((torch.rand((cfg.vocab, cfg.hidden // g), generator=rgen, device=device) / 8 + 1 / 64) * 0.5).to(bf)
    embed = (words, s, (-7.5 * s.float()).to(bf))
    head = random_q4(gen, sc.vocab, cfg.hidden, g, device)
    return Weights(sc, embed, layers, norm(cfg.hidden), head, cfg.inv_freq().to(device))


MOE_30B = dict(hidden=2048, intermediate=0, layers=48, heads=16, kv_heads=2, head_dim=256, vocab=151936, k_heads=16, v_heads=32,
               dk=128, dv=128, conv_kernel=4, interval=4, eps=1e-6, rope_dims=64, rope_theta=1e7, group=32, experts=128, top_k=8,
               moe_intermediate=768, shared_expert=True)

DENSE_27B = dict(hidden=5120, intermediate=17408, layers=64, heads=24, kv_heads=4, head_dim=256, vocab=248320, k_heads=16,
                 v_heads=32, dk=128, dv=128, conv_kernel=4, interval=4, eps=1e-6, rope_dims=64, rope_theta=1e7, group=64)


__all__ = ["DENSE_27B", "MOE_30B", "random_q4", "random_weights"]
