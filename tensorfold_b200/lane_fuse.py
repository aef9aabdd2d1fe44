"""Stacked projections: several 4-bit projections of the same input as ONE lane matmul, and the glue
kernels that read the stacked output in place.

Host-side mirror of the reference's ``lane_fuse`` (``kernels/qwen/dense/v1/lane_fuse.py:202-260`` ``gdn_in`` /
``attn_kv`` / ``mlp_gate_up`` / ``build`` / ``clear`` / ``stats``, ``:318-372`` ``gdn_pre`` / ``gdn_post`` /
``mlp_act`` on the stacked rows; CUDA ``qmm_fast.stack``). Same names and meaning:

* ``build(model)`` stacks, for every layer of a stored model (the dict ``forward.load_weights`` reads), the
  groups it finds: ``zba`` = [z | b | a] of a gated-DeltaNet layer, ``kv`` = [k | v] of an attention layer,
  ``gu`` = [gate | up] of an MLP, and returns {kind: groups stacked};
* ``gdn_in(layer, x)``, ``attn_kv(layer, x)``, ``mlp_gate_up(layer, x)`` run the group's one matmul and
  return the stacked rows, or None when the layer has no such stack (the caller then projects member by
  member, as the reference's callers do);
* ``gdn_pre`` / ``gdn_post`` / ``mlp_act`` take the stacked rows and read their members as column views,
  so nothing is copied apart.

The reference stacks only when the members' ``split_k`` agree, because its K schedule is per member; here
the schedule is a function of the stack's own shape, so a stack is always valid and a row of the stacked
matmul has the bits of that row alone (not of the unstacked members: those are different weights to this
library). The verify forward (``forward.load_weights``) stacks further, [qkv | z | b | a] and [q | k | v].
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from . import lane_glue
from .lane_qmm import Packed, QWeight, lane_matmul, tile_weight

GROUPS = {"zba": ("z", "b", "a"), "kv": ("k", "v"), "gu": ("gate", "up")}


@dataclass
class _Group:
    weight: QWeight
    sizes: tuple            # output rows of each member, in order
    added: int              # bytes the stack holds beyond its members (tile padding)


_stacks: dict[int, dict[str, _Group]] = {}


def _stack(layer: dict, kind: str, device, group: int) -> _Group:
    parts = [layer[name] for name in GROUPS[kind]]
    words = torch.cat([p.words for p in parts]).to(device).contiguous()
    scales = torch.cat([p.scales for p in parts]).to(device).contiguous()
    biases = torch.cat([p.biases for p in parts]).to(device).contiguous()
    q = tile_weight(words, scales, biases, group)
    plain = sum(p.words.numel() * 4 + p.scales.numel() * 2 + p.biases.numel() * 2 for p in parts)
    return _Group(q, tuple(int(p.words.shape[0]) for p in parts), q.nbytes() - plain)


def build(model: dict, device="cuda") -> dict[str, int]:
    """Stack every group of ``model`` now: {kind: groups stacked}."""

    group = getattr(model["config"], "group", 64)
    counts = {kind: 0 for kind in GROUPS}
    for layer in model["layers"]:
        for kind, names in GROUPS.items():
            if all(name in layer for name in names):
                _stacks.setdefault(id(layer), {})[kind] = _stack(layer, kind, device, group)
                counts[kind] += 1
    return counts


def clear(model: dict) -> None:
    """Drop every stack of ``model``."""

    for layer in model["layers"]:
        _stacks.pop(id(layer), None)


def stats(model: dict) -> dict:
    """Groups stacked per kind and the bytes the stacks add (tile padding of the stacked rows)."""

    counts = {kind: 0 for kind in GROUPS}
    added = 0
    for layer in model["layers"]:
        for kind, g in _stacks.get(id(layer), {}).items():
            counts[kind] += 1
            added += g.added
    return {"groups": counts, "added_bytes": added}


def _project(layer: dict, kind: str, x):
    g = _stacks.get(id(layer), {}).get(kind)
    if g is None:
        return None
    if not isinstance(x, Packed) and x.dtype != torch.bfloat16:
        raise ValueError("lane_fuse: x must be bf16 rows or packed rows")
    return lane_matmul(x, g.weight)


def gdn_in(layer: dict, x):
    """[z | b | a] of a gated-DeltaNet layer (..., nv*dv + 2 nv) in one lane matmul, or None."""

    return _project(layer, "zba", x)


def attn_kv(layer: dict, x):
    """[k | v] of an attention layer (..., 2 kv_heads * head_dim) in one lane matmul, or None."""

    return _project(layer, "kv", x)


def mlp_gate_up(layer: dict, x):
    """[gate | up] of an MLP block (..., 2 N) in one lane matmul, or None."""

    return _project(layer, "gu", x)


def gdn_pre(qkv: torch.Tensor, conv_state: torch.Tensor, conv_weight: torch.Tensor, row_seq: torch.Tensor, row_idx: torch.Tensor,
            zba: torch.Tensor, a_log: torch.Tensor, dt_bias: torch.Tensor, *, nk: int, nv: int, dk: int = 128, dv: int = 128):
    """``lane_glue.gdn_pre`` with b and a read in place from ``gdn_in``'s [z | b | a] rows (the chain's
    ``windows`` table of the reference is implied by ``row_idx``)."""

    zs = nv * dv + 2 * nv
    if zba.shape[-1] != zs:
        raise ValueError(f"gdn_pre: [z | b | a] rows of {zs} expected, got {zba.shape[-1]}")
    z2 = zba.reshape(-1, zs)
    return lane_glue.gdn_pre(qkv, conv_state, conv_weight, row_seq, row_idx, z2[:, nv * dv + nv:], z2[:, nv * dv:nv * dv + nv],
                             a_log, dt_bias, nk=nk, nv=nv, dk=dk, dv=dv)


def gdn_post(y: torch.Tensor, zba: torch.Tensor, weight: torch.Tensor, eps: float, *, group: int = 64, rows_out: bool = False):
    """``lane_glue.gdn_post`` with z read in place from the [z | b | a] rows."""

    m, nv, dv = y.shape
    zs = nv * dv + 2 * nv
    if zba.shape[-1] != zs:
        raise ValueError(f"gdn_post: [z | b | a] rows of {zs} expected, got {zba.shape[-1]}")
    return lane_glue.gdn_post(y, zba.reshape(m, zs)[:, :nv * dv], weight, eps, group=group, rows_out=rows_out)


def mlp_act(gate_up: torch.Tensor, *, group: int = 64, rows_out: bool = False):
    """``lane_glue.mlp_act`` on ``mlp_gate_up``'s [gate | up] rows of 2 N."""

    n2 = gate_up.shape[-1]
    if n2 % 2:
        raise ValueError("mlp_act: [gate | up] rows have an even width")
    g2 = gate_up.reshape(-1, n2)
    return lane_glue.mlp_act(g2[:, :n2 // 2], g2[:, n2 // 2:], group=group, rows_out=rows_out)


__all__ = ["GROUPS", "attn_kv", "build", "clear", "gdn_in", "gdn_post", "gdn_pre", "mlp_act", "mlp_gate_up", "stats"]
