"""Mixture-of-experts block of the lane forward: fp32 router, per-row top-k (ties to the lower id),
the window's distinct experts, grouped 4-bit expert projections, slot-ordered combine.

Host-side mirror of the reference's ``families/qwen4_exp/cuda/moe.py:42-163`` (``router``, ``select``,
``MoEBuffers``, ``moe``) and ``qmm.py:421-602`` (``Experts``, ``Group``, ``moe_gateup``, ``moe_down``).
A row's routing, its expert outputs and its combined result never depend on the rows beside it: the
expert projections run as 8-row problems of the lane matmul (``tf_qmm_grouped``), each row of which has
the bits of ``lane_matmul`` on that row alone. The shared expert is stored as expert ``E`` of the same
tables and rides as the last slot of every row.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from . import _lib
from .lane_qmm import QWeight, scratch_for, tile_weight

MAX_ROWS = 128


class ExpertGroup:
    """Expert parallelism over the ranks of a process group: routed expert e lives on rank
    ``e // (experts / world)``, the shared expert on every rank (its problems dealt round-robin). Every
    rank routes all rows; a rank computes the (row, expert) pairs of its own experts and stores the
    results into every rank's buffer in symmetric memory (16-byte self-signalling packets over NVLink,
    plain peer stores); the combine polls what it needs. The block's output has the bits of the one-GPU
    block. (The reference shards expert width across two ranks instead: ``families/qwen4_exp/cuda/comm.py``.)"""

    def __init__(self, experts: int, top_k: int, shared: bool, hidden: int, device, group=None, max_rows: int = MAX_ROWS):
        import os

        import torch.distributed as dist

        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")     # plain peer stores only
        import torch.distributed._symmetric_memory as symm_mem

        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        if experts % self.world:
            raise ValueError(f"{experts} experts do not split over {self.world} ranks")
        self.per = experts // self.world
        total, slots = experts + (1 if shared else 0), top_k + (1 if shared else 0)
        lib = _lib.load()
        self.slot_bytes = (lib.tf_moe_slot_bytes(lib.tf_moe_max_problems(max_rows, slots, total), hidden) + 255) // 256 * 256
        self.buf = symm_mem.empty(2 * self.slot_bytes, dtype=torch.uint8, device=device)
        self.buf.zero_()
        self.handle = symm_mem.rendezvous(self.buf, group=group if group is not None else dist.group.WORLD)
        self.state = torch.zeros(2, dtype=torch.int32, device=device)          # exchange number, CTA tickets
        self.count = 0
        torch.cuda.synchronize(device)
        dist.barrier(group)

    def local_experts(self, shared: bool = True) -> list:
        """Global ids of the experts this rank stores, in local slot order."""

        ids = list(range(self.rank * self.per, (self.rank + 1) * self.per))
        return ids + ([self.per * self.world] if shared else [])


@dataclass
class Experts:
    """The experts' projections, tiled and stacked: ``gate_up`` [(E+1), 2I, D] and ``down`` [(E+1), D, I]."""

    gate_up: torch.Tensor        # uint8, (E + 1) * tf_qmm_tiled_bytes(2I, D, group)
    down: torch.Tensor           # uint8, (E + 1) * tf_qmm_tiled_bytes(D, I, group)
    count: int                   # experts in the tables (routed + shared)
    hidden: int
    intermediate: int
    group: int

    def expert(self, e: int) -> tuple[QWeight, QWeight]:
        """Expert e's projections as ordinary lane-matmul weights (views, nothing copied)."""

        gu = self.gate_up.numel() // self.count
        dn = self.down.numel() // self.count
        return (QWeight(self.gate_up[e * gu:(e + 1) * gu], 2 * self.intermediate, self.hidden, self.group),
                QWeight(self.down[e * dn:(e + 1) * dn], self.hidden, self.intermediate, self.group))


def make_experts(gates, ups, downs, group: int = 32, device="cuda") -> Experts:
    """Stack stored-layout experts (objects with ``words``, ``scales``, ``biases``): ``[gate; up]`` rows
    of expert e tiled together, then its ``down``. Reference: ``qmm.make_experts``."""

    gu, dn = [], []
    for g, u, d in zip(gates, ups, downs):
        words = torch.cat([g.words, u.words]).to(device)
        gu.append(tile_weight(words, torch.cat([g.scales, u.scales]).to(device), torch.cat([g.biases, u.biases]).to(device), group).tiled)
        dn.append(tile_weight(d.words.to(device), d.scales.to(device), d.biases.to(device), group).tiled)
    inter, hidden = gates[0].words.shape[0], gates[0].words.shape[1] * 8
    return Experts(torch.cat(gu), torch.cat(dn), len(gu), hidden, inter, group)


class MoEBuffers:
    """Static scratch for one row count, so that a step can be captured in a CUDA graph (reference:
    ``moe.MoEBuffers``)."""

    def __init__(self, rows: int, experts: int, top_k: int, shared: bool, hidden: int, intermediate: int, group: int, device):
        if not 1 <= rows <= MAX_ROWS:
            raise ValueError(f"MoEBuffers: 1..{MAX_ROWS} rows, got {rows}")
        lib = _lib.load()
        self.rows, self.experts, self.top_k, self.shared = rows, experts, top_k, shared
        self.total = experts + (1 if shared else 0)
        self.slots = top_k + (1 if shared else 0)
        self.hidden, self.intermediate, self.group = hidden, intermediate, group
        self.max_probs = lib.tf_moe_max_problems(rows, self.slots, self.total)
        i32, f32 = torch.int32, torch.float32
        self.logits = torch.empty((rows, self.total), dtype=f32, device=device)
        self.pick = torch.empty((rows, self.slots), dtype=i32, device=device)
        self.wts = torch.empty((rows, self.slots), dtype=f32, device=device)
        self.prob_expert = torch.zeros(self.max_probs, dtype=i32, device=device)
        self.prob_count = torch.zeros(1, dtype=i32, device=device)
        self.prob_rows = torch.full((self.max_probs, 8), -1, dtype=i32, device=device)
        self.prob_sel = torch.zeros(self.max_probs, dtype=i32, device=device)       # expert parallelism: this rank's problems
        self.sel_count = torch.zeros(1, dtype=i32, device=device)
        self.pair_loc = torch.zeros((rows, self.slots), dtype=i32, device=device)
        self.x_packed = torch.empty(self.max_probs * lib.tf_packed_bytes(8, hidden, group), dtype=torch.uint8, device=device)
        self.gate_up = torch.empty((self.max_probs, 8, 2 * intermediate), dtype=torch.bfloat16, device=device)
        self.act_packed = torch.empty(self.max_probs * lib.tf_packed_bytes(8, intermediate, group), dtype=torch.uint8, device=device)
        self.y = torch.empty((self.max_probs * 8, hidden), dtype=f32, device=device)
        self.out = torch.empty((rows, hidden), dtype=torch.bfloat16, device=device)


def router(x: torch.Tensor, router_rows: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """x [R, D] bf16, router_rows [E (+1), D] bf16 -> logits [R, E (+1)] fp32."""

    _lib.need_cuda(x, router_rows)
    if x.dtype != torch.bfloat16 or router_rows.dtype != torch.bfloat16 or x.dim() != 2 or x.stride(1) != 1:
        raise ValueError("router: x and router_rows must be 2-D bf16 with unit inner stride")
    m, d = x.shape
    ne = router_rows.shape[0]
    if out is None:
        out = torch.empty((m, ne), dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        _lib.check(_lib.load().tf_moe_router(x.data_ptr(), x.stride(0), router_rows.contiguous().data_ptr(), out.data_ptr(), m, d, ne,
                                             _lib.stream()), "moe router")
    return out


def select(logits: torch.Tensor, buf: MoEBuffers, ep: ExpertGroup | None = None) -> None:
    """Each row's experts and weights, then the window's problem list (``buf.pick``, ``buf.wts``,
    ``buf.prob_*``, ``buf.pair_loc``)."""

    lib = _lib.load()
    rows = logits.shape[0]
    with torch.cuda.device(logits.device):
        _lib.check(lib.tf_moe_select(logits.data_ptr(), rows, buf.total, buf.experts, buf.top_k, buf.pick.data_ptr(),
                                     buf.wts.data_ptr(), _lib.stream()), "moe select")
        _lib.check(lib.tf_moe_group(buf.pick.data_ptr(), rows, buf.slots, buf.total, buf.max_probs, buf.prob_expert.data_ptr(),
                                    buf.prob_count.data_ptr(), buf.prob_rows.data_ptr(), buf.pair_loc.data_ptr(), buf.experts,
                                    ep.rank if ep else 0, ep.world if ep else 1, buf.prob_sel.data_ptr() if ep else None,
                                    buf.sel_count.data_ptr() if ep else None, _lib.stream()), "moe group")


def moe(x: torch.Tensor, router_rows: torch.Tensor, ex: Experts, buf: MoEBuffers, ep: ExpertGroup | None = None) -> torch.Tensor:
    """Route rows x [R, D] (bf16, already normalised) and run their experts:
    returns ``buf.out`` [R, D] bf16 = bf16(sum_k w_k y_k), slots in order, the shared expert last.

    With ``ep`` the experts are spread over the ranks (``ex`` holds this rank's, in
    ``ep.local_experts`` order); every rank must call with the same rows and gets the same output."""

    lib = _lib.load()
    rows, d = x.shape
    want = buf.total if ep is None else ep.per + (1 if buf.shared else 0)
    if rows != buf.rows or d != buf.hidden or ex.hidden != d or ex.intermediate != buf.intermediate or ex.count != want:
        raise ValueError("moe: buffers, experts and input do not match")
    dev = x.device
    router(x, router_rows, buf.logits)
    select(buf.logits, buf, ep)
    count = buf.sel_count if ep else buf.prob_count
    sel = buf.prob_sel.data_ptr() if ep else None
    scratch = scratch_for(dev)
    st = _lib.status(dev)
    g, inter = buf.group, buf.intermediate
    with torch.cuda.device(dev):
        s = _lib.stream()
        _lib.check(lib.tf_moe_pack(x.data_ptr(), x.stride(0), buf.prob_rows.data_ptr(), buf.prob_count.data_ptr(), buf.max_probs,
                                   buf.x_packed.data_ptr(), d, g, s), "moe pack")
        _lib.check(lib.tf_qmm_grouped(buf.x_packed.data_ptr(), ex.gate_up.data_ptr(), buf.prob_expert.data_ptr(),
                                      count.data_ptr(), sel, buf.max_probs, buf.gate_up.data_ptr(), scratch.data_ptr(),
                                      scratch.numel(), 2 * inter, d, g, 0, st.word.data_ptr(), s), "moe gate_up")
        _lib.check(lib.tf_moe_act(buf.gate_up.data_ptr(), buf.prob_count.data_ptr(), buf.max_probs, buf.act_packed.data_ptr(), inter,
                                  g, s), "moe act")
        _lib.check(lib.tf_qmm_grouped(buf.act_packed.data_ptr(), ex.down.data_ptr(), buf.prob_expert.data_ptr(),
                                      count.data_ptr(), sel, buf.max_probs, buf.y.data_ptr(), scratch.data_ptr(),
                                      scratch.numel(), d, inter, g, 1, st.word.data_ptr(), s), "moe down")
        if ep is None:
            _lib.check(lib.tf_moe_combine(buf.y.data_ptr(), buf.pair_loc.data_ptr(), buf.wts.data_ptr(), buf.slots,
                                          buf.out.data_ptr(), rows, d, s), "moe combine")
        else:
            if lib.tf_moe_slot_bytes(buf.max_probs, d) > ep.slot_bytes:
                raise ValueError("moe: the expert group's exchange buffer is too small for these buffers")
            ep.count += 1
            _lib.check(lib.tf_moe_push(buf.y.data_ptr(), buf.prob_sel.data_ptr(), buf.sel_count.data_ptr(), buf.max_probs, d,
                                       ep.handle.buffer_ptrs_dev, ep.slot_bytes, ep.rank, ep.world, ep.state[0:1].data_ptr(), s),
                       "moe push")
            _lib.check(lib.tf_moe_combine_peer(ep.buf.data_ptr(), ep.slot_bytes, buf.pair_loc.data_ptr(), buf.wts.data_ptr(),
                                               buf.slots, buf.out.data_ptr(), rows, d, ep.world, ep.state[0:1].data_ptr(),
                                               ep.state[1:2].data_ptr(), st.word.data_ptr(), s), "moe combine (peer)")
    return buf.out


__all__ = ["ExpertGroup", "Experts", "MoEBuffers", "make_experts", "moe", "router", "select"]
