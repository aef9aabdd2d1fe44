"""The verify forward of the dense hybrid decoder (gated-DeltaNet layers with a full-attention layer
every ``interval``-th), over the ragged chain windows of many sequences, and its commit.

Mirror of the reference's ``tree_forward`` / ``commit`` / ``State``
(``families/qwen3_5/cuda/forward.py:78-252``; Metal ``kernels/qwen/dense/v1/lane_tree.py:276-392``):
the committed state is read-only until ``commit``; a serial decode step is the same forward with a
one-row window followed by a one-row commit, so a window row has the bits of the serial step at its
position. Differences from the reference, all inside its contract: windows are chains (no trees);
many sequences ride in one forward as packed rows; the KV cache is paged (16-token pages); the
projections that share an input are stacked ([qkv|z|b|a], [q|k|v], [gate|up]).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Sequence

import torch

from . import lane_attention as LA
from . import lane_gdn, lane_glue
from . import lane_moe
from .lane_qmm import MAX_ROWS, QWeight, new_packed, tile_weight
from .lane_qmm import lane_matmul as _lane_matmul


@dataclass
class Config:
    """The fields of the reference's ``Config`` (``families/qwen3_5/cuda/weights.py:38-59``) the forward uses."""

    hidden: int
    intermediate: int
    layers: int
    heads: int
    kv_heads: int
    head_dim: int
    vocab: int
    k_heads: int
    v_heads: int
    dk: int = 128
    dv: int = 128
    conv_kernel: int = 4
    interval: int = 4
    eps: float = 1e-6
    rope_dims: int = 0
    rope_theta: float = 1e7
    group: int = 64
    experts: int = 0                  # routed experts per layer; 0: dense SwiGLU MLP (``intermediate``)
    top_k: int = 0
    moe_intermediate: int = 0
    shared_expert: bool = True        # one always-on expert, stored as expert id ``experts``

    def __post_init__(self):
        if not self.rope_dims:
            self.rope_dims = self.head_dim // 4
        if self.dk != 128 or self.dv != 128 or self.conv_kernel != 4:
            raise ValueError("this build supports GDN heads of 128 and a 4-tap conv")

    def is_linear(self, layer: int) -> bool:
        return (layer + 1) % self.interval != 0

    @property
    def conv_channels(self) -> int:
        return (2 * self.k_heads + self.v_heads) * 128

    def inv_freq(self) -> torch.Tensor:
        half = self.rope_dims // 2
        return (self.rope_theta ** (-torch.arange(0, half, dtype=torch.float64) / half)).to(torch.float32)


@dataclass
class LayerWeights:
    linear: bool
    input_norm: torch.Tensor
    post_norm: torch.Tensor
    in_proj: QWeight                  # GDN: [qkv | z | b | a]; attention: [q (with gates) | k | v]
    out_proj: QWeight
    gate_up: QWeight                  # [gate | up]
    down: QWeight
    conv: torch.Tensor | None = None
    A_log: torch.Tensor | None = None
    dt_bias: torch.Tensor | None = None
    norm: torch.Tensor | None = None
    q_norm: torch.Tensor | None = None
    k_norm: torch.Tensor | None = None
    router: torch.Tensor | None = None       # MoE layers: [experts (+1), hidden] bf16; gate_up/down are then None
    experts: object | None = None            # lane_moe.Experts


@dataclass
class Weights:
    config: Config
    embed: tuple                      # (words, scales, biases) in the stored layout
    layers: list
    norm: torch.Tensor
    head: QWeight
    inv_freq: torch.Tensor
    wide: dict | None = None          # id(QWeight) -> prefill_qmm.TCWeight, made by enable_wide

    def nbytes(self) -> int:
        """Bytes of 4-bit projection weights one forward streams (the weight-bytes roofline numerator)."""

        total = self.head.nbytes()
        for l in self.layers:
            total += l.in_proj.nbytes() + l.out_proj.nbytes()
            if l.experts is None:
                total += l.gate_up.nbytes() + l.down.nbytes()
        return total


def enable_wide(w: Weights) -> Weights:
    """Give every dense projection of ``w`` a twin in the wide-row kernel's tile layout (``prefill_qmm``), so that
    a ``State`` made with ``wide=True`` runs all its steps - serial and windowed - on the tcgen05 kernel (many
    concurrent sequences: 32..128 rows a step). Doubles the weight memory; the lane tiles stay for states made
    without it. A row's bits are then the wide kernel's in every step of that state."""

    from . import prefill_qmm
    from .lane_qmm import untile_weight

    if w.wide is None:
        w.wide = {}
        mats = [w.head]
        for l in w.layers:
            mats += [l.in_proj, l.out_proj] + ([l.gate_up, l.down] if l.experts is None else [])
        for q in mats:
            words, scales, biases = untile_weight(q)
            w.wide[id(q)] = prefill_qmm.tile_weight(words, scales, biases, q.group)
    return w


def _stack(parts, device, group) -> QWeight:
    """Several projections of the same input as one: stored-layout rows concatenated in order, then tiled
    (reference: ``qmm_fast.stack``)."""

    words = torch.cat([p.words for p in parts]).to(device)
    scales = torch.cat([p.scales for p in parts]).to(device)
    biases = torch.cat([p.biases for p in parts]).to(device)
    pad = -words.shape[0] % 8
    if pad:      # output rows in whole 16-byte units (narrow tensor-parallel shards): zero projections, never read
        words = torch.cat([words, words.new_zeros((pad, words.shape[1]))])
        scales = torch.cat([scales, scales.new_zeros((pad, scales.shape[1]))])
        biases = torch.cat([biases, biases.new_zeros((pad, biases.shape[1]))])
    return tile_weight(words.contiguous(), scales.contiguous(), biases.contiguous(), group)


def interleave_gate_up(gate, up):
    """[gate; up] rows in the order the fused SwiGLU wants: for activation tile a (16 columns) the 16 gate rows, then
    the 16 up rows. Returns objects with ``words``, ``scales``, ``biases`` for ``_stack``."""

    from types import SimpleNamespace

    def mix(g, u):
        n = g.shape[0]
        if n % 16:
            raise ValueError("the MLP width must be a multiple of 16")
        return torch.stack([g.reshape(n // 16, 16, -1), u.reshape(n // 16, 16, -1)], dim=1).reshape(2 * n, -1)
    return SimpleNamespace(words=mix(gate.words, up.words), scales=mix(gate.scales, up.scales), biases=mix(gate.biases, up.biases))


def load_weights(model: dict, device="cuda") -> Weights:
    """Build device weights from stored-layout arrays: ``model`` maps names to objects with ``words``,
    ``scales``, ``biases`` (4-bit projections) or to tensors, as ``families/qwen3_5/cuda/weights.py``
    reads them from a checkpoint: per layer ``qkv z b a out conv A_log dt_bias norm`` or ``q k v o q_norm
    k_norm``, plus ``input_norm post_norm gate up down``; top level ``embed norm head config``."""

    c = model["config"]
    cfg = Config(**{f: getattr(c, f) for f in Config.__dataclass_fields__ if hasattr(c, f)}) if not isinstance(c, Config) else c
    g = cfg.group
    layers = []
    for src in model["layers"]:
        def dev(name):
            return src[name].to(device).contiguous()
        moe = "router" in src
        gate_up = None if moe else _stack([interleave_gate_up(src["gate"], src["up"])], device, g)
        down = None if moe else _stack([src["down"]], device, g)
        extra = {}
        if moe:
            e = src["experts"]
            extra = dict(router=dev("router"), experts=lane_moe.make_experts(e["gate"], e["up"], e["down"], g, device))
        if src["linear"]:
            lw = LayerWeights(True, dev("input_norm"), dev("post_norm"), _stack([src["qkv"], src["z"], src["b"], src["a"]], device, g),
                              _stack([src["out"]], device, g), gate_up, down, conv=dev("conv"), A_log=dev("A_log").float(),
                              dt_bias=dev("dt_bias").float(), norm=dev("norm"), **extra)
        else:
            lw = LayerWeights(False, dev("input_norm"), dev("post_norm"), _stack([src["q"], src["k"], src["v"]], device, g),
                              _stack([src["o"]], device, g), gate_up, down, q_norm=dev("q_norm"), k_norm=dev("k_norm"), **extra)
        layers.append(lw)
    e = model["embed"]
    embed = (e.words.to(device).contiguous(), e.scales.to(device).contiguous(), e.biases.to(device).contiguous())
    return Weights(cfg, embed, layers, model["norm"].to(device).contiguous(), _stack([model["head"]], device, g),
                   cfg.inv_freq().to(device))


class State:
    """Committed state of ``n_seqs`` sequences: paged K/V for the attention layers, conv tail and fp32
    recurrent state for the GDN layers, and each sequence's committed length. Read-only during a
    forward; only ``commit`` writes it (reference: ``forward.State``)."""

    def __init__(self, w: Weights, n_seqs: int, max_context: int, device=None, num_pages: int | None = None,
                 wide: bool = False):
        c = w.config
        device = device or w.norm.device
        if wide and w.wide is None:
            raise ValueError("State(wide=True) needs weights prepared by enable_wide")
        self.wide = bool(wide)        # every step of this state multiplies on the wide-row (tcgen05) kernel
        self.n_seqs = n_seqs
        self.lens = [0] * n_seqs
        self.seq_lens = torch.zeros(n_seqs, dtype=torch.int32, device=device)
        self.gdn_layers = [i for i, l in enumerate(w.layers) if l.linear]
        self.att_layers = [i for i, l in enumerate(w.layers) if not l.linear]
        pages_per_seq = -(-(max_context + MAX_ROWS) // LA.PAGE)
        self.kv = LA.PagedKV(len(self.att_layers), n_seqs, num_pages or n_seqs * pages_per_seq, c.kv_heads, c.head_dim,
                             pages_per_seq, device)
        ng = max(len(self.gdn_layers), 1)
        self.conv = torch.zeros((ng, n_seqs, c.conv_kernel - 1, c.conv_channels), dtype=torch.bfloat16, device=device)
        self.rec = torch.zeros((ng, n_seqs, c.v_heads, c.dv, c.dk), dtype=torch.float32, device=device)

    def sync_lens(self) -> None:
        self.seq_lens.copy_(torch.tensor(self.lens, dtype=torch.int32), non_blocking=True)

    def snapshot(self) -> dict:
        """What the committed sequences keep outside the K/V pages' rows: the GDN states, the conv tails, the
        lengths (reference: ``families/qwen4_exp/cuda/forward.py:200-222``). The K/V rows below the lengths stay
        where they are (later commits only write at or past a sequence's length), so ``restore`` brings the
        sequences back to this point as long as their pages have not been released. The snapshot carries the
        kernel library's source hash: state made by other kernels has other bits and is refused."""

        from . import build

        return {"kernels": build.source_hash(), "lens": list(self.lens), "rec": self.rec.clone(), "conv": self.conv.clone()}

    def restore(self, snap: dict) -> None:
        from . import build

        if snap.get("kernels") != build.source_hash():
            raise ValueError("State.restore: the snapshot was made by a different build of the kernels")
        if snap["rec"].shape != self.rec.shape or snap["conv"].shape != self.conv.shape or len(snap["lens"]) != self.n_seqs:
            raise ValueError("State.restore: the snapshot belongs to a differently shaped state")
        if any(self.kv.owned[s] * LA.PAGE < n for s, n in enumerate(snap["lens"])):
            raise ValueError("State.restore: a sequence's pages were released since the snapshot")
        self.rec.copy_(snap["rec"])
        self.conv.copy_(snap["conv"])
        self.lens = list(snap["lens"])
        self.sync_lens()


@dataclass
class Batch:
    """Row bookkeeping of one forward: which sequence and which place in its chain each packed row has."""

    widths: list
    rows: int
    seq_start: torch.Tensor
    row_seq: torch.Tensor
    row_idx: torch.Tensor
    row_pos: torch.Tensor
    row_nkeys: torch.Tensor
    max_window: int
    max_chunks: int


def _batch_lists(st: State, widths):
    starts, seq, idx, pos, nk = [0], [], [], [], []
    for s, wd in enumerate(widths):
        starts.append(starts[-1] + wd)
        for t in range(wd):
            seq.append(s); idx.append(t); pos.append(st.lens[s] + t); nk.append(st.lens[s] + t + 1)
    return starts, seq, idx, pos, nk


def refresh_batch(b: Batch, st: State) -> None:
    """Rewrite a batch's position tensors in place from the state's current lengths (same widths):
    what a captured CUDA graph needs before each replay."""

    _, _, _, pos, nk = _batch_lists(st, b.widths)
    need = max(LA.chunks_for(st.lens[s] + wd) for s, wd in enumerate(b.widths))
    if need > b.max_chunks:
        raise ValueError(f"context needs {need} key chunks, the batch was built for {b.max_chunks}")
    b.row_pos.copy_(torch.tensor(pos, dtype=torch.int32), non_blocking=True)
    b.row_nkeys.copy_(torch.tensor(nk, dtype=torch.int32), non_blocking=True)


def make_batch(st: State, widths: Sequence[int], device, max_chunks: int | None = None) -> Batch:
    widths = [int(x) for x in widths]
    if len(widths) != st.n_seqs or any(x < 0 for x in widths) or sum(widths) < 1:
        raise ValueError("one window width per sequence (0 = idle), at least one row in all")
    rows = sum(widths)
    if rows > MAX_ROWS:
        raise ValueError(f"a forward takes at most {MAX_ROWS} packed rows, got {rows}")
    starts, seq, idx, pos, nk = _batch_lists(st, widths)
    need = max(LA.chunks_for(st.lens[s] + wd) for s, wd in enumerate(widths))
    def i32(v):
        return torch.tensor(v, dtype=torch.int32).to(device, non_blocking=True)
    return Batch(widths, rows, i32(starts), i32(seq), i32(idx), i32(pos), i32(nk), max(widths), max(max_chunks or 0, need, 1))


@dataclass
class Record:
    """What a forward leaves for ``commit``: per GDN layer the window's k, v, g, beta and stacked
    projection rows (qkv for the conv tail), per attention layer the window's K/V rows."""

    batch: Batch
    gdn_k: torch.Tensor
    gdn_v: torch.Tensor
    gdn_g: torch.Tensor
    gdn_beta: torch.Tensor
    gdn_in: torch.Tensor
    att_k: torch.Tensor
    att_v: torch.Tensor


@torch.no_grad()
def tree_forward(w: Weights, tokens: torch.Tensor, windows, st: State, *, full_logits: bool = True,
                 max_chunks: int | None = None, batch: Batch | None = None, tp=None, ep=None):
    """Logits (rows, vocab) bf16 for the window rows, and the record ``commit`` needs.

    ``windows``: one window width per sequence of ``st`` (packed rows are each sequence's chain in
    order), or, for a single sequence, the reference's ``parents`` list of a chain ([-1, 0, 1, ...]).
    The state is untouched. ``full_logits=False`` returns the final-normed hidden rows instead.
    ``tp``: a ``distributed.RankGroup`` when ``w`` is one rank's shard: the output and down projections
    then return fp32 partials, every rank gathers all of them and the next norm adds them in rank order
    (two collectives a layer); the logits are this rank's slice of the vocabulary.
    ``ep``: a ``lane_moe.ExpertGroup`` when the MoE layers' experts are spread over ranks (``w`` then holds
    this rank's experts; everything else is replicated and every rank computes the same rows).
    """

    c = w.config
    dev = w.norm.device
    if batch is None:
        windows = list(windows)
        if st.n_seqs == 1 and windows and windows[0] == -1:
            windows = [lane_gdn.chain_parents(windows)]
        for s, wd in enumerate(windows):
            if wd and st.kv.reserve(s, st.lens[s] + wd):
                st.kv.sync_table()
        st.sync_lens()
        batch = make_batch(st, windows, dev, max_chunks)
    b = batch
    R = b.rows
    if tokens.shape != (R,) or tokens.dtype not in (torch.int32, torch.int64) or tokens.device != dev:
        raise ValueError("tokens must be a 1-D int tensor on the weights' device, one per window row")
    g = c.group
    kd, vd = c.k_heads * c.dk, c.v_heads * c.dv
    ng, na = max(len(st.gdn_layers), 1), max(len(st.att_layers), 1)
    bf = dict(dtype=torch.bfloat16, device=dev)
    rec = Record(b, torch.empty((ng, R, c.k_heads, c.dk), **bf), torch.empty((ng, R, c.v_heads, c.dv), **bf),
                 torch.empty((ng, R, c.v_heads), dtype=torch.float32, device=dev),
                 torch.empty((ng, R, c.v_heads), dtype=torch.float32, device=dev),
                 torch.empty((ng, R, -(-(2 * kd + 2 * vd + 2 * c.v_heads) // 8) * 8), **bf),
                 torch.empty((na, R, c.kv_heads, c.head_dim), **bf), torch.empty((na, R, c.kv_heads, c.head_dim), **bf))
    q_att = torch.empty((R, c.heads, c.head_dim), **bf)
    att_in = torch.empty((R, c.heads * 2 * c.head_dim + 2 * c.kv_heads * c.head_dim), **bf)
    mlp_in = torch.empty((R, 2 * c.intermediate), **bf) if c.experts == 0 else None
    moe_buf = None
    if c.experts:
        if tp is not None:
            raise ValueError("tree_forward: mixture-of-experts layers shard by expert, not by tensor-parallel rank")
        moe_buf = lane_moe.MoEBuffers(R, c.experts, c.top_k, c.shared_expert, c.hidden, c.moe_intermediate, g, dev)
    scratch = torch.empty(LA.scratch_bytes(R, c.heads, c.head_dim, b.max_chunks), dtype=torch.uint8, device=dev)
    scale = c.head_dim ** -0.5

    fused_tp = tp is not None and getattr(tp, "fused", False) and not st.wide
    if st.wide:
        from . import prefill_qmm

        if c.experts:
            raise ValueError("tree_forward: the wide-row kernel covers the dense projections only")
        kmax = max(q.k for q in (w.head, *(m for l in w.layers for m in (l.in_proj, l.out_proj, l.gate_up, l.down))))
        staging = torch.empty(prefill_qmm.packed_bytes(R, kmax, g), dtype=torch.uint8, device=dev)

        def lane_matmul(x_, weight, *, f32=False, out=None, next_weight=None, peer=None, act_out=None):      # noqa: F811
            return prefill_qmm.prefill_matmul(x_, w.wide[id(weight)], f32=f32, out=out, staging=staging)
    else:
        lane_matmul = _lane_matmul

    def row_parallel(act, weight, nxt):
        """(residual rows, gathered partials): one of the two is None; both are when the exchange is fused
        into this matmul's epilogue and the next norm kernel."""
        if tp is None:
            return lane_matmul(act, weight, next_weight=nxt), None
        if fused_tp:
            lane_matmul(act, weight, next_weight=nxt, peer=tp)
            return None, None
        return None, tp.gather_partials(lane_matmul(act, weight, f32=True, next_weight=nxt))

    def norm(x_, res, wt, first=False, **kw):
        # with the fused exchange every norm but the first one (after the embedding) adds a peer sum
        return lane_glue.norm_xs(x_, res, wt, c.eps, group=g, peer=tp if fused_tp and not first else None, **kw)

    # each matmul tells the kernel which weight streams next, so that its first bytes wait in L2
    def after(li):
        return w.layers[li + 1].in_proj if li + 1 < len(w.layers) else (w.head if full_logits else None)

    x = lane_glue.embed(tokens.to(torch.int32), *w.embed, c.hidden, g)
    pending = parts = None
    gi = ai = 0
    for li, layer in enumerate(w.layers):
        x, h = norm(x, pending, layer.input_norm, first=li == 0, partials=parts)
        if layer.linear:
            proj = lane_matmul(h, layer.in_proj, out=rec.gdn_in[gi], next_weight=layer.out_proj)
            qkv, z = proj[:, :2 * kd + vd], proj[:, 2 * kd + vd:2 * kd + 2 * vd]
            bb, aa = proj[:, 2 * kd + 2 * vd:2 * kd + 2 * vd + c.v_heads], proj[:, 2 * kd + 2 * vd + c.v_heads:2 * kd + 2 * vd + 2 * c.v_heads]
            # conv + gates, recurrence and gated norm in one launch; k, v, g, beta land in the record for the commit
            mixed = lane_gdn.gdn_mixer(qkv, z, aa, bb, st.conv[gi], layer.conv, layer.A_log, layer.dt_bias, layer.norm, st.rec[gi],
                                       b.seq_start, nk=c.k_heads, nv=c.v_heads, eps=c.eps, group=g,
                                       record=(rec.gdn_k[gi], rec.gdn_v[gi], rec.gdn_g[gi], rec.gdn_beta[gi]))
            gi += 1
        else:
            proj = lane_matmul(h, layer.in_proj, out=att_in, next_weight=layer.out_proj)
            nq = c.heads * 2 * c.head_dim
            nkv = c.kv_heads * c.head_dim
            lane_glue.attn_prep(proj[:, :nq], proj[:, nq:nq + nkv], proj[:, nq + nkv:], layer.q_norm, layer.k_norm, b.row_pos,
                                w.inv_freq, c.eps, heads=c.heads, kv_heads=c.kv_heads, head_dim=c.head_dim,
                                out=(q_att, rec.att_k[ai], rec.att_v[ai]))
            mixed = new_packed(R, c.heads * c.head_dim, g, dev)
            LA.lane_attention(q_att, rec.att_k[ai], rec.att_v[ai], st.kv.k[ai], st.kv.v[ai], st.kv.table, st.seq_lens,
                              b.seq_start, b.row_nkeys, scale=scale, max_window=b.max_window, max_chunks=b.max_chunks,
                              scratch=scratch, gate=proj[:, :nq], packed_out=mixed)      # output gate + packing in the merge
            ai += 1
        r, rparts = row_parallel(mixed, layer.out_proj, layer.gate_up if layer.experts is None else after(li))
        if layer.experts is not None:
            x, hrows = norm(x, r, layer.post_norm, partials=rparts, rows_out=True, packed_out=False)
            pending, parts = lane_moe.moe(hrows, layer.router, layer.experts, moe_buf, ep), None
            continue
        x, h = norm(x, r, layer.post_norm, partials=rparts)
        if R <= 8 and not st.wide:
            # SwiGLU in the gate_up matmul's epilogue (the same bits as the separate kernel below)
            act = lane_matmul(h, layer.gate_up, act_out=new_packed(R, c.intermediate, g, dev), next_weight=layer.down)
        else:
            gu = lane_matmul(h, layer.gate_up, out=mlp_in, next_weight=layer.down)
            act = lane_glue.mlp_act_tiled(gu, c.intermediate, group=g)
        pending, parts = row_parallel(act, layer.down, after(li))
    if not full_logits:
        _, hrows = norm(x, pending, w.norm, rows_out=True, packed_out=False, partials=parts)
        return hrows, rec
    _, h = norm(x, pending, w.norm, partials=parts)
    return lane_matmul(h, w.head), rec


@torch.no_grad()
def commit(st: State, record: Record, keep: Sequence[int]) -> None:
    """Keep the first ``keep[s]`` rows of every sequence's window: K/V rows go into the pages, the GDN
    state is replayed over them and the conv tail shifted, for all layers in three launches
    (reference: ``forward.commit`` with an accepted path)."""

    b = record.batch
    keep = [int(k) for k in keep]
    if len(keep) != st.n_seqs or any(k < 0 or k > wd for k, wd in zip(keep, b.widths)):
        raise ValueError("keep must give, per sequence, a row count within its window")
    dev = st.seq_lens.device
    keep_t = torch.tensor(keep, dtype=torch.int32).to(dev, non_blocking=True)
    if st.gdn_layers:
        lane_gdn.replay(record.gdn_k, record.gdn_v, record.gdn_g, record.gdn_beta, st.rec, b.seq_start, keep_t)
        lane_gdn.conv_commit(record.gdn_in, st.conv, b.seq_start, keep_t, st.conv.shape[-1])
    if st.att_layers:
        LA.kv_commit(record.att_k, record.att_v, st.kv, st.seq_lens, b.seq_start, keep_t)
    for s, k in enumerate(keep):
        st.lens[s] += k
    st.sync_lens()


def accept_path(drafted: Sequence[int], verified: Sequence[int]) -> int:
    """Rows of a chain window to keep: row 0 is always kept (its input token was already decided);
    row t+1 is kept while the token verified at row t equals the token drafted as row t+1's input
    (reference: ``lane_tree.accept_path`` for a chain)."""

    n = 1
    while n < len(drafted) and int(drafted[n]) == int(verified[n - 1]):
        n += 1
    return n


__all__ = ["Batch", "Config", "LayerWeights", "Record", "State", "Weights", "accept_path", "commit", "load_weights",
           "make_batch", "refresh_batch", "tree_forward"]
