"""The forward's glue in a few kernels: everything between two lane matmuls.

Host-side mirror of the reference's glue interfaces (Metal ``kernels/qwen/dense/v1/lane_glue.py:237-317``
``norm_xs / gdn_pre / gdn_post / mlp_act``; CUDA ``families/qwen3_5/cuda/glue.py`` ``add_rmsnorm /
gdn_pre / gated_norm / swiglu / attn_prep / gate_mul / embed``). Every value is a function of its own
row only. A kernel that feeds a matmul returns the matmul's input already ``Packed`` (group sums
included), which is this library's form of the reference's "``x`` comes with its group sums remembered".
"""

from __future__ import annotations

import torch

from . import _lib
from .lane_qmm import MAX_ROWS, Packed, new_packed


def _rows(t: torch.Tensor) -> int:
    m = t.shape[0]
    if not 1 <= m <= MAX_ROWS:
        raise ValueError(f"glue kernels take 1..{MAX_ROWS} rows, got {m}")
    return m


def _bf16(*tensors):
    for t in tensors:
        if t is not None and t.dtype != torch.bfloat16:
            raise ValueError("expected bf16 tensors")
    _lib.need_cuda(*tensors)


def norm_xs(hidden: torch.Tensor, residual: torch.Tensor | None, weight: torch.Tensor, eps: float, *, group: int = 64,
            partials: torch.Tensor | None = None, rows_out: bool = False, packed_out: bool = True,
            out: Packed | None = None, h_out: torch.Tensor | None = None, peer=None):
    """(h, x): h = hidden + residual (hidden itself when there is no residual), x = RMSNorm(h) * weight.

    ``residual`` is bf16 (M, D), or ``partials`` holds a row-parallel projection's fp32 per-rank
    outputs (ranks, M, D) that are added in rank order and rounded once. ``x`` is returned packed for
    the next matmul (``packed_out``) and/or as plain rows (``rows_out``): (h, packed), (h, rows) or
    (h, packed, rows). ``peer``: a ``distributed.RankGroup`` with the fused exchange: the addend is the
    rank-ordered sum of the partials the ranks' ``lane_matmul(..., peer=...)`` calls stored in this rank's
    exchange buffer. Reference: ``lane_glue.norm_xs`` / ``glue.add_rmsnorm``.
    """

    _bf16(hidden, residual, weight)
    m, d = hidden.shape
    _rows(hidden)
    if d % 256 or d > 8192:
        raise ValueError(f"norm_xs: the hidden size must be a multiple of 256 up to 8192, got {d}")
    hidden = hidden.contiguous()
    nparts, pstride = 0, 0
    if partials is not None:
        if residual is not None or partials.dtype != torch.float32 or partials.shape[1:] != (m, d):
            raise ValueError("norm_xs: partials must be fp32 (ranks, M, D) and exclude a bf16 residual")
        partials = partials.contiguous()
        nparts, pstride = partials.shape[0], m * d
    if residual is not None:
        residual = residual.contiguous()
    if peer is not None and (residual is not None or nparts > 0):
        raise ValueError("norm_xs: a peer exchange excludes a residual and gathered partials")
    has_res = residual is not None or nparts > 0 or peer is not None
    if has_res and h_out is None:
        h_out = torch.empty_like(hidden)
    h = h_out if has_res else hidden
    packed = (out if out is not None else new_packed(m, d, group, hidden.device)) if packed_out else None
    rows = torch.empty_like(hidden) if rows_out else None
    with torch.cuda.device(hidden.device):
        if peer is not None:
            _, slot_bytes, seq, tickets, mine = peer.peer_args()
        else:
            slot_bytes, seq, tickets, mine = 0, None, None, None
        _lib.check(_lib.load().tf_norm_xs_peer(hidden.data_ptr(), _lib.ptr(residual), _lib.ptr(partials), nparts, pstride,
                                               weight.data_ptr(), _lib.ptr(h_out) if has_res else None, _lib.ptr(rows),
                                               packed.data.data_ptr() if packed else None, m, d, group, float(eps),
                                               mine, slot_bytes, seq, tickets, peer.world if peer is not None else 0,
                                               _lib.status(hidden.device).word.data_ptr(), _lib.stream()), "norm_xs")
    if packed_out and rows_out:
        return h, packed, rows
    return h, (packed if packed_out else rows)


def mlp_act(gate: torch.Tensor, up: torch.Tensor, *, group: int = 64, rows_out: bool = False, out: Packed | None = None):
    """SiLU(gate) * up -> packed input of the down projection (and the plain rows with ``rows_out``).
    ``gate`` and ``up`` may be column views of one stacked projection output.
    Reference: ``lane_glue.mlp_act`` / ``glue.swiglu``."""

    _bf16(gate, up)
    m, n = gate.shape
    _rows(gate)
    if up.shape != gate.shape or gate.stride(1) != 1 or up.stride(1) != 1 or gate.stride(0) != up.stride(0):
        raise ValueError("mlp_act: gate and up must be (M, I) views with the same row stride")
    packed = out if out is not None else new_packed(m, n, group, gate.device)
    rows = torch.empty((m, n), dtype=torch.bfloat16, device=gate.device) if rows_out else None
    with torch.cuda.device(gate.device):
        _lib.check(_lib.load().tf_swiglu(gate.data_ptr(), up.data_ptr(), gate.stride(0), packed.data.data_ptr(),
                                         _lib.ptr(rows), m, n, group, _lib.stream()), "mlp_act")
    return (packed, rows) if rows_out else packed


swiglu = mlp_act


def mlp_act_tiled(gate_up: torch.Tensor, intermediate: int, *, group: int = 64, rows_out: bool = False,
                  out: Packed | None = None):
    """``mlp_act`` for the output (M, >= 2 I) of a stacked [gate; up] projection whose columns are interleaved by
    16-column tile (``forward.interleave_gate_up``): the same bits as ``mlp_act`` on the separate halves."""

    _bf16(gate_up)
    m = gate_up.shape[0]
    _rows(gate_up)
    if gate_up.dim() != 2 or gate_up.shape[1] < 2 * intermediate or gate_up.stride(1) != 1:
        raise ValueError("mlp_act_tiled: gate_up must be (M, >= 2 I) rows")
    packed = out if out is not None else new_packed(m, intermediate, group, gate_up.device)
    rows = torch.empty((m, intermediate), dtype=torch.bfloat16, device=gate_up.device) if rows_out else None
    with torch.cuda.device(gate_up.device):
        _lib.check(_lib.load().tf_swiglu_tiled(gate_up.data_ptr(), gate_up.stride(0), packed.data.data_ptr(), _lib.ptr(rows), m,
                                               intermediate, group, _lib.stream()), "mlp_act_tiled")
    return (packed, rows) if rows_out else packed


def gdn_post(y: torch.Tensor, z: torch.Tensor, weight: torch.Tensor, eps: float, *, group: int = 64,
             rows_out: bool = False, out: Packed | None = None):
    """SiLU(z) * RMSNorm(y) * weight per value head: y (M, nv, dv), z (M, nv*dv) -> packed (M, nv*dv).
    Reference: ``lane_glue.gdn_post`` / ``glue.gated_norm``."""

    _bf16(y, z, weight)
    m, nv, dv = y.shape
    _rows(y)
    if dv != 128 or z.shape != (m, nv * dv) or z.stride(1) != 1:
        raise ValueError("gdn_post: needs value heads of 128 and z (M, nv*dv)")
    y = y.contiguous()
    packed = out if out is not None else new_packed(m, nv * dv, group, y.device)
    rows = torch.empty((m, nv * dv), dtype=torch.bfloat16, device=y.device) if rows_out else None
    with torch.cuda.device(y.device):
        _lib.check(_lib.load().tf_gated_norm(y.data_ptr(), z.data_ptr(), z.stride(0), weight.data_ptr(),
                                             packed.data.data_ptr(), _lib.ptr(rows), m, nv, dv, group, float(eps),
                                             _lib.stream()), "gdn_post")
    return (packed, rows) if rows_out else packed


gated_norm = gdn_post


def gate_mul(o: torch.Tensor, qg: torch.Tensor, *, heads: int, head_dim: int, group: int = 64, rows_out: bool = False,
             out: Packed | None = None):
    """Attention output (M, H, D) times sigmoid(gate), the gate being the second half of each head's
    [q | gate] block of ``qg`` (M, H*2*D; may be a column view). Reference: ``glue.gate_mul``."""

    _bf16(o, qg)
    m = _rows(o)
    if o.shape != (m, heads, head_dim) or qg.shape != (m, heads * 2 * head_dim) or qg.stride(1) != 1:
        raise ValueError("gate_mul: shapes do not match heads and head_dim")
    o = o.contiguous()
    packed = out if out is not None else new_packed(m, heads * head_dim, group, o.device)
    rows = torch.empty((m, heads * head_dim), dtype=torch.bfloat16, device=o.device) if rows_out else None
    with torch.cuda.device(o.device):
        _lib.check(_lib.load().tf_gate_mul(o.data_ptr(), qg.data_ptr(), qg.stride(0), packed.data.data_ptr(),
                                           _lib.ptr(rows), m, heads, head_dim, group, _lib.stream()), "gate_mul")
    return (packed, rows) if rows_out else packed


def attn_prep(qg: torch.Tensor, k: torch.Tensor, v: torch.Tensor, q_norm: torch.Tensor, k_norm: torch.Tensor,
              pos: torch.Tensor, inv_freq: torch.Tensor, eps: float, *, heads: int, kv_heads: int, head_dim: int,
              out: tuple | None = None):
    """Per-head RMSNorm and partial rotate-half RoPE at each row's own position: queries from the
    [q_h | gate_h] rows ``qg``, keys from ``k``; ``v`` is copied into a contiguous record.
    Returns q (M, H, D), k and v (M, HKV, D). Reference: ``glue.attn_prep``."""

    _bf16(qg, k, v, q_norm, k_norm)
    m = qg.shape[0]
    if pos.dtype != torch.int32 or pos.shape != (m,) or inv_freq.dtype != torch.float32:
        raise ValueError("attn_prep: pos must be int32 (M,) and inv_freq fp32")
    if qg.stride(1) != 1 or k.stride(1) != 1 or v.stride(1) != 1:
        raise ValueError("attn_prep: inputs must be row views with unit column stride")
    dev = qg.device
    if out is None:
        out = (torch.empty((m, heads, head_dim), dtype=torch.bfloat16, device=dev),
               torch.empty((m, kv_heads, head_dim), dtype=torch.bfloat16, device=dev),
               torch.empty((m, kv_heads, head_dim), dtype=torch.bfloat16, device=dev))
    qo, ko, vo = out
    with torch.cuda.device(dev):
        _lib.check(_lib.load().tf_attn_prep(qg.data_ptr(), qg.stride(0), k.data_ptr(), k.stride(0), v.data_ptr(),
                                            v.stride(0), q_norm.data_ptr(), k_norm.data_ptr(), pos.data_ptr(),
                                            inv_freq.data_ptr(), inv_freq.numel(), qo.data_ptr(), ko.data_ptr(),
                                            vo.data_ptr(), m, heads, kv_heads, head_dim, float(eps), _lib.stream()),
                   "attn_prep")
    return qo, ko, vo


def gdn_pre(qkv: torch.Tensor, conv_state: torch.Tensor, conv_weight: torch.Tensor, row_seq: torch.Tensor,
            row_idx: torch.Tensor, a: torch.Tensor, b: torch.Tensor, a_log: torch.Tensor, dt_bias: torch.Tensor, *,
            nk: int, nv: int, dk: int = 128, dv: int = 128, out: tuple | None = None):
    """q, k (M, nk, dk), v (M, nv, dv) bf16 and g, beta (M, nv) fp32 for the window rows.

    ``qkv`` (M, C) rows (may be a column view); ``conv_state`` (n_seqs, 3, C); ``conv_weight`` (C, 4);
    ``row_seq`` / ``row_idx`` int32 (M,): each row's sequence and its place in that sequence's chain.
    Reference: ``lane_glue.gdn_pre`` / ``glue.gdn_pre`` (the ``windows`` table of a chain is implied by
    ``row_idx``)."""

    _bf16(qkv, conv_state, conv_weight, a, b)
    m, c = qkv.shape
    if c != (2 * nk + nv) * 128 or dk != 128 or dv != 128 or conv_weight.shape != (c, 4):
        raise ValueError("gdn_pre: needs head_k_dim == head_v_dim == 128 and a 4-tap conv")
    if a.stride(0) != b.stride(0) or qkv.stride(1) != 1:
        raise ValueError("gdn_pre: a and b must share a row stride")
    dev = qkv.device
    if out is None:
        out = (torch.empty((m, nk, dk), dtype=torch.bfloat16, device=dev), torch.empty((m, nk, dk), dtype=torch.bfloat16, device=dev),
               torch.empty((m, nv, dv), dtype=torch.bfloat16, device=dev), torch.empty((m, nv), dtype=torch.float32, device=dev),
               torch.empty((m, nv), dtype=torch.float32, device=dev))
    q, k, v, g, beta = out
    with torch.cuda.device(dev):
        _lib.check(_lib.load().tf_gdn_pre(qkv.data_ptr(), qkv.stride(0), conv_state.data_ptr(), conv_weight.data_ptr(),
                                          row_seq.data_ptr(), row_idx.data_ptr(), a.data_ptr(), b.data_ptr(), a.stride(0),
                                          a_log.data_ptr(), dt_bias.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(),
                                          g.data_ptr(), beta.data_ptr(), m, nk, nv, dk, dv, 4, _lib.stream()), "gdn_pre")
    return q, k, v, g, beta


def embed(ids: torch.Tensor, weight: torch.Tensor, scales: torch.Tensor, biases: torch.Tensor, d: int, group: int = 64,
          out: torch.Tensor | None = None) -> torch.Tensor:
    """Dequantise one 4-bit embedding row per token id (stored MLX layout). Reference: ``glue.embed``."""

    _lib.need_cuda(ids, weight, scales, biases)
    if ids.dtype != torch.int32 or ids.dim() != 1:
        raise ValueError("embed: ids must be a 1-D int32 tensor")
    m = ids.shape[0]
    if out is None:
        out = torch.empty((m, d), dtype=torch.bfloat16, device=ids.device)
    with torch.cuda.device(ids.device):
        _lib.check(_lib.load().tf_embed(ids.data_ptr(), weight.data_ptr(), scales.data_ptr(), biases.data_ptr(),
                                        out.data_ptr(), m, d, group, weight.shape[0], _lib.stream()), "embed")
    return out


__all__ = ["attn_prep", "embed", "gate_mul", "gated_norm", "gdn_post", "gdn_pre", "mlp_act", "mlp_act_tiled", "norm_xs", "swiglu"]
