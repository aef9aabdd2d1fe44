"""Gated-DeltaNet recurrence for verify windows, and its commit.

Host-side mirror of the reference's ``gated_delta_tree`` / ``replay_path``
(``kernels/qwen/dense/v1/lane_tree.py:132-182``), ``tree / replay / replay_many``
(``families/qwen3_5/cuda/gdn_tree.py:29-53``) and the batched-sequence step of ``LaneGDNCache``
(``kernels/qwen/dense/v1/lane_gdn.py:377-450``), for chain windows of many sequences at once. The
committed state is read-only during a forward; ``replay`` advances it over the accepted rows with
the kernel's own arithmetic, so it equals the state serial one-row steps would have left.
"""

from __future__ import annotations

import torch

from . import _lib


def chain_parents(parents) -> int:
    """Validate a reference-style ``parents`` list as one chain ([-1, 0, 1, ...]); returns its length."""

    parents = [int(p) for p in parents]
    if not parents or parents[0] != -1:
        raise ValueError("a verify window needs a root at row zero")
    if any(p != i - 1 for i, p in enumerate(parents)):
        raise ValueError("this build verifies chain windows only (parents must be [-1, 0, 1, ...])")
    return len(parents)


def gated_delta_chain(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, g: torch.Tensor, beta: torch.Tensor,
                      state: torch.Tensor, seq_start: torch.Tensor, *, state_out: torch.Tensor | None = None,
                      out: torch.Tensor | None = None) -> torch.Tensor:
    """y (R, Hv, Dv) bf16 for the packed window rows of every sequence, from the untouched ``state``.

    q, k (R, Hk, 128) bf16; v (R, Hv, Dv) bf16; g, beta (R, Hv) fp32; state (S, Hv, Dv, 128) fp32;
    ``seq_start`` int32 (S+1,) first packed row of each sequence. ``state_out`` (optional) receives
    the state after each sequence's last row.
    """

    _lib.need_cuda(q, k, v, g, beta, state, seq_start)
    r, hk, dk = q.shape
    hv, dv = v.shape[1], v.shape[2]
    s = state.shape[0]
    if (q.dtype != torch.bfloat16 or k.shape != q.shape or v.shape[0] != r or g.shape != (r, hv) or beta.shape != g.shape
            or g.dtype != torch.float32 or state.dtype != torch.float32 or state.shape != (s, hv, dv, dk)
            or seq_start.dtype != torch.int32 or seq_start.shape != (s + 1,)):
        raise ValueError("gated_delta_chain: inconsistent shapes or dtypes")
    for t in (q, k, v, g, beta, state):
        if not t.is_contiguous():
            raise ValueError("gated_delta_chain: tensors must be contiguous")
    if out is None:
        out = torch.empty((r, hv, dv), dtype=torch.bfloat16, device=q.device)
    with torch.cuda.device(q.device):
        _lib.check(_lib.load().tf_gdn_chain(q.data_ptr(), k.data_ptr(), v.data_ptr(), g.data_ptr(), beta.data_ptr(),
                                            state.data_ptr(), _lib.ptr(state_out), out.data_ptr(), seq_start.data_ptr(),
                                            s, hk, hv, dk, dv, _lib.stream()), "gated_delta_chain")
    return out


def gdn_mixer(qkv: torch.Tensor, z: torch.Tensor, a: torch.Tensor, b: torch.Tensor, conv_state: torch.Tensor,
              conv_weight: torch.Tensor, a_log: torch.Tensor, dt_bias: torch.Tensor, norm_weight: torch.Tensor,
              state: torch.Tensor, seq_start: torch.Tensor, *, nk: int, nv: int, eps: float, group: int = 64,
              record: tuple, out=None, rows_out: bool = False):
    """The GDN layer between its input and output projections in one launch: conv + gates
    (``lane_glue.gdn_pre``), recurrence (``gated_delta_chain``) and gated norm (``lane_glue.gdn_post``),
    with the bits of the three run one after the other (reference: the fused chain kernel of
    ``families/qwen4_exp/cuda/gdn.cu:49-152``).

    qkv (R, C), z (R, nv*128), a, b (R, nv): column views of the stacked projection's rows. ``record`` =
    (k (R, nk, 128), v (R, nv, 128) bf16, g, beta (R, nv) fp32): what ``replay`` needs at commit. Returns
    the packed rows for the output projection (and the plain rows with ``rows_out``)."""

    from .lane_qmm import new_packed

    _lib.need_cuda(qkv, z, a, b, conv_state, conv_weight, state, seq_start)
    r, c = qkv.shape
    s = state.shape[0]
    k_rec, v_rec, g_rec, beta_rec = record
    if (c != (2 * nk + nv) * 128 or z.shape != (r, nv * 128) or a.shape != (r, nv) or b.shape != (r, nv) or a.stride(0) != b.stride(0)
            or qkv.stride(1) != 1 or z.stride(1) != 1 or conv_state.shape != (s, 3, c) or conv_weight.shape != (c, 4)
            or state.shape != (s, nv, 128, 128) or state.dtype != torch.float32 or seq_start.shape != (s + 1,)
            or k_rec.shape != (r, nk, 128) or v_rec.shape != (r, nv, 128) or g_rec.shape != (r, nv) or beta_rec.shape != (r, nv)):
        raise ValueError("gdn_mixer: inconsistent shapes")
    for t in (conv_state, conv_weight, state, k_rec, v_rec, g_rec, beta_rec):
        if not t.is_contiguous():
            raise ValueError("gdn_mixer: state, weights and record tensors must be contiguous")
    packed = out if out is not None else new_packed(r, nv * 128, group, qkv.device)
    rows = torch.empty((r, nv * 128), dtype=torch.bfloat16, device=qkv.device) if rows_out else None
    with torch.cuda.device(qkv.device):
        _lib.check(_lib.load().tf_gdn_fused(
            qkv.data_ptr(), qkv.stride(0), z.data_ptr(), z.stride(0), a.data_ptr(), b.data_ptr(), a.stride(0),
            conv_state.data_ptr(), conv_weight.data_ptr(), a_log.data_ptr(), dt_bias.data_ptr(), norm_weight.data_ptr(),
            state.data_ptr(), k_rec.data_ptr(), v_rec.data_ptr(), g_rec.data_ptr(), beta_rec.data_ptr(), packed.data.data_ptr(),
            _lib.ptr(rows), seq_start.data_ptr(), r, s, nk, nv, 128, 128, 4, group, float(eps), _lib.stream()), "gdn_mixer")
    return (packed, rows) if rows_out else packed


class LaneGDNCache:
    """Many lanes forked from one committed state, advanced one position at a time (reference:
    ``LaneGDNCache.step``, ``kernels/qwen/dense/v1/lane_gdn.py:377-450``). The reference keeps the shared
    state S0 plus a per-lane history; here every lane owns its fp32 state (Hv x Dv x Dk, 64 KB a head: HBM
    is not the scarce resource on this machine) and a step is the chain kernel over one-row windows, so a
    lane's outputs have the bits of the serial recurrence."""

    def __init__(self, s0: torch.Tensor, lanes: int):
        if s0.dim() != 3 or s0.dtype != torch.float32 or lanes < 1:
            raise ValueError("LaneGDNCache: s0 must be an fp32 (Hv, Dv, Dk) state")
        _lib.need_cuda(s0)
        self.lanes = lanes
        self.state = s0.unsqueeze(0).repeat(lanes, 1, 1, 1).contiguous()
        self.t = 0
        self._starts = torch.arange(lanes + 1, dtype=torch.int32, device=s0.device)

    def step(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, log_g: torch.Tensor, beta: torch.Tensor) -> torch.Tensor:
        """One position for every lane. q, k: [N, Hk, Dk]; v: [N, Hv, Dv]; log_g, beta: [N, Hv] -> y [N, Hv, Dv]."""

        if q.shape[0] != self.lanes:
            raise ValueError(f"LaneGDNCache.step: {self.lanes} lanes, got {q.shape[0]} rows")
        y = gated_delta_chain(q.contiguous(), k.contiguous(), v.contiguous(), torch.exp(log_g.float()).contiguous(),
                              beta.float().contiguous(), self.state, self._starts, state_out=self.state)
        self.t += 1
        return y


def gated_delta_tree(q, k, v, g, beta, state, parents) -> torch.Tensor:
    """Reference signature for one sequence: ``parents`` must describe a chain."""

    n = chain_parents(parents if not torch.is_tensor(parents) else parents.tolist())
    seq_start = torch.tensor([0, n], dtype=torch.int32, device=q.device)
    return gated_delta_chain(q, k, v, g, beta, state.reshape(1, *state.shape[-3:]), seq_start)


def replay(k: torch.Tensor, v: torch.Tensor, g: torch.Tensor, beta: torch.Tensor, state: torch.Tensor,
           seq_start: torch.Tensor, keep: torch.Tensor) -> None:
    """Advance ``state`` in place over the first ``keep[s]`` window rows of every sequence, for one layer
    (k (R, Hk, 128) ...) or for all layers in one launch (k (Layers, R, Hk, 128), state (Layers, S, ...))."""

    _lib.need_cuda(k, v, g, beta, state, seq_start, keep)
    many = k.dim() == 4
    layers = k.shape[0] if many else 1
    r, hk, dk = k.shape[-3:]
    hv, dv = v.shape[-2:]
    s = state.shape[-4]
    if keep.dtype != torch.int32 or keep.shape != (s,) or seq_start.shape != (s + 1,) or state.dtype != torch.float32:
        raise ValueError("replay: keep and seq_start must be int32 per sequence, state fp32")
    for t in (k, v, g, beta, state):
        if not t.is_contiguous():
            raise ValueError("replay: tensors must be contiguous")
    with torch.cuda.device(k.device):
        _lib.check(_lib.load().tf_gdn_replay(k.data_ptr(), v.data_ptr(), g.data_ptr(), beta.data_ptr(), state.data_ptr(),
                                             seq_start.data_ptr(), keep.data_ptr(), s, layers, r * hk * dk, r * hv * dv,
                                             r * hv, s * hv * dv * dk, hk, hv, dk, dv, _lib.stream()), "replay")


replay_path = replay


def conv_commit(qkv: torch.Tensor, conv_state: torch.Tensor, seq_start: torch.Tensor, keep: torch.Tensor, channels: int) -> None:
    """conv_state[s] <- last 3 rows of [conv_state[s]; the first keep[s] window rows], in place.
    ``qkv`` (R, >=C) row views or (Layers, R, >=C); conv_state (S, 3, C) or (Layers, S, 3, C)."""

    many = qkv.dim() == 3
    layers = qkv.shape[0] if many else 1
    s = conv_state.shape[-3]
    with torch.cuda.device(qkv.device):
        _lib.check(_lib.load().tf_conv_commit(qkv.data_ptr(), qkv.stride(-2), qkv.stride(0) if many else 0,
                                              conv_state.data_ptr(), conv_state.stride(0) if many else 0,
                                              seq_start.data_ptr(), keep.data_ptr(), s, layers, channels, _lib.stream()),
                   "conv_commit")


__all__ = ["LaneGDNCache", "chain_parents", "conv_commit", "gated_delta_chain", "gdn_mixer", "gated_delta_tree", "replay", "replay_path"]
