"""Row-invariant 4-bit projections on B200: the lane matmul.

Host-side mirror of the reference's ``lane_qmm`` interface (Metal:
``kernels/qwen/dense/v1/lane_qmm.py:244-335``; CUDA: ``families/qwen3_5/cuda/qmm.py:38-144`` and
``qmm_fast.py:80-215``; group 32: ``families/qwen4_exp/cuda/qmm.py:56-125,246-285``). Same names,
argument meaning and errors; the arithmetic is this library's own (see ``csrc/qmm.cu``): one chain
of tensor-core steps per output for every row count, K segments fixed by the weight's shape.

Weights are MLX affine 4-bit: ``(N, K/8)`` uint32 words, element i of a row at bits ``4*(i%8)`` of
word ``i//8``, with ``(N, K/group)`` bf16 scales and biases, group 64 or 32. ``tile_weight`` regroups
them once into the streaming layout the kernel reads (same bits, no information lost;
``untile_weight`` restores the stored layout).
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from . import _lib

MAX_ROWS = 128           # rows one kernel launch accepts (reference: lane_qmm.MAX_ROWS)
WORKERS = 148            # persistent CTAs the K schedule is cut for (a library constant, not the device's SM count)
COLUMN_BLOCK = 256       # output columns per column block
MAX_CUTS_NARROW = 8      # a weight of fewer than 18 column blocks is cut into at most this many items a block


@dataclass
class QWeight:
    """A 4-bit projection in the kernel's tile layout."""

    tiled: torch.Tensor      # uint8, tf_qmm_tiled_bytes(n, k, group)
    n: int
    k: int
    group: int

    def nbytes(self) -> int:
        return self.tiled.numel()

    @property
    def device(self):
        return self.tiled.device


def _check_weight(weight: torch.Tensor, scales: torch.Tensor, biases: torch.Tensor, group: int | None):
    if weight.dim() != 2 or weight.dtype not in (torch.int32, torch.uint32):
        raise ValueError("lane_qmm: weight must be (N, K/8) 32-bit words")
    n, k8 = weight.shape
    k = k8 * 8
    if group is None:
        group = k // scales.shape[1]
    if group not in (32, 64) or k % 64 or scales.shape != (n, k // group) or biases.shape != scales.shape:
        raise ValueError(f"lane_qmm: unsupported weight {tuple(weight.shape)} with scales {tuple(scales.shape)}")
    if scales.dtype != torch.bfloat16 or biases.dtype != torch.bfloat16:
        raise ValueError("lane_qmm: scales and biases must be bf16")
    return n, k, group


def tile_weight(weight: torch.Tensor, scales: torch.Tensor, biases: torch.Tensor, group: int | None = None) -> QWeight:
    """Stored MLX layout -> the kernel's tile layout (one device pass; same bits, new order)."""

    n, k, group = _check_weight(weight, scales, biases, group)
    _lib.need_cuda(weight, scales, biases)
    lib = _lib.load()
    out = torch.empty(lib.tf_qmm_tiled_bytes(n, k, group), dtype=torch.uint8, device=weight.device)
    with torch.cuda.device(weight.device):
        _lib.check(lib.tf_qmm_tile(weight.contiguous().data_ptr(), scales.contiguous().data_ptr(),
                                   biases.contiguous().data_ptr(), out.data_ptr(), n, k, group, _lib.stream()),
                   "tile_weight")
    return QWeight(out, n, k, group)


def untile_weight(q: QWeight) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """``tile_weight`` undone: (words int32 (N, K/8), scales, biases bf16 (N, K/group))."""

    lib = _lib.load()
    dev = q.tiled.device
    words = torch.empty((q.n, q.k // 8), dtype=torch.int32, device=dev)
    scales = torch.empty((q.n, q.k // q.group), dtype=torch.bfloat16, device=dev)
    biases = torch.empty_like(scales)
    with torch.cuda.device(dev):
        _lib.check(lib.tf_qmm_untile(q.tiled.data_ptr(), words.data_ptr(), scales.data_ptr(), biases.data_ptr(),
                                     q.n, q.k, q.group, _lib.stream()), "untile_weight")
    return words, scales, biases


def pack_scales(scales: torch.Tensor, biases: torch.Tensor) -> torch.Tensor:
    """(N, K/g) scales and biases -> (K/g, N, 2) bf16 pairs, group-major (the reference's helper;
    this library keeps the pairs inside the tiled weight instead)."""

    return torch.stack([scales.t(), biases.t()], dim=-1).to(torch.bfloat16).contiguous()


def segments(n: int, k: int) -> list[list[tuple[int, int]]]:
    """The K schedule: for each 256-column block, the k-tile ranges (64 inputs a tile) whose sums are
    formed separately and then added in order. A function of the shape and the worker count only —
    never of the row count."""

    kt = k // 64
    cb = -(-n // COLUMN_BLOCK)
    kts = -(-kt // MAX_CUTS_NARROW) if cb * MAX_CUTS_NARROW < WORKERS else 1     # k tiles per schedule item
    spb = -(-kt // kts)
    total = cb * spb
    bounds = [i * total // WORKERS for i in range(WORKERS + 1)]
    out: list[list[tuple[int, int]]] = [[] for _ in range(cb)]
    for i in range(WORKERS):
        it = bounds[i]
        while it < bounds[i + 1]:
            c = it // spb
            end = min((c + 1) * spb, bounds[i + 1])
            out[c].append(((it - c * spb) * kts, min(kt, (end - c * spb) * kts)))
            it = end
    return out


def split_k(n: int, k: int) -> int:
    """K segments an (n, k) weight's columns are summed in (the most any column block gets):
    fixed by the shape, never by the row count (reference: ``lane_qmm.split_k``)."""

    return max(len(s) for s in segments(n, k))


@dataclass
class Packed:
    """M activation rows in the form the lane matmul reads (``tf_pack_rows``): per 64-input k tile,
    the rows' 128-byte slices, then that tile's group sums. Glue kernels write it directly."""

    data: torch.Tensor       # uint8, tf_packed_bytes(m, k, group)
    m: int
    k: int
    group: int


def padded_rows(m: int) -> int:
    """Rows a packed buffer holds for m rows: the row bucket (8, 16, 32, 64, 128) the kernel runs m in."""

    for b in (8, 16, 32, 64, 128):
        if m <= b:
            return b
    raise ValueError(f"at most {MAX_ROWS} rows per packed buffer, got {m}")


def packed_bytes(m: int, k: int, group: int) -> int:
    return (k // 64) * padded_rows(m) * (128 + 4 * (64 // group))


def new_packed(m: int, k: int, group: int, device) -> Packed:
    return Packed(torch.empty(packed_bytes(m, k, group), dtype=torch.uint8, device=device), m, k, group)


def pack_rows(x: torch.Tensor, group: int = 64, *, want_sums: bool = False):
    """(M, K) bf16 row-major -> ``Packed`` (and, with ``want_sums``, the (M, K/group) fp32 group sums)."""

    if x.dim() != 2 or x.dtype != torch.bfloat16:
        raise ValueError("pack_rows: x must be a 2-D bf16 tensor")
    _lib.need_cuda(x)
    m, k = x.shape
    if m < 1 or k % 64 or group not in (32, 64):
        raise ValueError(f"pack_rows: unsupported shape {tuple(x.shape)} / group {group}")
    x = x.contiguous()
    out = new_packed(m, k, group, x.device)
    xs = torch.empty((m, k // group), dtype=torch.float32, device=x.device) if want_sums else None
    with torch.cuda.device(x.device):
        _lib.check(_lib.load().tf_pack_rows(x.data_ptr(), out.data.data_ptr(), _lib.ptr(xs), m, k, group,
                                            _lib.stream()), "pack_rows")
    return (out, xs) if want_sums else out


def group_sums(x: torch.Tensor, group: int = 64) -> torch.Tensor:
    """(M, K) bf16 -> (M, K/group) fp32 sums of each input group (reference: ``qmm.group_sums``)."""

    return pack_rows(x, group, want_sums=True)[1]


_scratch: dict[tuple[int, int], torch.Tensor] = {}


def scratch_for(device: torch.device) -> torch.Tensor:
    """Per (device, stream) matmul scratch (zeroed once): parked K segments, their ready tags, launch numbers."""

    key = (device.index or 0, torch.cuda.current_stream(device).cuda_stream)
    buf = _scratch.get(key)
    if buf is None:
        buf = torch.zeros(_lib.load().tf_qmm_scratch_bytes(), dtype=torch.uint8, device=device)
        _scratch[key] = buf
    return buf


_tiled_cache: dict[tuple, QWeight] = {}


def _as_qweight(weight, scales, biases) -> QWeight:
    """The reference's call shape: stored words + scales + biases. Tiled once per (words, scales, biases)
    storage and remembered, as the reference remembers its regrouped weights."""

    key = (weight.data_ptr(), scales.data_ptr(), biases.data_ptr(), tuple(weight.shape))
    q = _tiled_cache.get(key)
    if q is None:
        q = _tiled_cache[key] = tile_weight(weight, scales, biases)
    return q


def lane_matmul(x: torch.Tensor | Packed, weight, scales: torch.Tensor | None = None, biases: torch.Tensor | None = None, *,
                xs: torch.Tensor | None = None, sk: int | None = None, f32: bool = False,
                out: torch.Tensor | None = None, next_weight: QWeight | None = None, peer=None,
                act_out: Packed | None = None) -> torch.Tensor:
    """x (..., K) bf16 — or rows already ``Packed`` by the producing kernel — times the 4-bit
    ``weight`` (N, K) transposed -> (..., N) bf16.

    ``weight`` is a ``QWeight`` (tiled once by ``tile_weight``) or, in the reference's call shape
    ``lane_matmul(x, weight, scales, biases, xs=..., sk=...)``, the stored (N, K/8) words with their scales
    and biases (tiled on first use). ``xs`` (the input's group sums) is accepted for that call shape and not
    needed: packing forms the sums; ``sk`` must be None or the shape's own ``split_k``.
    ``f32``: return the unrounded fp32 sums (a tensor-parallel rank's partial). More than
    ``MAX_ROWS`` rows run as several launches; a row's bits do not depend on which launch it rides in.
    ``next_weight``: the weight of the matmul launched next on this stream; its first bytes are pulled
    into L2 while this one finishes (a hint only). ``peer``: a ``distributed.RankGroup`` with the fused
    exchange: the fp32 sums go straight into every rank's exchange buffer (nothing is returned; the next
    ``norm_xs(..., peer=...)`` adds the ranks' partials). ``act_out``: for a stacked [gate; up] weight with columns
    interleaved by 16-column tile and at most 8 rows: the SwiGLU runs in the matmul's epilogue and its packed result
    (the down projection's input, N / 2 wide) is written to ``act_out``, which is returned - the bits
    ``lane_glue.mlp_act_tiled`` gives on the projection's output.
    """

    lib = _lib.load()
    if not isinstance(weight, QWeight):
        if scales is None or biases is None:
            raise ValueError("lane_matmul: stored words need their scales and biases")
        weight = _as_qweight(weight, scales, biases)
    if sk is not None and sk != split_k(weight.n, weight.k):
        raise ValueError(f"lane_matmul: the K schedule is fixed by the shape (split_k = {split_k(weight.n, weight.k)}), got sk={sk}")
    if isinstance(x, Packed):
        if x.k != weight.k or x.group != weight.group:
            raise ValueError(f"lane_matmul: packed rows (K={x.k}, group {x.group}) do not match the weight "
                             f"(K={weight.k}, group {weight.group})")
        if x.m > MAX_ROWS:
            raise ValueError(f"lane_matmul: packed input holds {x.m} rows, at most {MAX_ROWS} per call")
        chunks, lead, m, dev = [x], (x.m,), x.m, x.data.device
    else:
        if x.dtype != torch.bfloat16:
            raise ValueError("lane_matmul: x must be bf16")
        if x.shape[-1] != weight.k:
            raise ValueError(f"lane_matmul: weight (N={weight.n}, K={weight.k}) does not match K={x.shape[-1]}")
        _lib.need_cuda(x)
        lead, dev = x.shape[:-1], x.device
        x2 = x.reshape(-1, weight.k)
        m = x2.shape[0]
        if m < 1:
            raise ValueError("lane_matmul: needs at least one row")
        chunks = [pack_rows(x2[r0:r0 + MAX_ROWS], weight.group) for r0 in range(0, m, MAX_ROWS)]
    if peer is not None:
        if len(chunks) != 1:
            raise ValueError("lane_matmul: a tensor-parallel partial is at most MAX_ROWS rows")
        bufs, slot_bytes, seq, _, _ = peer.peer_args()
        nw = next_weight
        with torch.cuda.device(dev):
            scratch = scratch_for(dev)
            _lib.check(lib.tf_qmm_peer(chunks[0].data.data_ptr(), weight.tiled.data_ptr(), scratch.data_ptr(), scratch.numel(), m,
                                       weight.n, weight.k, weight.group, bufs, slot_bytes, seq, peer.rank, peer.world,
                                       nw.tiled.data_ptr() if nw is not None else None, nw.n if nw is not None else 0,
                                       nw.k if nw is not None else 0, nw.group if nw is not None else 0,
                                       _lib.status(dev).word.data_ptr(), _lib.stream()), "lane_matmul (peer)")
        return None
    if act_out is not None:
        if len(chunks) != 1 or m > 8 or weight.n % 32 or act_out.m != m or act_out.k != weight.n // 2 or act_out.group != weight.group:
            raise ValueError("lane_matmul: act_out needs at most 8 rows and a packed buffer of N / 2 inputs")
        nw = next_weight
        with torch.cuda.device(dev):
            scratch = scratch_for(dev)
            _lib.check(lib.tf_qmm_act(chunks[0].data.data_ptr(), weight.tiled.data_ptr(), act_out.data.data_ptr(), scratch.data_ptr(),
                                      scratch.numel(), m, weight.n, weight.k, weight.group,
                                      nw.tiled.data_ptr() if nw is not None else None, nw.n if nw is not None else 0,
                                      nw.k if nw is not None else 0, nw.group if nw is not None else 0,
                                      _lib.status(dev).word.data_ptr(), _lib.stream()), "lane_matmul (act)")
        return act_out
    dtype = torch.float32 if f32 else torch.bfloat16
    if out is None:
        out = torch.empty((m, weight.n), dtype=dtype, device=dev)
    elif out.shape != (m, weight.n) or out.dtype != dtype or not out.is_contiguous():
        raise ValueError("lane_matmul: out has the wrong shape or dtype")
    scratch = scratch_for(dev)
    st = _lib.status(dev)
    with torch.cuda.device(dev):
        r0 = 0
        for c in chunks:
            nw = next_weight if c is chunks[-1] else weight
            _lib.check(lib.tf_qmm_next(c.data.data_ptr(), weight.tiled.data_ptr(), out[r0:r0 + c.m].data_ptr(),
                                       scratch.data_ptr(), scratch.numel(), c.m, weight.n, weight.k, weight.group,
                                       1 if f32 else 0, nw.tiled.data_ptr() if nw is not None else None,
                                       nw.n if nw is not None else 0, nw.k if nw is not None else 0,
                                       nw.group if nw is not None else 0, st.word.data_ptr(), _lib.stream()), "lane_matmul")
            r0 += c.m
    return out.reshape(*lead, weight.n)


__all__ = ["MAX_ROWS", "Packed", "QWeight", "group_sums", "lane_matmul", "new_packed", "pack_rows", "pack_scales",
           "packed_bytes", "segments", "split_k", "tile_weight", "untile_weight"]
