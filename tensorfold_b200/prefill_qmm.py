"""Wide-row 4-bit projections on the tcgen05 tensor cores.

The reference runs prompt prefill and many-row windows through its lane kernels in chains of up to 128
rows (``families/qwen3_5/cuda/decode.py:34-60``); this module is this library's own wide-row path:
the same 4-bit weights, regrouped for ``csrc/qmm_tc.cu``, dequantised to bf16 in flight and multiplied on
``tcgen05.mma`` (bf16 x bf16 -> fp32 in tensor memory). A row's bits are independent of the other rows
in the call, but they are this kernel's bits, not the lane kernel's: an engine runs all its steps through
one of the two.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from . import _lib
from .lane_qmm import MAX_ROWS, _check_weight, scratch_for


@dataclass
class TCWeight:
    """A 4-bit projection in the prefill kernel's tile layout."""

    tiled: torch.Tensor      # uint8, tf_qmm_tc_tiled_bytes(n, k, group)
    n: int
    k: int
    group: int


def tile_weight(weight: torch.Tensor, scales: torch.Tensor, biases: torch.Tensor, group: int | None = None) -> TCWeight:
    """Stored MLX layout -> the prefill kernel's tile layout (same bits, new order)."""

    n, k, group = _check_weight(weight, scales, biases, group)
    _lib.need_cuda(weight, scales, biases)
    lib = _lib.load()
    out = torch.empty(lib.tf_qmm_tc_tiled_bytes(n, k, group), dtype=torch.uint8, device=weight.device)
    with torch.cuda.device(weight.device):
        _lib.check(lib.tf_qmm_tc_tile(weight.contiguous().data_ptr(), scales.contiguous().data_ptr(),
                                      biases.contiguous().data_ptr(), out.data_ptr(), n, k, group, _lib.stream()),
                   "prefill tile_weight")
    return TCWeight(out, n, k, group)


def untile_weight(q: TCWeight) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    lib = _lib.load()
    dev = q.tiled.device
    words = torch.empty((q.n, q.k // 8), dtype=torch.int32, device=dev)
    scales = torch.empty((q.n, q.k // q.group), dtype=torch.bfloat16, device=dev)
    biases = torch.empty_like(scales)
    with torch.cuda.device(dev):
        _lib.check(lib.tf_qmm_tc_untile(q.tiled.data_ptr(), words.data_ptr(), scales.data_ptr(), biases.data_ptr(),
                                        q.n, q.k, q.group, _lib.stream()), "prefill untile_weight")
    return words, scales, biases


def packed_bytes(rows: int, k: int, group: int) -> int:
    return int(_lib.load().tf_packed_tc_bytes(rows, k, group))


def prefill_matmul(x, weight: TCWeight, *, f32: bool = False, out: torch.Tensor | None = None,
                   staging: torch.Tensor | None = None) -> torch.Tensor:
    """x (..., K) bf16 (or a ``lane_qmm.Packed``: the rows every glue kernel writes, at most ``MAX_ROWS``)
    times the 4-bit ``weight`` (N, K) transposed -> (..., N), in launches of up to ``MAX_ROWS`` rows.
    ``staging``: a uint8 buffer of ``packed_bytes(rows, K, group)`` for the regrouped rows (so that a
    captured step allocates nothing)."""

    from .lane_qmm import Packed

    lib = _lib.load()
    if isinstance(x, Packed):
        if x.k != weight.k or x.group != weight.group:
            raise ValueError("prefill_matmul: packed rows do not match the weight")
        dev, m, lead = x.data.device, x.m, (x.m,)
        x2 = None
    else:
        if x.dtype != torch.bfloat16:
            raise ValueError("prefill_matmul: x must be bf16")
        if x.shape[-1] != weight.k:
            raise ValueError(f"prefill_matmul: weight (N={weight.n}, K={weight.k}) does not match K={x.shape[-1]}")
        _lib.need_cuda(x)
        lead, dev = x.shape[:-1], x.device
        x2 = x.reshape(-1, weight.k).contiguous()
        m = x2.shape[0]
    if m < 1:
        raise ValueError("prefill_matmul: needs at least one row")
    dtype = torch.float32 if f32 else torch.bfloat16
    if out is None:
        out = torch.empty((m, weight.n), dtype=dtype, device=dev)
    elif out.shape != (m, weight.n) or out.dtype != dtype or not out.is_contiguous():
        raise ValueError("prefill_matmul: out has the wrong shape or dtype")
    scratch = scratch_for(dev)
    st = _lib.status(dev)
    with torch.cuda.device(dev):
        for r0 in range(0, m, MAX_ROWS):
            rows = min(MAX_ROWS, m - r0)
            need = lib.tf_packed_tc_bytes(rows, weight.k, weight.group)
            packed = staging if staging is not None else torch.empty(need, dtype=torch.uint8, device=dev)
            if packed.numel() < need:
                raise ValueError("prefill_matmul: staging buffer too small")
            if x2 is None:
                _lib.check(lib.tf_repack_tc(x.data.data_ptr(), packed.data_ptr(), rows, weight.k, weight.group, _lib.stream()),
                           "prefill repack")
            else:
                _lib.check(lib.tf_pack_rows_tc(x2[r0:r0 + rows].data_ptr(), packed.data_ptr(), None, rows, weight.k,
                                               weight.group, _lib.stream()), "prefill pack_rows")
            _lib.check(lib.tf_qmm_tc(packed.data_ptr(), weight.tiled.data_ptr(), out[r0:r0 + rows].data_ptr(),
                                     scratch.data_ptr(), scratch.numel(), rows, weight.n, weight.k, weight.group,
                                     1 if f32 else 0, st.word.data_ptr(), _lib.stream()), "prefill_matmul")
    return out.reshape(*lead, weight.n)


__all__ = ["TCWeight", "packed_bytes", "prefill_matmul", "tile_weight", "untile_weight"]
