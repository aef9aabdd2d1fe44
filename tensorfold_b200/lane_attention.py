"""Lane GQA attention over a paged KV cache.

Host-side mirror of the reference's ``lane_sdpa`` / ``lane_tree_sdpa`` / ``lane_attention``
(``kernels/qwen/dense/v1/lane_attention.py:430-550``) and the CUDA ``attention(q, k_nodes, v_nodes,
k_cache, v_cache, parents, scale=...)`` (``families/qwen3_5/cuda/attention.py:152-201``), extended to
the ragged windows of many sequences and to 16-token pages. Chain windows only.
"""

from __future__ import annotations

import torch

from . import _lib

PAGE = 16


def chunks_for(n_keys: int) -> int:
    """Key chunks that hold positions 0..n_keys-1 (128 keys a chunk below 8192, 512 up to 65536, 2048 beyond)."""

    return int(_lib.load().tf_attention_chunks(int(n_keys)))


class PagedKV:
    """Paged K/V storage for ``layers`` attention layers: pages [layer, page, kv_head, 16, D] bf16, one
    page table shared by the layers. Pages are handed out from a host-side free list."""

    def __init__(self, layers: int, n_seqs: int, num_pages: int, kv_heads: int, head_dim: int, max_pages_per_seq: int,
                 device) -> None:
        self.layers, self.n_seqs, self.num_pages = layers, n_seqs, num_pages
        self.kv_heads, self.head_dim, self.max_pages = kv_heads, head_dim, max_pages_per_seq
        shape = (max(layers, 1), num_pages, kv_heads, PAGE, head_dim)
        self.k = torch.zeros(shape, dtype=torch.bfloat16, device=device)
        self.v = torch.zeros(shape, dtype=torch.bfloat16, device=device)
        self.table_host = torch.zeros((n_seqs, max_pages_per_seq), dtype=torch.int32)
        self.table = torch.zeros((n_seqs, max_pages_per_seq), dtype=torch.int32, device=device)
        self.owned = [0] * n_seqs
        self.free = list(range(num_pages - 1, -1, -1))

    def reserve(self, seq: int, tokens: int) -> bool:
        """Make sure sequence ``seq`` owns pages for ``tokens`` positions; True if the table changed."""

        need = -(-tokens // PAGE)
        if need > self.max_pages:
            raise ValueError(f"sequence {seq} needs {need} pages, the table holds {self.max_pages}")
        changed = False
        while self.owned[seq] < need:
            if not self.free:
                raise RuntimeError("out of KV pages")
            self.table_host[seq, self.owned[seq]] = self.free.pop()
            self.owned[seq] += 1
            changed = True
        return changed

    def release(self, seq: int) -> None:
        for i in range(self.owned[seq]):
            self.free.append(int(self.table_host[seq, i]))
        self.owned[seq] = 0

    def sync_table(self) -> None:
        self.table.copy_(self.table_host, non_blocking=True)


def scratch_bytes(rows: int, heads: int, head_dim: int, max_chunks: int) -> int:
    return max_chunks * rows * heads * (head_dim + 2) * 4


def lane_attention(q: torch.Tensor, k_new: torch.Tensor, v_new: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                   page_table: torch.Tensor, seq_lens: torch.Tensor, seq_start: torch.Tensor, row_nkeys: torch.Tensor, *,
                   scale: float, max_window: int, max_chunks: int, scratch: torch.Tensor | None = None,
                   out: torch.Tensor | None = None, gate: torch.Tensor | None = None, packed_out=None) -> torch.Tensor:
    """Attend (R, H, D) queries to each row's sequence: committed pages, then the window rows up to its own.

    k_new, v_new (R, HK, D) window rows; k_pages, v_pages (pages, HK, 16, D); page_table (S, max_pages),
    seq_lens (S,), seq_start (S+1,), row_nkeys (R,) int32 on the device (row_nkeys = committed length +
    place in window + 1). ``max_window`` bounds a sequence's rows, ``max_chunks`` the key chunks
    (``chunks_for`` of the longest key count). ``gate``: the q projection's output rows ([q_h ; gate_h] per
    head, a view with a row stride): the result is multiplied by sigmoid(gate_h). ``packed_out``: a
    ``lane_qmm.Packed`` that receives the result as the output projection's input.
    """

    _lib.need_cuda(q, k_new, v_new, k_pages, v_pages, page_table, seq_lens, seq_start, row_nkeys)
    r, h, d = q.shape
    hk = k_new.shape[1]
    s = seq_lens.shape[0]
    if (q.dtype != torch.bfloat16 or k_new.shape != (r, hk, d) or v_new.shape != k_new.shape or d not in (128, 256)
            or h % hk or h // hk > 16 or k_pages.shape[-3:] != (hk, PAGE, d) or v_pages.shape != k_pages.shape):
        raise ValueError("unsupported attention shape")
    for t in (q, k_new, v_new, k_pages, v_pages, page_table):
        if not t.is_contiguous():
            raise ValueError("attention tensors must be contiguous")
    for t in (page_table, seq_lens, seq_start, row_nkeys):
        if t.dtype != torch.int32:
            raise ValueError("page_table, seq_lens, seq_start and row_nkeys must be int32")
    if not (scale > 0):
        raise ValueError("scale must be positive and finite")
    need = scratch_bytes(r, h, d, max_chunks)
    if scratch is None:
        scratch = torch.empty(need, dtype=torch.uint8, device=q.device)
    if out is None and packed_out is None:
        out = torch.empty_like(q)
    if gate is not None and (gate.dtype != torch.bfloat16 or gate.shape != (r, h * 2 * d) or gate.stride(1) != 1):
        raise ValueError("gate must be the (R, H * 2 * D) bf16 rows of the q projection")
    if packed_out is not None and (packed_out.m != r or packed_out.k != h * d):
        raise ValueError("packed_out must hold R rows of H * D inputs")
    with torch.cuda.device(q.device):
        _lib.check(_lib.load().tf_lane_attention_paged_gated(
            q.data_ptr(), k_new.data_ptr(), v_new.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), page_table.data_ptr(),
            page_table.shape[1], seq_lens.data_ptr(), seq_start.data_ptr(), row_nkeys.data_ptr(), _lib.ptr(out),
            _lib.ptr(gate), gate.stride(0) if gate is not None else 0,
            packed_out.data.data_ptr() if packed_out is not None else None, packed_out.group if packed_out is not None else 64,
            scratch.data_ptr(), scratch.numel(), r, s, max_window, max_chunks, h, hk, d, float(scale),
            _lib.status(q.device).word.data_ptr(), _lib.stream()), "lane_attention")
    return out if out is not None else packed_out


def lane_sdpa(queries: torch.Tensor, keys: torch.Tensor, values: torch.Tensor, scale: float) -> torch.Tensor:
    """Reference shape: the last T rows of one sequence attend causally to (L, HK, D) keys/values, the
    last T of which are their own. Builds a throw-away paged cache; meant for tests and small calls."""

    t, h, d = queries.shape
    l, hk, _ = keys.shape
    committed = l - t
    dev = queries.device
    pages = max(1, -(-committed // PAGE))
    kv = PagedKV(1, 1, pages, hk, d, pages, dev)
    kv.reserve(0, max(committed, 1))
    kv.sync_table()
    if committed:
        pad = pages * PAGE - committed
        kc = torch.cat([keys[:committed], keys.new_zeros((pad, hk, d))]).reshape(pages, PAGE, hk, d).permute(0, 2, 1, 3)
        vc = torch.cat([values[:committed], values.new_zeros((pad, hk, d))]).reshape(pages, PAGE, hk, d).permute(0, 2, 1, 3)
        idx = kv.table_host[0, :pages].to(dev).long()
        kv.k[0, idx] = kc
        kv.v[0, idx] = vc
    seq_lens = torch.tensor([committed], dtype=torch.int32, device=dev)
    seq_start = torch.tensor([0, t], dtype=torch.int32, device=dev)
    nkeys = torch.arange(committed + 1, l + 1, dtype=torch.int32, device=dev)
    return lane_attention(queries.contiguous(), keys[committed:].contiguous(), values[committed:].contiguous(), kv.k[0], kv.v[0],
                          kv.table, seq_lens, seq_start, nkeys, scale=scale, max_window=t, max_chunks=chunks_for(l))


def lane_tree_sdpa(queries: torch.Tensor, keys: torch.Tensor, values: torch.Tensor, scale: float, parents) -> torch.Tensor:
    """The reference's tree form (``lane_attention.lane_tree_sdpa``, ``:462-518``) for the windows this library
    verifies: ``parents`` must describe a chain ([-1, 0, 1, ...]), in which case row t sees the prefix and rows
    0..t and the call is ``lane_sdpa``; a branching tree raises ``ValueError`` (chains only)."""

    parents = [int(p) for p in parents]
    if len(parents) != queries.shape[0] or any(p != i - 1 for i, p in enumerate(parents)):
        raise ValueError("lane_tree_sdpa: only chain windows are supported (parents must be [-1, 0, 1, ...])")
    return lane_sdpa(queries, keys, values, scale)


def kv_commit(k_new: torch.Tensor, v_new: torch.Tensor, kv: PagedKV, seq_lens: torch.Tensor, seq_start: torch.Tensor,
              keep: torch.Tensor) -> None:
    """Write the first keep[s] window rows of every sequence into its pages at positions seq_lens[s]..,
    for all layers at once: k_new, v_new (Layers, R, HK, D)."""

    layers, r, hk, d = k_new.shape
    with torch.cuda.device(k_new.device):
        _lib.check(_lib.load().tf_kv_commit(k_new.data_ptr(), v_new.data_ptr(), r * hk * d, kv.k.data_ptr(), kv.v.data_ptr(),
                                            kv.k.stride(0), kv.table.data_ptr(), kv.max_pages, seq_lens.data_ptr(),
                                            seq_start.data_ptr(), keep.data_ptr(), kv.n_seqs, layers, hk, d, _lib.stream()),
                   "kv_commit")


__all__ = ["PAGE", "chunks_for", "lane_tree_sdpa", "PagedKV", "kv_commit", "lane_attention", "lane_sdpa", "scratch_bytes"]
