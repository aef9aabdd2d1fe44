"""A verify step as one CUDA-graph replay.

A 27B-class forward is ~700 kernel launches; queued one by one from Python the host becomes the
bottleneck at B200 speeds (the reference meets the same wall and replays one CUDA graph per window,
``families/qwen4_exp/cuda/graphs.py:52-66``). ``LaneRunner`` captures forward + greedy/keyed token
choice for a fixed set of window widths once, and then only rewrites small device tensors (tokens,
positions) between replays. The committed state stays read-only inside the graph; ``commit`` is a
second, tiny graph-free call.
"""

from __future__ import annotations

from typing import Sequence

import torch

from . import _lib, exact_sampling
from .forward import Batch, Record, State, Weights, commit, make_batch, refresh_batch, tree_forward


class LaneRunner:
    def __init__(self, w: Weights, st: State, widths: Sequence[int], *, max_context: int, sampling=None, tp=None, ep=None):
        self.w, self.st, self.tp, self.ep, self.sampling = w, st, tp, ep, sampling
        dev = w.norm.device
        self.device = dev
        for s, wd in enumerate(widths):
            if wd:
                st.kv.reserve(s, max_context + wd)     # pages for the whole run: the captured graph never reallocates
        st.kv.sync_table()
        st.sync_lens()
        from . import lane_attention as LA

        chunks = LA.chunks_for(max_context + max(widths))
        self.batch: Batch = make_batch(st, widths, dev, max_chunks=chunks)
        self.rows = self.batch.rows
        self.tokens = torch.zeros(self.rows, dtype=torch.int32, device=dev)
        self.host_tokens = torch.zeros(self.rows, dtype=torch.int32).pin_memory()
        self.host_out = torch.zeros(self.rows, dtype=torch.int32).pin_memory()
        self.positions = torch.zeros(self.rows, dtype=torch.int64, device=dev)
        self.graph: torch.cuda.CUDAGraph | None = None
        self.record: Record | None = None
        self.logits = self.chosen = None
        self.launches = 0

    def _body(self):
        self.logits, self.record = tree_forward(self.w, self.tokens, None, self.st, batch=self.batch, tp=self.tp, ep=self.ep)
        if self.tp is None:
            self.chosen = exact_sampling.sample_rows(self.logits, self.positions, self.sampling)
        else:
            from .distributed_head import choose_split

            self.chosen = choose_split(self.logits, self.positions, self.sampling, self.tp, self.w.config.vocab)

    def capture(self) -> None:
        """Run the step once eagerly (allocates scratch on the capture stream), then record it."""

        stream = torch.cuda.Stream(self.device)
        stream.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(stream):
            self._body()
            stream.synchronize()
            _lib.status(self.device).raise_if_set()
            before = _lib.launch_count()
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph, stream=stream):
                self._body()
            self.launches = _lib.launch_count() - before
        torch.cuda.current_stream(self.device).wait_stream(stream)

    def refresh(self) -> None:
        """Pick up the state's current lengths (after a commit) for the next replay."""

        refresh_batch(self.batch, self.st)
        self.st.sync_lens()
        pos = self.batch.row_pos.to(torch.int64) + 1            # the token a row verifies sits one past its input
        self.positions.copy_(pos)

    def step_device(self) -> torch.Tensor:
        """Replay with the tokens already in ``self.tokens``; returns the chosen tokens (device)."""

        self.graph.replay()
        return self.chosen

    def step(self, tokens: Sequence[int] | torch.Tensor) -> torch.Tensor:
        """The call a user makes: host tokens in, verified tokens out (pinned host tensor)."""

        if torch.is_tensor(tokens):
            self.host_tokens.copy_(tokens)
        else:
            self.host_tokens.copy_(torch.tensor(list(tokens), dtype=torch.int32))
        self.tokens.copy_(self.host_tokens, non_blocking=True)
        self.graph.replay()
        self.host_out.copy_(self.chosen, non_blocking=True)
        torch.cuda.current_stream(self.device).synchronize()
        return self.host_out

    def commit(self, keep: Sequence[int]) -> None:
        commit(self.st, self.record, keep)
        self.refresh()


__all__ = ["LaneRunner"]
