"""The round loop around the verify forward: serial decoding, and drafted decoding in which each round
verifies a chain of guessed tokens per sequence, keeps the matching prefix and commits it.

Mirror of the reference's ``families/qwen3_5/cuda/decode.py:83-100`` (``serial_decode``) and
``:188-281`` (``draft_decode``) for chain windows, extended to many ragged sequences decoded together
(one forward a round over all of them). Because a window row has the bits of the serial step at its
position and the draw is keyed by (seed, position, token id), the drafted run emits exactly the serial
run's tokens, whatever the drafter proposes; only the number of rounds changes.
"""

from __future__ import annotations

import hashlib
import time
from dataclasses import dataclass, field
from typing import Callable, Sequence

import torch

from .exact_sampling import Sampling, sample_rows
from .forward import State, Weights, accept_path, commit, tree_forward
from .lane_qmm import MAX_ROWS


@dataclass
class DecodeResult:
    tokens: list                       # per sequence: the pending token, then what was generated
    seconds: float
    rounds: int
    drafted_rows: int = 0
    accepted_drafts: int = 0
    widths: list = field(default_factory=list)

    def sha256(self) -> str:
        """Digest of all sequences' tokens (the reference compares serial and drafted runs this way)."""

        h = hashlib.sha256()
        for seq in self.tokens:
            h.update(",".join(str(int(t)) for t in seq).encode() + b";")
        return h.hexdigest()


class CopyIndex:
    """N-gram copy drafter: where each ``min_match``-gram of a context last occurred. ``propose`` returns
    the continuation after the latest earlier occurrence of the context's last ``min_match`` tokens
    (reference: ``decode.CopyIndex`` / ``copy_chain``)."""

    def __init__(self, min_match: int = 2):
        self.n = min_match
        self.where: dict[tuple, int] = {}
        self.seen = 0

    def propose(self, context: Sequence[int], max_nodes: int) -> list:
        n = self.n
        # index every n-gram that ends before the last position (the last one is the query)
        while self.seen + n <= len(context) - 1:
            self.where[tuple(context[self.seen:self.seen + n])] = self.seen + n
            self.seen += 1
        if len(context) < n or max_nodes < 1:
            return []
        at = self.where.get(tuple(context[-n:]))
        if at is None:
            return []
        out = list(context[at:at + max_nodes])
        return out if len(out) >= 1 else []


def _tokens(rows: Sequence[int], device) -> torch.Tensor:
    return torch.tensor(list(rows), dtype=torch.int32, device=device)


@torch.no_grad()
def prefill(w: Weights, st: State, prompts: Sequence[Sequence[int]], sampling: Sampling | None = None, chunk: int = 8) -> list:
    """Run the prompts through the lane forward, ``chunk`` rows per sequence a round, committing every
    row; returns each sequence's first sampled token (the "pending" token of the decode loops)."""

    dev = w.norm.device
    n = st.n_seqs
    if len(prompts) != n or any(len(p) < 1 for p in prompts):
        raise ValueError("one non-empty prompt per sequence")
    done = [0] * n
    pending = [0] * n
    while any(done[s] < len(prompts[s]) for s in range(n)):
        widths = [min(chunk, len(prompts[s]) - done[s]) for s in range(n)]
        while sum(widths) > MAX_ROWS:
            widths[widths.index(max(widths))] -= 1
        rows = [t for s in range(n) for t in prompts[s][done[s]:done[s] + widths[s]]]
        logits, rec = tree_forward(w, _tokens(rows, dev), widths, st)
        ends, r = [], 0
        for s in range(n):
            r += widths[s]
            ends.append(r - 1)
        finishing = [s for s in range(n) if widths[s] and done[s] + widths[s] == len(prompts[s])]
        if finishing:
            idx = torch.tensor([ends[s] for s in finishing], device=dev)
            picked = sample_rows(logits[idx].contiguous(), [len(prompts[s]) for s in finishing], sampling).tolist()
            for s, t in zip(finishing, picked):
                pending[s] = int(t)
        commit(st, rec, widths)
        for s in range(n):
            done[s] += widths[s]
    return pending


@torch.no_grad()
def serial_decode(w: Weights, st: State, pending: Sequence[int], count: int, sampling: Sampling | None = None) -> DecodeResult:
    """One row per sequence and round: the baseline every drafted run must reproduce token for token."""

    if count < 1:
        raise ValueError("count must include the first sampled token")
    dev = w.norm.device
    n = st.n_seqs
    out = [[int(p)] for p in pending]
    start = time.perf_counter()
    rounds = 0
    while len(out[0]) < count:
        logits, rec = tree_forward(w, _tokens([o[-1] for o in out], dev), [1] * n, st)
        nxt = sample_rows(logits, [st.lens[s] + 1 for s in range(n)], sampling).tolist()
        commit(st, rec, [1] * n)
        for s in range(n):
            out[s].append(int(nxt[s]))
        rounds += 1
    torch.cuda.synchronize(dev)
    return DecodeResult(out, time.perf_counter() - start, rounds, widths=[n] * rounds)


@torch.no_grad()
def draft_decode(w: Weights, st: State, prompts: Sequence[Sequence[int]], pending: Sequence[int], count: int,
                 sampling: Sampling | None = None, *, max_rows: int = 8,
                 draft: Callable[[int, Sequence[int], int], Sequence[int]] | None = None) -> DecodeResult:
    """Each round: per sequence a chain [last token, guesses...] of up to ``max_rows`` rows is verified in
    one forward over all sequences; the rows whose input token matched what the target chose are kept
    and committed, and the target's own token after the last kept row is appended.

    ``draft(seq, context, k)`` proposes up to k next tokens for a sequence; by default an n-gram copy of
    the sequence's own context (``CopyIndex``). A sequence that reached ``count`` tokens rides along with
    an empty window.
    """

    if count < 1 or not 1 <= max_rows <= MAX_ROWS:
        raise ValueError(f"count >= 1 and 1 <= max_rows <= {MAX_ROWS} required")
    dev = w.norm.device
    n = st.n_seqs
    out = [[int(p)] for p in pending]
    context = [list(prompts[s]) + out[s] for s in range(n)]
    copies = [CopyIndex() for _ in range(n)]
    rounds = drafted = accepted = 0
    widths_log = []
    start = time.perf_counter()
    while any(len(o) < count for o in out):
        budget = max(1, MAX_ROWS // max(1, sum(len(o) < count for o in out)))
        windows, rows = [], []
        for s in range(n):
            if len(out[s]) >= count:
                windows.append([])
                continue
            k = min(max_rows, budget, count - len(out[s])) - 1
            guesses = list(draft(s, context[s], k) if draft is not None else copies[s].propose(context[s], k))[:max(k, 0)]
            windows.append([out[s][-1]] + [int(g) for g in guesses])
        widths = [len(wd) for wd in windows]
        rows = [t for wd in windows for t in wd]
        logits, rec = tree_forward(w, _tokens(rows, dev), widths, st)
        positions = [st.lens[s] + t + 1 for s in range(n) for t in range(widths[s])]
        verified = sample_rows(logits, positions, sampling).tolist()
        keep, r = [], 0
        for s in range(n):
            if not widths[s]:
                keep.append(0)
                continue
            v = verified[r:r + widths[s]]
            k = accept_path(windows[s], v)
            new = windows[s][1:k] + [int(v[k - 1])]
            out[s].extend(new)
            context[s].extend(new)
            keep.append(k)
            drafted += widths[s] - 1
            accepted += k - 1
            r += widths[s]
        commit(st, rec, keep)
        rounds += 1
        widths_log.append(sum(widths))
    torch.cuda.synchronize(dev)
    return DecodeResult([o[:count] for o in out], time.perf_counter() - start, rounds, drafted, accepted, widths_log)


class Engine:
    """The engine contract the reference's server drives (``cuda/server.py:9-15``): ``eos`` and
    ``generate(prompt, max_tokens, sampling, on_tokens) -> dict`` for one request at a time, decoded as one
    exact stream: prefill through the lane forward, then drafted rounds (n-gram copy drafter) whose output is
    token for token what serial decoding gives. A prompt that extends the previous request's reuses its
    committed state (``State.snapshot`` / ``restore`` at the end of the shared prefix is the caller's tool for
    anything finer)."""

    def __init__(self, w: Weights, *, max_context: int = 8192, eos: Sequence[int] = (), max_rows: int = 8):
        self.w, self.eos, self.max_rows, self.max_context = w, tuple(int(t) for t in eos), max_rows, max_context
        self.state = State(w, 1, max_context)
        self.committed: list = []              # tokens whose state is committed

    def _reset(self) -> None:
        self.state.kv.release(0)
        self.state = State(self.w, 1, self.max_context)
        self.committed = []

    def generate(self, prompt: Sequence[int], max_tokens: int, sampling: Sampling | None = None,
                 on_tokens: Callable[[list], bool] | None = None) -> dict:
        prompt = [int(t) for t in prompt]
        if not prompt or max_tokens < 1 or len(prompt) + max_tokens > self.max_context:
            raise ValueError("generate: needs a non-empty prompt that fits the context with max_tokens")
        keep = len(self.committed)
        if keep == 0 or keep >= len(prompt) or prompt[:keep] != self.committed:
            self._reset()
            keep = 0
        start = time.perf_counter()
        pending = prefill(self.w, self.state, [prompt[keep:]], sampling)[0] if keep == 0 else None
        if pending is None:
            # the shared prefix is committed already: only the new tail runs; positions continue from it
            pending = _prefill_tail(self.w, self.state, prompt[keep:], sampling)
        self.committed = list(prompt)
        out = [int(pending)]
        stopped = bool(on_tokens(list(out))) if on_tokens else False
        rounds = 0
        while not stopped and len(out) < max_tokens and out[-1] not in self.eos:
            want = min(max_tokens - len(out) + 1, 4 * self.max_rows)
            res = draft_decode(self.w, self.state, [self.committed], [out[-1]], want, sampling, max_rows=self.max_rows)
            new = res.tokens[0][1:]
            for i, t in enumerate(new):                # stop at the first end token
                if t in self.eos:
                    new = new[:i + 1]
                    break
            # draft_decode committed every token it emitted but the last: mirror that in the bookkeeping
            self.committed.extend([out[-1]] + res.tokens[0][1:-1])
            if len(new) < len(res.tokens[0]) - 1:
                self._reset()                          # tokens past the end token were committed: start clean next time
            out.extend(new)
            rounds += res.rounds
            if on_tokens and new:
                stopped = bool(on_tokens(list(new)))
        return {"tokens": out[:max_tokens], "seconds": time.perf_counter() - start, "rounds": rounds, "prompt_tokens": len(prompt)}


def _prefill_tail(w: Weights, st: State, tail: Sequence[int], sampling: Sampling | None, chunk: int = 8) -> int:
    dev = w.norm.device
    done, pending = 0, 0
    while done < len(tail):
        n = min(chunk, len(tail) - done)
        logits, rec = tree_forward(w, _tokens(tail[done:done + n], dev), [n], st)
        if done + n == len(tail):
            pending = int(sample_rows(logits[n - 1:n].contiguous(), [st.lens[0] + n], sampling).tolist()[0])
        commit(st, rec, [n])
        done += n
    return pending


__all__ = ["CopyIndex", "DecodeResult", "Engine", "draft_decode", "prefill", "serial_decode"]
