"""The round loop: drafted decoding emits the serial run's tokens, whatever the drafter proposes.

Pattern of the reference's ``tests/cuda/test_qwen27_decode.py`` (serial vs drafted token equality, digest
compare) extended to several ragged sequences decoded together.
"""

import pytest
import torch

from oracle import lane_oracle as O

pytestmark = pytest.mark.gpu

TINY = dict(hidden=256, intermediate=512, layers=4, heads=4, kv_heads=2, head_dim=128, vocab=512, k_heads=2, v_heads=4,
            dk=128, dv=128)


@pytest.fixture(scope="module")
def setup(lib):
    from tensorfold_b200 import decode, forward as F
    from tensorfold_b200.exact_sampling import Sampling

    w = F.load_weights(O.random_model(O.Config(**TINY), seed=41), "cuda")
    gen = torch.Generator().manual_seed(9)
    prompts = [torch.randint(0, TINY["vocab"], (n,), generator=gen).tolist() for n in (5, 19, 33)]
    return decode, F, Sampling, w, prompts


@pytest.mark.parametrize("sampled", [False, True])
def test_drafted_tokens_equal_serial_tokens(setup, sampled):
    decode, F, Sampling, w, prompts = setup
    sampling = Sampling(seed=5, temperature=0.8, top_k=20, top_p=0.95) if sampled else None
    count = 24

    def fresh():
        st = F.State(w, len(prompts), 256)
        return st, decode.prefill(w, st, prompts, sampling)

    st, pending = fresh()
    serial = decode.serial_decode(w, st, pending, count, sampling)
    assert all(len(t) == count for t in serial.tokens)

    # a drafter that knows the serial answer but gets every fourth guess wrong: hits, misses, full windows
    def teacher(seq, context, k):
        done = len(context) - len(prompts[seq])
        guess = list(serial.tokens[seq][done:done + k])
        return [(t + 1) % TINY["vocab"] if (done + i) % 4 == 3 else t for i, t in enumerate(guess)]

    st, pending2 = fresh()
    assert pending2 == pending
    drafted = decode.draft_decode(w, st, prompts, pending2, count, sampling, max_rows=8, draft=teacher)
    assert drafted.tokens == serial.tokens
    assert drafted.sha256() == serial.sha256()
    assert drafted.accepted_drafts > 0 and drafted.rounds < serial.rounds
    assert drafted.accepted_drafts < drafted.drafted_rows          # some guesses were rejected

    # a drafter that is always wrong changes nothing but the number of rounds
    st, pending3 = fresh()
    wrong = decode.draft_decode(w, st, prompts, pending3, count, sampling, max_rows=4,
                                draft=lambda seq, context, k: [(context[-1] + 7) % TINY["vocab"]] * k)
    assert wrong.tokens == serial.tokens and wrong.accepted_drafts <= 2

    # the default n-gram copy drafter
    st, pending4 = fresh()
    copied = decode.draft_decode(w, st, prompts, pending4, count, sampling, max_rows=8)
    assert copied.sha256() == serial.sha256()


def test_snapshot_restore_and_generate(setup):
    """``State.snapshot`` / ``restore`` (reference: families/qwen4_exp/cuda/forward.py:200-222) bring the sequences
    back bit for bit, refuse a snapshot of other kernels, and ``Engine.generate`` (the contract of cuda/server.py:9-15)
    emits the serial tokens, streams them through ``on_tokens`` and reuses a committed prefix."""

    decode, F, Sampling, w, prompts = setup
    sampling = Sampling(seed=3, temperature=0.7, top_k=20, top_p=0.9)
    st = F.State(w, len(prompts), 256)
    pending = decode.prefill(w, st, prompts, sampling)
    snap = st.snapshot()
    first = decode.serial_decode(w, st, pending, 10, sampling)
    st.restore(snap)
    again = decode.serial_decode(w, st, pending, 10, sampling)
    assert first.tokens == again.tokens
    with pytest.raises(ValueError):
        st.restore(dict(snap, kernels="another build"))

    # one request at a time through the engine
    st1 = F.State(w, 1, 256)
    p1 = decode.prefill(w, st1, [prompts[1]], sampling)
    want = decode.serial_decode(w, st1, p1, 20, sampling).tokens[0]
    eng = decode.Engine(w, max_context=256)
    seen = []
    got = eng.generate(prompts[1], 20, sampling, on_tokens=lambda new: seen.extend(new) or False)
    assert got["tokens"] == want and seen == want and got["prompt_tokens"] == len(prompts[1])
    # a follow-up whose prompt extends the finished exchange reuses the committed prefix
    longer = prompts[1] + want[:12]
    st2 = F.State(w, 1, 256)
    p2 = decode.prefill(w, st2, [longer], sampling)
    want2 = decode.serial_decode(w, st2, p2, 8, sampling).tokens[0]
    assert eng.generate(longer, 8, sampling)["tokens"] == want2
    # stopping early through the callback
    short = decode.Engine(w, max_context=256).generate(prompts[0], 20, sampling, on_tokens=lambda new: True)
    assert len(short["tokens"]) == 1
