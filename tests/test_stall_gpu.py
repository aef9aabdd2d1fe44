"""Bounded waits that run out: a rank alone against exchange packets nobody sends.

One GPU, one process, one kernel at a time: the exchange kernels are launched as rank 0 of a world of two
whose second buffer is local memory no one writes rank 1's block of. The wait must end by its poll limit,
report TF_ESTALL through the status word, leave the context usable, and the next call must not wait again.
Nothing here faults or hangs the device: the limit is a few thousand polls.
"""

import time

import pytest
import torch

from tensorfold_b200._lib import TF_ESTALL

pytestmark = pytest.mark.gpu



@pytest.fixture()
def lib():
    from tensorfold_b200 import _lib

    handle = _lib.load()
    handle.tf_set_poll_limit(2000)
    yield handle
    handle.tf_set_poll_limit(0)          # 0 restores the default
    _lib.status("cuda:0").word.zero_()


def _world_of_two(lib, rows, d):
    slot = (lib.tf_peer_slot_bytes(rows, d, 2) + 255) // 256 * 256
    bufs = [torch.zeros(2 * slot, dtype=torch.uint8, device="cuda") for _ in range(2)]
    table = torch.tensor([b.data_ptr() for b in bufs], dtype=torch.int64, device="cuda")
    state = torch.zeros(2, dtype=torch.int32, device="cuda")
    return slot, bufs, table, state


def _timed(fn):
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    rc = fn()
    torch.cuda.synchronize()
    return rc, time.perf_counter() - t0


def test_exchange_alone_runs_out_and_reports_a_stall(lib):
    from tensorfold_b200 import _lib

    rows, d = 8, 1024
    slot, bufs, table, state = _world_of_two(lib, rows, d)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    local = torch.randn(rows, d, device="cuda")
    gathered = torch.zeros(2, rows, d, device="cuda")

    def call():
        return lib.tf_peer_exchange(local.data_ptr(), rows, d, table.data_ptr(), slot, gathered.data_ptr(), 0, 2,
                                    state[0:1].data_ptr(), state[1:2].data_ptr(), status.data_ptr(), _lib.stream())

    rc, first = _timed(call)
    assert rc == 0
    assert int(status.item()) == TF_ESTALL
    assert first < 2.0                                   # 2000 polls a thread, not the default four million
    assert torch.equal(gathered[0], local)               # its own block did arrive
    assert int(state[0].item()) == 1                     # the exchange number still advanced: ranks stay in step
    # the status word is sticky: the next exchange sees it and does not poll at all
    rc, second = _timed(call)
    assert rc == 0 and int(status.item()) == TF_ESTALL
    assert second < 0.5
    # the context is alive and, with the status cleared and a peer that does send, the exchange completes
    status.zero_()
    want = int(state[0].item()) + 1
    pkts = bufs[0][(want & 1) * slot:(want & 1) * slot + 2 * rows * d * 8].view(torch.int32).view(2, rows * d // 2, 4)
    theirs = torch.randn(rows, d, device="cuda")
    pkts[1, :, 0] = theirs.view(-1, 2)[:, 0].view(torch.int32)
    pkts[1, :, 2] = theirs.view(-1, 2)[:, 1].view(torch.int32)
    pkts[1, :, 1] = want
    pkts[1, :, 3] = want
    rc, _ = _timed(call)
    assert rc == 0 and int(status.item()) == 0
    assert torch.equal(gathered[0], local) and torch.equal(gathered[1], theirs)


def test_fused_norm_alone_runs_out_and_reports_a_stall(lib):
    from tensorfold_b200 import _lib, lane_qmm

    rows, d = 8, 1024
    slot, bufs, table, state = _world_of_two(lib, rows, d)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    hidden = torch.randn(rows, d, device="cuda").to(torch.bfloat16)
    weight = torch.ones(d, device="cuda", dtype=torch.bfloat16)
    h_out = torch.zeros_like(hidden)
    packed = lane_qmm.new_packed(rows, d, 64, hidden.device)

    def call():
        return lib.tf_norm_xs_peer(hidden.data_ptr(), None, None, 0, 0, weight.data_ptr(), h_out.data_ptr(), None,
                                   packed.data.data_ptr(), rows, d, 64, 1e-6, bufs[0].data_ptr(), slot, state[0:1].data_ptr(),
                                   state[1:2].data_ptr(), 2, status.data_ptr(), _lib.stream())

    rc, first = _timed(call)
    assert rc == 0 and int(status.item()) == TF_ESTALL and first < 2.0
    assert int(state[0].item()) == 1
    rc, second = _timed(call)
    assert rc == 0 and int(status.item()) == TF_ESTALL and second < 0.5
    # and through the host mirror the stall surfaces as an exception at the next sync point
    word = _lib.status("cuda:0")
    word.word.fill_(TF_ESTALL)
    with pytest.raises(RuntimeError, match="TF_ESTALL"):
        word.raise_if_set()
    assert int(word.word.item()) == 0
