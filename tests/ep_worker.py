"""One rank of the expert-parallel check (launched by test_tp_gpu.py under torchrun, NCCL for the
rendezvous, one GPU each): the MoE block with its experts spread over the ranks gives, on every rank, the
bits of the one-GPU block; a row alone gives the bits it has inside a window."""

import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

from oracle import lane_oracle as O  # noqa: E402
from tensorfold_b200 import _lib, lane_moe  # noqa: E402

D, INTER, E, TOPK, G = 512, 128, 16, 4, 32


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    gen = torch.Generator().manual_seed(31)
    gates = [O.random_q4(gen, INTER, D, G) for _ in range(E + 1)]
    ups = [O.random_q4(gen, INTER, D, G) for _ in range(E + 1)]
    downs = [O.random_q4(gen, D, INTER, G) for _ in range(E + 1)]
    router_rows = (0.05 * torch.randn((E + 1, D), generator=gen)).to(torch.bfloat16).to(dev)
    ep = lane_moe.ExpertGroup(E, TOPK, True, D, dev)
    mine = ep.local_experts(True)
    ex_local = lane_moe.make_experts([gates[i] for i in mine], [ups[i] for i in mine], [downs[i] for i in mine], G, dev)
    ex_full = lane_moe.make_experts(gates, ups, downs, G, dev)
    ok = True
    for rows in (1, 13, 40, 128):
        x = torch.randn((rows, D), generator=gen).to(torch.bfloat16).to(dev)
        buf = lane_moe.MoEBuffers(rows, E, TOPK, True, D, INTER, G, dev)
        got = lane_moe.moe(x, router_rows, ex_local, buf, ep).clone()
        want = lane_moe.moe(x, router_rows, ex_full, lane_moe.MoEBuffers(rows, E, TOPK, True, D, INTER, G, dev)).clone()
        ok &= bool(torch.equal(got.view(torch.int16), want.view(torch.int16)))
        one = lane_moe.MoEBuffers(1, E, TOPK, True, D, INTER, G, dev)
        alone = lane_moe.moe(x[rows // 2:rows // 2 + 1], router_rows, ex_local, one, ep)
        ok &= bool(torch.equal(alone.view(torch.int16), got[rows // 2:rows // 2 + 1].view(torch.int16)))
    torch.cuda.synchronize(dev)
    _lib.status(dev).raise_if_set()
    # One row, no shared expert, many exchanges with no host synchronisation between them: most ranks own no
    # problem in most exchanges, and the odd ranks are slowed by unrelated work, so a fast rank runs ahead as far
    # as the exchange lets it. Every rank's presence cell per exchange is what keeps it from overwriting a slot
    # a slow rank still reads.
    steps = 300
    ep1 = lane_moe.ExpertGroup(E, TOPK, False, D, dev, max_rows=1)
    mine1 = ep1.local_experts(False)
    ex1 = lane_moe.make_experts([gates[i] for i in mine1], [ups[i] for i in mine1], [downs[i] for i in mine1], G, dev)
    ex1_full = lane_moe.make_experts(gates[:E], ups[:E], downs[:E], G, dev)
    xs = torch.randn((steps, 1, D), generator=gen).to(torch.bfloat16).to(dev)
    buf1 = lane_moe.MoEBuffers(1, E, TOPK, False, D, INTER, G, dev)
    ballast = torch.randn((2048, 2048), device=dev)
    got1 = torch.empty((steps, D), dtype=torch.bfloat16, device=dev)
    for i in range(steps):
        if rank % 2 == 1 and i % 3 == 0:
            ballast = torch.tanh(ballast @ ballast) * 0.01
        got1[i] = lane_moe.moe(xs[i], router_rows[:E], ex1, buf1, ep1)[0]
    torch.cuda.synchronize(dev)
    stalled = int(_lib.status(dev).word.item()) != 0
    _lib.status(dev).word.zero_()
    buf1f = lane_moe.MoEBuffers(1, E, TOPK, False, D, INTER, G, dev)
    want1 = torch.stack([lane_moe.moe(xs[i], router_rows[:E], ex1_full, buf1f)[0].clone() for i in range(steps)])
    one_row_ok = (not stalled) and bool(torch.equal(got1.view(torch.int16), want1.view(torch.int16)))
    flag = torch.tensor([int(ok), int(one_row_ok)], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print(f"EP_RESULT world={world} equals_one_gpu={int(flag[0])} one_row_{steps}_exchanges_ok={int(flag[1])}", flush=True)
    dist.barrier()
    # a stalled teardown must not outlive the result
    import threading
    threading.Timer(20, lambda: os._exit(0)).start()
    dist.destroy_process_group()
    os._exit(0)


if __name__ == "__main__":
    main()
