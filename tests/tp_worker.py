"""One rank of the tensor-parallel check (launched by test_tp_gpu.py under torchrun, NCCL, one GPU each).

Within a world size the contract is the single-GPU one: the rows of a verify window have the bits of
the same rows decoded one at a time by the same ranks. Across world sizes results differ by rounding
(the reference asserts cosine > 0.999, ``tests/cuda/test_flashnext_tp.py:218-227``); rank 0 also
compares against a one-GPU run of the full model and the chosen tokens of the vocabulary-split head
against the whole-vocabulary draw over the gathered logits.
"""

import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

from oracle import lane_oracle as O  # noqa: E402
from tensorfold_b200 import distributed, forward as F  # noqa: E402
from tensorfold_b200.distributed_head import choose_split  # noqa: E402
from tensorfold_b200.exact_sampling import Sampling, sample_rows  # noqa: E402

SMALL = dict(hidden=1024, intermediate=2048, layers=4, heads=8, kv_heads=2, head_dim=256, vocab=4096, k_heads=8, v_heads=16,
             dk=128, dv=128)


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    cfg = O.Config(**SMALL)
    tp = distributed.RankGroup(exchange=os.environ.get("TP_EXCHANGE", "peer"), hidden=cfg.hidden, device=dev)
    model = O.random_model(cfg, seed=5)                       # the same full model on every rank
    w = F.load_weights(distributed.split_model(model, rank, world), dev)
    gen = torch.Generator().manual_seed(3)
    tokens = torch.randint(0, cfg.vocab, (20,), generator=gen).tolist()

    def run(tokens, windows, st):
        return F.tree_forward(w, torch.tensor(tokens, dtype=torch.int32, device=dev), windows, st, tp=tp)

    st = F.State(w, 1, 256, dev)
    serial = []
    for t in tokens:
        logits, rec = run([t], [-1], st)
        F.commit(st, rec, [1])
        serial.append(logits)
    serial = torch.cat(serial)
    st2 = F.State(w, 1, 256, dev)
    l1, rec = run(tokens[:12], [-1] + list(range(11)), st2)
    F.commit(st2, rec, [12])
    l2, rec = run(tokens[12:], [8], st2)
    window = torch.cat([l1, l2])
    same = bool(torch.equal(window.view(torch.int16), serial.view(torch.int16)))

    # the split head against the whole-vocabulary draw on the gathered logits
    positions = torch.arange(12, 20, device=dev, dtype=torch.int64)
    sampling = Sampling(seed=11, temperature=0.9, top_k=20, top_p=0.95)
    picked = choose_split(l2, positions, sampling, tp, w.config.vocab)
    parts = [torch.empty_like(l2) for _ in range(world)]
    dist.all_gather(parts, l2.contiguous())
    full = torch.cat(parts, dim=-1)
    want = sample_rows(full, positions.tolist(), sampling)
    head_ok = bool(torch.equal(picked.cpu(), want.cpu()))

    cos = 1.0
    if rank == 0:
        w1 = F.load_weights(model, dev)
        st1 = F.State(w1, 1, 256, dev)
        ref, _ = F.tree_forward(w1, torch.tensor(tokens[:12], dtype=torch.int32, device=dev), [-1] + list(range(11)), st1)
    # gather the prefill logits of all ranks for the cross-world comparison
    parts1 = [torch.empty_like(l1) for _ in range(world)]
    dist.all_gather(parts1, l1.contiguous())
    if rank == 0:
        full1 = torch.cat(parts1, dim=-1).float().flatten()
        r = ref.float().flatten()
        cos = float(torch.dot(full1, r) / (full1.norm() * r.norm()))
    # the exchange fused into the matmul epilogue and the norm kernel carries the bits of the plain
    # all-gather + rank-ordered sum (same order, one rounding)
    fused_ok = True
    if tp.exchange == "peer":
        st3 = F.State(w, 1, 256, dev)
        tp_fused = distributed.RankGroup(exchange="peer", hidden=cfg.hidden, device=dev, fused=True)
        tp_nccl = distributed.RankGroup(exchange="nccl")
        for other in (tp_fused, tp_nccl):
            l1n, _ = F.tree_forward(w, torch.tensor(tokens[:12], dtype=torch.int32, device=dev), [-1] + list(range(11)), st3, tp=other)
            fused_ok &= bool(torch.equal(l1n.view(torch.int16), l1.view(torch.int16)))
    flags = torch.tensor([int(same), int(head_ok), int(fused_ok)], device=dev)
    dist.all_reduce(flags, op=dist.ReduceOp.MIN)
    if rank == 0:
        from tensorfold_b200 import _lib
        _lib.status(dev).raise_if_set()
        print(f"TP_RESULT world={world} window_equals_serial={int(flags[0])} head_ok={int(flags[1])} cos_vs_one_gpu={cos:.6f} "
              f"fused_equals_gathered={int(flags[2])} exchange={tp.exchange}", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
