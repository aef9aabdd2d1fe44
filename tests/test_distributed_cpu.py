"""Tensor-parallel host logic without a GPU: the partition map, the rank-ordered partial sum over a
real two-process gloo group, and the vocabulary-split candidate merge.

After the reference's ``tests/cuda/test_qwen27_distributed.py:36-91,140-190`` (partition map on CPU, gloo pair
via ``torch.multiprocessing.spawn``) and ``test_qwen27_split_sampling.py`` (split == whole-vocabulary draw).
"""

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

from oracle import lane_oracle as O
from tensorfold_b200 import distributed as D
from tensorfold_b200 import distributed_head as H
from tensorfold_b200 import exact_sampling as S
from tensorfold_b200.forward import Config

C27 = dict(hidden=5120, intermediate=17408, layers=64, heads=24, kv_heads=4, head_dim=256, vocab=248320, k_heads=16, v_heads=32)


def test_shard_config_splits_heads_and_replicates_kv():
    cfg = Config(**C27)
    assert D.shard_config(cfg, 0, 1) is cfg
    s2, s4, s8 = (D.shard_config(cfg, 0, w) for w in (2, 4, 8))
    assert (s2.heads, s2.kv_heads, s2.k_heads, s2.v_heads, s2.intermediate, s2.vocab) == (12, 2, 8, 16, 8704, 124160)
    assert (s4.heads, s4.kv_heads) == (6, 1)
    assert (s8.heads, s8.kv_heads, s8.intermediate, s8.vocab) == (3, 1, 2176, 31040)     # 4 KV heads on 8 ranks: replicated
    assert [list(D.kv_head_of_rank(cfg, r, 8)) for r in range(8)] == [[0], [0], [1], [1], [2], [2], [3], [3]]
    assert [list(D.kv_head_of_rank(cfg, r, 2)) for r in range(2)] == [[0, 1], [2, 3]]
    # every rank's query heads belong to the KV head it holds
    for r in range(8):
        q_heads = range(r * 3, r * 3 + 3)
        assert {h // 6 for h in q_heads} == set(D.kv_head_of_rank(cfg, r, 8))
    with pytest.raises(ValueError):
        D.shard_config(cfg, 0, 5)
    with pytest.raises(ValueError):
        D.shard_config(cfg, 3, 2)


def test_sum_rank_partials_rounds_once():
    # the reference's example: three small addends survive only if the sum is rounded once, at the end
    a, b = torch.full((2, 4), 1.0), torch.full((2, 4), 0.003)
    parts = torch.stack([a, b, b])
    assert torch.equal(D.sum_rank_partials(parts), (a + b + b).to(torch.bfloat16))
    assert not torch.equal(D.sum_rank_partials(parts), ((a.bfloat16() + b.bfloat16()) + b.bfloat16()))


def _worker(rank, world, port, out):
    import torch.distributed as dist

    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        tp = D.RankGroup()
        local = torch.full((3, 8), float(rank + 1))
        local[0, 0] = 2.0 ** -9 if rank else 1.0
        gathered = tp.gather_partials(local)
        assert gathered.shape == (world, 3, 8)
        total = D.sum_rank_partials(gathered)
        # vocabulary-split greedy pick: rank r holds ids [r*5, r*5+5)
        logits = torch.tensor([[0.0, 1.0, 3.0, 3.0, 2.0]]) if rank == 0 else torch.tensor([[3.0, 0.5, 0.0, 4.0, 4.0]])
        val, idx = logits.max(dim=-1, keepdim=True)
        all_idx = torch.empty((world, 1, 1), dtype=torch.int64)
        all_val = torch.empty((world, 1, 1))
        dist.all_gather_into_tensor(all_idx.view(-1, 1), (idx + rank * 5).contiguous())
        dist.all_gather_into_tensor(all_val.view(-1, 1), val.contiguous())
        midx, _ = H.merge_candidates(all_idx, all_val, 1)
        out[rank] = (gathered[:, 0, 0].tolist(), total[0, 0].item(), int(midx[0, 0]))
    finally:
        dist.destroy_process_group()


def test_gloo_two_ranks_gather_in_rank_order():
    import socket

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    out = mp.Manager().dict()
    mp.spawn(_worker, args=(2, port, out), nprocs=2, join=True)
    for rank in range(2):
        first, total, pick = out[rank]
        assert first == [1.0, 2.0 ** -9]                    # rank 0's partial first on every rank
        assert total == float(torch.tensor(1.0 + 2.0 ** -9).bfloat16())
        assert pick == 8                                    # 4.0 at global ids 8 and 9: the lower id wins


def test_split_vocabulary_candidates_contain_the_whole_vocabulary_draw():
    rng = np.random.default_rng(3)
    vocab, world, rows = 4000, 4, 12
    logits = np.round(rng.normal(size=(rows, vocab)) * 4) / 4
    s = S.Sampling(seed=77, top_k=20, top_p=0.9)
    positions = rng.integers(0, 10000, size=rows)
    whole = O.sample_rows(logits.astype(np.float32), positions, O.Sampling(seed=77, top_k=20, top_p=0.9))
    per = vocab // world
    idx, val = [], []
    for r in range(world):
        i, v = O.topk_rows(logits[:, r * per:(r + 1) * per], 28)
        idx.append(torch.from_numpy(i.astype(np.int64) + r * per)); val.append(torch.from_numpy(v))
    midx, mval = H.merge_candidates(torch.stack(idx), torch.stack(val), 28)
    wi, wv = O.topk_rows(logits, 28)
    assert np.array_equal(midx.numpy(), wi) and np.array_equal(mval.numpy(), wv)
    assert O.choose_rows(mval.numpy(), midx.numpy(), positions, O.Sampling(seed=77, top_k=20, top_p=0.9)) == whole


def test_split_model_shards_reassemble_into_the_stored_model():
    """Column-parallel shards are whole output rows, row-parallel shards whole input groups: stacking
    them back gives the stored arrays (reference: tests/cuda/test_qwen27_tp.py partition checks)."""

    from oracle import lane_oracle as O
    from tensorfold_b200 import distributed as D

    cfg = O.Config(hidden=512, intermediate=1024, layers=4, heads=8, kv_heads=2, head_dim=128, vocab=1024, k_heads=8,
                   v_heads=16, dk=128, dv=128)
    model = O.random_model(cfg, 5)
    for world in (2, 4, 8):
        shards = [D.split_model(model, r, world) for r in range(world)]
        lin, att = model["layers"][0], model["layers"][3]
        assert lin["linear"] and not att["linear"]
        for name in ("gate", "up", "z", "b", "a"):
            assert torch.equal(torch.cat([s["layers"][0][name].words for s in shards]), lin[name].words)
            assert torch.equal(torch.cat([s["layers"][0][name].scales for s in shards]), lin[name].scales)
        for name in ("down", "out"):
            assert torch.equal(torch.cat([s["layers"][0][name].words for s in shards], 1), lin[name].words)
            assert torch.equal(torch.cat([s["layers"][0][name].biases for s in shards], 1), lin[name].biases)
        kd = cfg.k_heads * cfg.dk
        kdl = kd // world
        q_rows = torch.cat([s["layers"][0]["qkv"].words[:kdl] for s in shards])
        assert torch.equal(q_rows, lin["qkv"].words[:kd])
        assert torch.equal(torch.cat([s["layers"][0]["conv"][:kdl] for s in shards]), lin["conv"][:kd])
        assert torch.equal(torch.cat([s["layers"][3]["q"].words for s in shards]), att["q"].words)
        assert torch.equal(torch.cat([s["layers"][3]["o"].words for s in shards], 1), att["o"].words)
        # KV heads: split while they last, then one replicated head per rank
        per = max(1, cfg.kv_heads // world)
        for r, s in enumerate(shards):
            h0 = D.kv_head_of_rank(cfg, r, world).start
            assert torch.equal(s["layers"][3]["k"].words, att["k"].words[h0 * 128:(h0 + per) * 128])
            assert s["config"].kv_heads == per and s["config"].vocab == cfg.vocab // world
        assert torch.equal(torch.cat([s["head"].words for s in shards]), model["head"].words)


def test_copy_drafter_and_digest():
    """Host logic of the round loop (reference: decode.CopyIndex, copy_chain)."""

    from tensorfold_b200.decode import CopyIndex, DecodeResult
    from tensorfold_b200.forward import accept_path

    ctx = [1, 2, 3, 4, 9, 9, 1, 2, 3]
    idx = CopyIndex(min_match=2)
    assert idx.propose(ctx, 3) == [4, 9, 9]              # continuation after the earlier "2 3"
    ctx += [4, 9]
    assert idx.propose(ctx, 2) == [9, 1]                 # the index follows the growing context
    assert CopyIndex().propose([5, 6, 7], 4) == []       # nothing seen twice
    assert accept_path([10, 11, 12, 13], [11, 12, 99, 7]) == 3
    assert accept_path([10, 11], [5, 5]) == 1
    a, b = DecodeResult([[1, 2], [3]], 0.0, 1), DecodeResult([[1, 2], [3]], 1.0, 2)
    assert a.sha256() == b.sha256() != DecodeResult([[1, 2, 3]], 0.0, 1).sha256()


def test_checkpoint_roundtrip_keeps_every_array(tmp_path):
    """safetensors + config.json under the reference's tensor names (weights.py:151-198) -> the stored model."""

    from oracle import lane_oracle as O
    from tensorfold_b200 import weights

    cfg = O.Config(hidden=256, intermediate=512, layers=4, heads=4, kv_heads=2, head_dim=128, vocab=512, k_heads=2, v_heads=4,
                   dk=128, dv=128)
    model = O.random_model(cfg, 3)
    weights.save(model, tmp_path)
    got = weights.load(tmp_path)
    c = got["config"]
    assert (c.hidden, c.layers, c.heads, c.kv_heads, c.k_heads, c.v_heads, c.group, c.rope_dims) == (256, 4, 4, 2, 2, 4, 64, 32)
    for a, b in zip(model["layers"], got["layers"]):
        assert a["linear"] == b["linear"]
        for name, va in a.items():
            vb = b[name]
            if hasattr(va, "words"):
                assert torch.equal(va.words, vb.words) and torch.equal(va.scales, vb.scales) and torch.equal(va.biases, vb.biases)
            elif torch.is_tensor(va):
                assert torch.equal(va.float(), vb.float()), name
    assert torch.equal(model["head"].words, got["head"].words) and torch.equal(model["embed"].scales, got["embed"].scales)
    import safetensors.torch as st_
    tensors = st_.load_file(str(tmp_path / "model.safetensors"))
    tensors["model.layers.0.unknown.weight"] = torch.zeros(1)
    st_.save_file(tensors, str(tmp_path / "model.safetensors"))
    with pytest.raises(ValueError):
        weights.load(tmp_path)


# ---- failure handling on the host: nothing here touches a GPU ------------------------------------------

def _settings_worker(rank, world, port, out):
    import torch.distributed as dist

    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        tp = D.RankGroup()
        tp.check_settings({"max_rows": 8, "split_head": True})           # equal everywhere: passes
        try:
            tp.check_settings({"max_rows": 8 if rank == 0 else 16, "split_head": True})
            out[rank] = "started"
        except RuntimeError as exc:
            out[rank] = str(exc)
    finally:
        dist.destroy_process_group()


def _port():
    import socket

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_ranks_with_different_settings_refuse_to_start():
    """After the reference's start-up check (families/qwen3_5/cuda/engine.py:54-62, tests/cuda/test_flashnext_tp.py:436-457)."""

    out = mp.Manager().dict()
    mp.spawn(_settings_worker, args=(2, _port(), out), nprocs=2, join=True)
    for rank in range(2):
        assert "different settings" in out[rank] and "max_rows" in out[rank], out[rank]


def _absent_worker(rank, world, port, out):
    import datetime

    import torch.distributed as dist

    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=3))
    tp = D.RankGroup()
    if rank == 1:
        out[rank] = "left before the exchange"       # a rank that never arrives at the collective
        return
    try:
        tp.gather_partials(torch.ones((2, 8)))
        out[rank] = "gathered"
    except Exception as exc:                          # the short group timeout ends the wait with an error
        out[rank] = f"error: {type(exc).__name__}"


def test_a_rank_that_never_arrives_ends_the_others_wait_with_an_error():
    out = mp.Manager().dict()
    mp.spawn(_absent_worker, args=(2, _port(), out), nprocs=2, join=True)
    assert out[1] == "left before the exchange"
    assert out[0].startswith("error"), out[0]


def _raising_worker(rank, world, port, out):
    import datetime

    import torch.distributed as dist

    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=3))
    tp = D.RankGroup()
    first = tp.gather_partials(torch.full((1, 8), float(rank)))
    out[f"first{rank}"] = first[:, 0, 0].tolist()
    if rank == 1:
        raise ValueError("rank 1 fails between two steps")
    try:
        tp.gather_partials(torch.ones((1, 8)))
        out[rank] = "gathered"
    except Exception as exc:
        out[rank] = f"error: {type(exc).__name__}"


def test_a_rank_that_raises_between_steps_is_seen_by_the_others():
    out = mp.Manager().dict()
    with pytest.raises(Exception):                    # the failing rank's exception reaches the launcher
        mp.spawn(_raising_worker, args=(2, _port(), out), nprocs=2, join=True)
    assert out["first0"] == [0.0, 1.0]               # the step before the failure completed on rank 0


# ---- the expert-parallel exchange's slot-reuse rule, as a model ------------------------------------------------
def _simulate_expert_exchange(world, exchanges, presence, seed):
    """Ranks as state machines under a random scheduler. Exchange n: a rank pushes the results of the problems
    it owns (possibly none) into slot n & 1 of every rank's buffer, plus - with ``presence`` - its presence cell;
    its combine then needs the data of all owners and, with ``presence``, every rank's cell, and only then
    advances its exchange number. Returns the first overwrite of a slot that its reader has not finished with."""

    import random

    rng = random.Random(seed)
    owners = [[r for r in range(world) if rng.random() < 0.4] for _ in range(exchanges + 1)]     # owners[n]; may be empty
    done = [0] * world                           # exchanges a rank has completed
    pushed = [0] * world                         # exchanges a rank has pushed
    data = [[{} for _ in range(2)] for _ in range(world)]       # data[rank][slot][owner] = n
    cell = [[{} for _ in range(2)] for _ in range(world)]
    while min(done) < exchanges:
        r = rng.randrange(world)
        n = done[r] + 1
        if n > exchanges:
            continue
        if pushed[r] < n:                        # push n
            for peer in range(world):
                if presence:
                    cell[peer][n & 1][r] = n
                if r in owners[n]:
                    if done[peer] < n - 2:       # peer has not finished the exchange that used this slot before
                        return (r, peer, n)
                    data[peer][n & 1][r] = n
            pushed[r] = n
        elif all(data[r][n & 1].get(o) == n for o in owners[n]) and \
                (not presence or all(cell[r][n & 1].get(p) == n for p in range(world))):
            done[r] = n                          # combine n passed
    return None


def test_presence_cells_keep_a_fast_rank_from_overwriting_a_slot_in_use():
    for seed in range(200):
        assert _simulate_expert_exchange(4, 40, True, seed) is None
    # the model does find the overwrite when only data packets couple the ranks
    assert any(_simulate_expert_exchange(4, 40, False, seed) is not None for seed in range(200))


def test_gate_up_interleave_is_a_permutation_by_column_tile():
    """The stacked [gate; up] order of the fused SwiGLU: tile 2a holds gate rows 16a..16a+15, tile 2a+1 the up rows."""

    from types import SimpleNamespace

    from tensorfold_b200.forward import interleave_gate_up

    n, kw = 64, 4
    mk = lambda base: SimpleNamespace(words=(base + torch.arange(n * kw)).reshape(n, kw).to(torch.int32),
                                      scales=(base + torch.arange(n * 2)).reshape(n, 2).float(),
                                      biases=(base - torch.arange(n * 2)).reshape(n, 2).float())
    gate, up = mk(0), mk(100000)
    mixed = interleave_gate_up(gate, up)
    assert mixed.words.shape == (2 * n, kw)
    for a in range(n // 16):
        assert torch.equal(mixed.words[32 * a:32 * a + 16], gate.words[16 * a:16 * a + 16])
        assert torch.equal(mixed.words[32 * a + 16:32 * a + 32], up.words[16 * a:16 * a + 16])
        assert torch.equal(mixed.scales[32 * a + 16:32 * a + 32], up.scales[16 * a:16 * a + 16])
        assert torch.equal(mixed.biases[32 * a:32 * a + 16], gate.biases[16 * a:16 * a + 16])
    with pytest.raises(ValueError):
        interleave_gate_up(SimpleNamespace(words=torch.zeros((24, 4)), scales=torch.zeros((24, 2)), biases=torch.zeros((24, 2))),
                           SimpleNamespace(words=torch.zeros((24, 4)), scales=torch.zeros((24, 2)), biases=torch.zeros((24, 2))))
