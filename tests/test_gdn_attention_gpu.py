"""GDN recurrence, paged lane attention, top-k and the keyed draw on the GPU.

Ideas from the reference's ``tests/cuda/test_qwen27_gdn_tree.py`` (chain rows == serial steps, zero-step
commit, replay_many == per-layer replay), ``tests/cuda/test_qwen27_attention.py`` / ``tests/test_lane_tree.py``
(window rows == serial rows at chunk boundaries), ``tests/test_topk.py`` and ``tests/test_exact_sampling.py``.
"""

from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import lane_oracle as O
from tests.helpers import assert_close, assert_same_bits

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def gdn_inputs(seed, widths, hk=2, hv=4, dv=128):
    gen = torch.Generator().manual_seed(seed)
    r = sum(widths)
    q = torch.nn.functional.normalize(torch.randn((r, hk, 128), generator=gen), dim=-1).to(BF)
    k = torch.nn.functional.normalize(torch.randn((r, hk, 128), generator=gen), dim=-1).to(BF)
    v = torch.randn((r, hv, dv), generator=gen).to(BF)
    beta = torch.sigmoid(torch.randn((r, hv), generator=gen))
    g = torch.exp(-torch.nn.functional.softplus(torch.randn((r, hv), generator=gen)))
    state = 0.1 * torch.randn((len(widths), hv, dv, 128), generator=gen)
    starts = torch.tensor([0] + list(np.cumsum(widths)), dtype=torch.int32)
    return q, k, v, g, beta, state, starts


def test_gdn_chain_matches_oracle_and_serial_steps(lib):
    from tensorfold_b200 import lane_gdn

    widths = [8, 3, 1]
    q, k, v, g, beta, state, starts = gdn_inputs(1, widths)
    dev = [t.cuda() for t in (q, k, v, g, beta, state, starts)]
    final = torch.empty_like(dev[5])
    y = lane_gdn.gated_delta_chain(*dev, state_out=final)
    r0 = 0
    for s, wd in enumerate(widths):
        y_ref, s_ref = O.gdn_recurrence(q[r0:r0 + wd], k[r0:r0 + wd], v[r0:r0 + wd], g[r0:r0 + wd], beta[r0:r0 + wd], state[s])
        err = (y[r0:r0 + wd].float().cpu() - y_ref.float()).abs().max()
        assert err < 0.05 * y_ref.float().abs().max()          # the reference's own bound (test_flashnext_kernels.py:216-218)
        assert_close(y[r0:r0 + wd], y_ref, f"seq {s} y", rel=2e-2, abs_=2e-3)
        assert (final[s].cpu() - s_ref).abs().max() < 1e-2
        r0 += wd
    # window rows == serial one-row steps with the state replayed in between (bit equality)
    st = dev[5].clone()
    one = torch.ones(len(widths), dtype=torch.int32).cuda()
    for t in range(max(widths)):
        rows = [int(starts[s]) + t for s, wd in enumerate(widths) if t < wd]
        seqs = [s for s, wd in enumerate(widths) if t < wd]
        sel = torch.tensor(rows).cuda()
        ss = torch.arange(len(rows) + 1, dtype=torch.int32).cuda()
        sub = st[seqs].contiguous()
        ys = lane_gdn.gated_delta_chain(dev[0][sel].contiguous(), dev[1][sel].contiguous(), dev[2][sel].contiguous(),
                                        dev[3][sel].contiguous(), dev[4][sel].contiguous(), sub, ss)
        assert_same_bits(ys, y[sel], f"step {t}")
        lane_gdn.replay(dev[1][sel].contiguous(), dev[2][sel].contiguous(), dev[3][sel].contiguous(), dev[4][sel].contiguous(),
                        sub, ss, one[:len(rows)].contiguous())
        st[seqs] = sub
    assert_same_bits(st, final, "replayed state == state after the window")
    # replay(keep) == state after keep serial steps; zero-step commit leaves the state alone
    for keep in ([0, 0, 0], [3, 1, 1], [8, 3, 1]):
        st2 = dev[5].clone()
        lane_gdn.replay(dev[1], dev[2], dev[3], dev[4], st2, dev[6], torch.tensor(keep, dtype=torch.int32).cuda())
        r0 = 0
        for s, wd in enumerate(widths):
            _, s_ref = O.gdn_recurrence(q[r0:r0 + keep[s]], k[r0:r0 + keep[s]], v[r0:r0 + keep[s]], g[r0:r0 + keep[s]],
                                        beta[r0:r0 + keep[s]], state[s]) if keep[s] else (None, state[s])
            assert (st2[s].cpu() - s_ref).abs().max() < 1e-2
            r0 += wd
        if keep == [0, 0, 0]:
            assert_same_bits(st2, dev[5])
        if keep == widths:
            assert_same_bits(st2, final)


def test_gdn_replay_many_layers_equals_per_layer(lib):
    from tensorfold_b200 import lane_gdn

    widths = [4, 2]
    layers = [gdn_inputs(10 + i, widths) for i in range(3)]
    stack = [torch.stack([l[j] for l in layers]).cuda() for j in range(6)]
    starts = layers[0][6].cuda()
    keep = torch.tensor([3, 2], dtype=torch.int32).cuda()
    many = stack[5].clone()
    lane_gdn.replay(stack[1], stack[2], stack[3], stack[4], many, starts, keep)
    for i in range(3):
        single = stack[5][i].clone()
        lane_gdn.replay(stack[1][i], stack[2][i], stack[3][i], stack[4][i], single, starts, keep)
        assert_same_bits(many[i], single, f"layer {i}")


def test_conv_commit(lib):
    from tensorfold_b200 import lane_gdn

    gen = torch.Generator().manual_seed(2)
    c = 512
    qkv = torch.randn((2, 7, c + 64), generator=gen).to(BF).cuda()
    state = torch.randn((2, 2, 3, c), generator=gen).to(BF).cuda()
    starts = torch.tensor([0, 5, 7], dtype=torch.int32).cuda()
    for keep in ([0, 0], [1, 2], [5, 1], [2, 0]):
        st = state.clone()
        lane_gdn.conv_commit(qkv[:, :, :c], st, starts, torch.tensor(keep, dtype=torch.int32).cuda(), c)
        for l in range(2):
            for s in range(2):
                r0 = int(starts[s])
                want = torch.cat([state[l, s], qkv[l, r0:r0 + keep[s], :c]])[-3:]
                assert_same_bits(st[l, s], want, f"keep {keep} layer {l} seq {s}")


def paged_setup(seed, lens, widths, h, hk, d):
    from tensorfold_b200 import lane_attention as LA

    gen = torch.Generator().manual_seed(seed)
    s = len(lens)
    kv = LA.PagedKV(1, s, sum(-(-(l + w) // 16) + 1 for l, w in zip(lens, widths)), hk, d, max(-(-(l + w) // 16) for l, w in zip(lens, widths)) + 1, "cuda")
    keys, vals = [], []
    # interleave page ownership so that a sequence's pages are not contiguous
    for step in range(max(-(-(l + w) // 16) for l, w in zip(lens, widths)) + 1):
        for i in range(s):
            if step * 16 < lens[i] + widths[i]:
                kv.reserve(i, min(lens[i] + widths[i], (step + 1) * 16))
    kv.sync_table()
    for i in range(s):
        k = torch.randn((lens[i] + widths[i], hk, d), generator=gen).to(BF)
        v = torch.randn((lens[i] + widths[i], hk, d), generator=gen).to(BF)
        keys.append(k); vals.append(v)
        for p in range(lens[i]):
            page = int(kv.table_host[i, p // 16])
            kv.k[0, page, :, p % 16] = k[p].cuda()
            kv.v[0, page, :, p % 16] = v[p].cuda()
    r = sum(widths)
    q = torch.randn((r, h, d), generator=gen).to(BF)
    k_new = torch.cat([keys[i][lens[i]:] for i in range(s)])
    v_new = torch.cat([vals[i][lens[i]:] for i in range(s)])
    starts = torch.tensor([0] + list(np.cumsum(widths)), dtype=torch.int32)
    nkeys = torch.tensor([lens[i] + t + 1 for i in range(s) for t in range(widths[i])], dtype=torch.int32)
    return kv, q, k_new, v_new, keys, vals, starts, nkeys


@pytest.mark.parametrize("d,h,hk", [(256, 6, 1), (128, 8, 2), (256, 24, 4)])
def test_lane_attention_ragged_windows(lib, d, h, hk):
    from tensorfold_b200 import lane_attention as LA

    lens, widths = [0, 5, 509, 1030, 3], [3, 8, 8, 1, 16]
    kv, q, k_new, v_new, keys, vals, starts, nkeys = paged_setup(3, lens, widths, h, hk, d)
    seq_lens = torch.tensor(lens, dtype=torch.int32).cuda()
    need = -(-(max(lens) + max(widths)) // LA.CHUNK)
    args = dict(scale=d ** -0.5, max_window=max(widths), max_chunks=need)
    out = LA.lane_attention(q.cuda(), k_new.cuda(), v_new.cuda(), kv.k[0], kv.v[0], kv.table, seq_lens, starts.cuda(),
                            nkeys.cuda(), **args)
    r0 = 0
    for i, wd in enumerate(widths):
        want = O.attention(q[r0:r0 + wd], keys[i], vals[i], nkeys[r0:r0 + wd], d ** -0.5)
        assert_close(out[r0:r0 + wd], want, f"seq {i}", rel=2e-2, abs_=1e-2)  # P is bf16 on the tensor cores, as in the reference kernels (its own bound: err < 0.02)
        r0 += wd
    # serial form: commit t rows, then the next row alone (its own K/V as the one window row)
    for i, t in ((2, 5), (1, 7), (4, 15), (0, 0)):
        r = int(starts[i]) + t
        kv2 = LA.PagedKV(1, 1, kv.num_pages, hk, d, kv.max_pages, "cuda")
        kv2.reserve(0, lens[i] + t + 1); kv2.sync_table()
        for p in range(lens[i] + t):
            page = int(kv2.table_host[0, p // 16])
            kv2.k[0, page, :, p % 16] = keys[i][p].cuda()
            kv2.v[0, page, :, p % 16] = vals[i][p].cuda()
        one = LA.lane_attention(q[r:r + 1].cuda(), k_new[r:r + 1].cuda(), v_new[r:r + 1].cuda(), kv2.k[0], kv2.v[0], kv2.table,
                                torch.tensor([lens[i] + t], dtype=torch.int32).cuda(), torch.tensor([0, 1], dtype=torch.int32).cuda(),
                                nkeys[r:r + 1].cuda(), scale=d ** -0.5, max_window=1, max_chunks=need)
        assert_same_bits(one, out[r:r + 1], f"seq {i} row {t}: window row == serial row")
    # a larger chunk budget than needed changes nothing
    out2 = LA.lane_attention(q.cuda(), k_new.cuda(), v_new.cuda(), kv.k[0], kv.v[0], kv.table, seq_lens, starts.cuda(),
                             nkeys.cuda(), scale=d ** -0.5, max_window=max(widths), max_chunks=need + 4)
    assert_same_bits(out2, out, "chunk budget")


def test_lane_sdpa_reference_shape_and_kv_commit(lib):
    from tensorfold_b200 import lane_attention as LA

    gen = torch.Generator().manual_seed(4)
    l, t, h, hk, d = 700, 4, 4, 2, 128
    q = torch.randn((t, h, d), generator=gen).to(BF)
    k = torch.randn((l, hk, d), generator=gen).to(BF)
    v = torch.randn((l, hk, d), generator=gen).to(BF)
    out = LA.lane_sdpa(q.cuda(), k.cuda(), v.cuda(), d ** -0.5)
    want = O.attention(q, k, v, torch.arange(l - t + 1, l + 1), d ** -0.5)
    assert_close(out, want, "lane_sdpa", rel=2e-2, abs_=1e-2)
    # kv_commit writes kept rows where the next forward reads them
    kv = LA.PagedKV(2, 2, 8, hk, d, 4, "cuda")
    kv.reserve(0, 20); kv.reserve(1, 40); kv.sync_table()
    k_new = torch.randn((2, 6, hk, d), generator=gen).to(BF).cuda()
    v_new = torch.randn((2, 6, hk, d), generator=gen).to(BF).cuda()
    lens = torch.tensor([14, 31], dtype=torch.int32).cuda()
    LA.kv_commit(k_new, v_new, kv, lens, torch.tensor([0, 4, 6], dtype=torch.int32).cuda(), torch.tensor([3, 2], dtype=torch.int32).cuda())
    for layer in range(2):
        for s, (l0, r0, keep) in enumerate(((14, 0, 3), (31, 4, 2))):
            for j in range(keep):
                p = l0 + j
                page = int(kv.table_host[s, p // 16])
                assert_same_bits(kv.k[layer, page, :, p % 16], k_new[layer, r0 + j])
                assert_same_bits(kv.v[layer, page, :, p % 16], v_new[layer, r0 + j])
            p = l0 + keep
            assert not kv.k[layer, int(kv.table_host[s, p // 16]), :, p % 16].any()


def test_topk_rows_matches_lexsort_rule(lib):
    from tensorfold_b200 import topk

    gen = torch.Generator().manual_seed(6)
    x = torch.randn((5, 248320), generator=gen).to(BF)
    x[1] = (x[1] * 2).round() / 2                   # heavy ties
    x[2] = 0.25                                      # all equal
    x[3, ::7] = float("-inf")
    x[4] = -x[4].abs()
    for k in (1, 20, 28, 64):
        idx, val = topk.topk_rows(x.cuda(), k)
        widx, wval = O.topk_rows(x.float().numpy(), k)
        assert np.array_equal(idx.cpu().numpy(), widx), k
        assert np.array_equal(val.cpu().numpy(), wval), k
    small = torch.randn((3, 100), generator=gen).to(BF)
    idx, _ = topk.topk_rows(small.cuda(), 64)
    assert np.array_equal(idx.cpu().numpy(), O.topk_rows(small.float().numpy(), 64)[0])
    wide = torch.randn((3, 100011), generator=gen).to(BF)      # rows that start off a 16-byte boundary, several slices
    view = wide.cuda()[:, 3:100006]
    idx, val = topk.topk_rows(view, 28)
    widx, wval = O.topk_rows(wide[:, 3:100006].float().numpy(), 28)
    assert np.array_equal(idx.cpu().numpy(), widx) and np.array_equal(val.cpu().numpy(), wval)
    one = topk.topk_rows(x[1:2].cuda(), 28)[0]
    assert torch.equal(one, topk.topk_rows(x.cuda(), 28)[0][1:2])
    with pytest.raises(ValueError):
        topk.topk_rows(x.cuda(), 65)


def test_keyed_sampling_matches_reference_fixture(lib):
    from tensorfold_b200 import exact_sampling as S

    z = np.load(Path(__file__).parent / "golden" / "exact_sampling.npz")
    vals, ids, positions = z["vals"], z["ids"], z["positions"]
    assert np.array_equal(S.uniform_rows(1234, positions[:8], ids[:8]), z["u"])
    for name, s in (("default", S.Sampling(seed=1234)), ("hot", S.Sampling(seed=99, temperature=1.7, top_k=10, top_p=0.8))):
        assert S.choose_rows(vals, ids, positions, s) == z["pick_" + name].tolist()
    # the device draw on logits rows whose top candidates are the fixture's rows
    vocab = 5000
    logits = torch.full((64, vocab), -30.0)
    for r in range(64):
        logits[r, torch.from_numpy(ids[r])] = torch.from_numpy(vals[r])
    logits = logits.to(BF).cuda()                      # quarter steps are exact in bf16
    for name, s in (("default", S.Sampling(seed=1234)), ("hot", S.Sampling(seed=99, temperature=1.7, top_k=10, top_p=0.8))):
        got = S.sample_rows(logits, positions.tolist(), s).cpu().tolist()
        assert got == z["pick_" + name].tolist(), name
        alone = S.sample_rows(logits[7:8], positions[7:8].tolist(), s).cpu().tolist()
        assert alone == got[7:8]
    greedy = S.sample_rows(logits, positions.tolist(), None).cpu().numpy()
    assert np.array_equal(greedy, np.array(O.sample_rows(logits.float().cpu().numpy(), positions, None)))
