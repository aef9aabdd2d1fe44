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
    need = LA.chunks_for(max(lens) + max(widths))
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


def test_gated_attention_equals_attention_then_gate(lib):
    """The merge kernel's fused output gate and packed output carry the bits of the two separate steps."""

    from tensorfold_b200 import lane_attention as LA, lane_glue, lane_qmm

    d, h, hk = 256, 24, 4
    lens, widths = [300, 9000], [8, 5]
    kv, q, k_new, v_new, keys, vals, starts, nkeys = paged_setup(11, lens, widths, h, hk, d)
    seq_lens = torch.tensor(lens, dtype=torch.int32).cuda()
    need = LA.chunks_for(max(l + w for l, w in zip(lens, widths)))
    r = sum(widths)
    qg = torch.randn((r, h * 2 * d + 64), generator=torch.Generator().manual_seed(5)).to(BF).cuda()[:, :h * 2 * d]
    args = (q.cuda(), k_new.cuda(), v_new.cuda(), kv.k[0], kv.v[0], kv.table, seq_lens, starts.cuda(), nkeys.cuda())
    kw = dict(scale=d ** -0.5, max_window=max(widths), max_chunks=need)
    plain = LA.lane_attention(*args, **kw)
    want_packed, want_rows = lane_glue.gate_mul(plain, qg, heads=h, head_dim=d, group=64, rows_out=True)
    rows = torch.empty_like(plain)
    packed = lane_qmm.new_packed(r, h * d, 64, "cuda")
    packed.data.fill_(7)
    LA.lane_attention(*args, out=rows, gate=qg, packed_out=packed, **kw)
    assert_same_bits(rows.reshape(r, -1), want_rows, "gated rows")
    assert torch.equal(packed.data, want_packed.data), "packed output of the fused merge"
    r0 = 0
    for i, wd in enumerate(widths):
        want = O.attention(q[r0:r0 + wd], keys[i], vals[i], nkeys[r0:r0 + wd], d ** -0.5)
        assert_close(plain[r0:r0 + wd], want, f"seq {i}", rel=2e-2, abs_=1e-2)
        r0 += wd


@pytest.mark.parametrize("ctx", [4096, 20000, 32768])
def test_lane_attention_long_context(lib, ctx):
    """Config-3 attention shape (24 query / 4 KV heads of 256) at the benchmarked context lengths and at the
    reference's own long case (20000 keys, tests/test_lane_attention.py:25-49): W = 8 window rows against the
    fp32 oracle, and the last row alone (serial form) bit-equal to the same row inside the window."""

    from tensorfold_b200 import lane_attention as LA

    d, h, hk, w = 256, 24, 4, 8
    gen = torch.Generator().manual_seed(ctx)
    keys = torch.randn((ctx + w, hk, d), generator=gen).to(BF)
    vals = torch.randn((ctx + w, hk, d), generator=gen).to(BF)
    q = torch.randn((w, h, d), generator=gen).to(BF)
    out = LA.lane_sdpa(q.cuda(), keys.cuda(), vals.cuda(), d ** -0.5)
    nkeys = torch.arange(ctx + 1, ctx + w + 1)
    want = O.attention(q, keys, vals, nkeys, d ** -0.5)
    assert_close(out, want, f"context {ctx}", rel=2e-2, abs_=1e-2)
    one = LA.lane_sdpa(q[w - 1:].cuda(), keys.cuda(), vals.cuda(), d ** -0.5)
    assert_same_bits(one, out[w - 1:], "last row alone == last row of the window")


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
    assert np.array_equal(O.uniform_rows(1234, positions[:8], ids[:8]), z["u"])
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


def _mixer_inputs(seed, widths, nk, nv):
    gen = torch.Generator().manual_seed(seed)
    r, s = sum(widths), len(widths)
    c = (2 * nk + nv) * 128
    proj = torch.randn((r, c + nv * 128 + 2 * nv), generator=gen).to(BF)          # [qkv | z | b | a] rows of the stacked projection
    conv_state = torch.randn((s, 3, c), generator=gen).to(BF)
    conv_w = (0.3 * torch.randn((c, 4), generator=gen)).to(BF)
    a_log, dt_bias = 0.5 * torch.randn(nv, generator=gen), 0.5 * torch.randn(nv, generator=gen)
    norm_w = (1 + 0.05 * torch.randn(128, generator=gen)).to(BF)
    state = 0.1 * torch.randn((s, nv, 128, 128), generator=gen)
    starts = torch.tensor([0] + list(np.cumsum(widths)), dtype=torch.int32)
    row_seq = torch.tensor([i for i, w in enumerate(widths) for _ in range(w)], dtype=torch.int32)
    row_idx = torch.tensor([t for w in widths for t in range(w)], dtype=torch.int32)
    return proj, conv_state, conv_w, a_log, dt_bias, norm_w, state, starts, row_seq, row_idx


@pytest.mark.parametrize("widths,nk,nv,group", [([8, 3, 1, 13], 2, 4, 64), ([5, 8], 2, 4, 32), ([8] * 16, 16, 32, 64)])
def test_gdn_mixer_in_one_launch_has_the_bits_of_the_three_kernels(lib, widths, nk, nv, group):
    """Conv + gates, recurrence and gated norm fused (tf_gdn_fused) against gdn_pre -> gated_delta_chain ->
    gdn_post; the last case has the head counts of the benchmark's gated-DeltaNet layers (16 key / 32 value
    heads of 128) at the 128 rows one forward takes, also checked against the fp32 oracle recurrence."""

    from tensorfold_b200 import lane_gdn, lane_glue

    proj, conv_state, conv_w, a_log, dt_bias, norm_w, state, starts, row_seq, row_idx = _mixer_inputs(len(widths), widths, nk, nv)
    r, c = sum(widths), (2 * nk + nv) * 128
    d = lambda t: t.cuda()
    projc = d(proj)
    qkv, z = projc[:, :c], projc[:, c:c + nv * 128]
    bb, aa = projc[:, c + nv * 128:c + nv * 128 + nv], projc[:, c + nv * 128 + nv:]
    q, k, v, g, beta = lane_glue.gdn_pre(qkv, d(conv_state), d(conv_w), d(row_seq), d(row_idx), aa, bb, d(a_log), d(dt_bias), nk=nk, nv=nv)
    y = lane_gdn.gated_delta_chain(q, k, v, g, beta, d(state), d(starts))
    want_packed, want_rows = lane_glue.gdn_post(y, z, d(norm_w), 1e-6, group=group, rows_out=True)
    rec = (torch.empty_like(k), torch.empty_like(v), torch.empty_like(g), torch.empty_like(beta))
    packed, rows = lane_gdn.gdn_mixer(qkv, z, aa, bb, d(conv_state), d(conv_w), d(a_log), d(dt_bias), d(norm_w), d(state), d(starts),
                                      nk=nk, nv=nv, eps=1e-6, group=group, record=rec, rows_out=True)
    assert_same_bits(rows, want_rows, "mixer rows")
    assert torch.equal(packed.data, want_packed.data), "mixer packed output"
    for got, want, name in zip(rec, (k, v, g, beta), ("k", "v", "g", "beta")):
        assert torch.equal(got.view(torch.int32) if got.dtype == torch.float32 else got.view(torch.int16),
                           want.view(torch.int32) if want.dtype == torch.float32 else want.view(torch.int16)), f"record {name}"
    if len(widths) == 16:
        # the recurrence at this shape against the fp32 oracle (tolerance of tests/cuda/test_flashnext_kernels.py:216-218)
        for s in (0, 7, 15):
            r0 = int(starts[s])
            sl = slice(r0, r0 + widths[s])
            y_ref, _ = O.gdn_recurrence(q[sl].cpu(), k[sl].cpu(), v[sl].cpu(), g[sl].cpu(), beta[sl].cpu(), state[s])
            err = (y[sl].float().cpu() - y_ref.float()).abs().max()
            assert err < 0.05 * y_ref.float().abs().max()


def test_gdn_lane_step_at_config_2_shape(lib):
    """The gated-DeltaNet lane step as the benchmark configs give it: 32 sequences x 8 rows, 16 key / 32 value
    heads of 128, fp32 state [32, 32, 128, 128] ~ N(0, 0.1): the 8-row window against the fp32 oracle, and its
    rows bit-equal to 8 one-row steps with the state replayed in between (replay(keep) == state after keep steps)."""

    from tensorfold_b200 import lane_gdn

    widths = [8] * 32
    q, k, v, g, beta, state, starts = gdn_inputs(2, widths, hk=16, hv=32)
    dev = [t.cuda() for t in (q, k, v, g, beta, state, starts)]
    y = lane_gdn.gated_delta_chain(*dev)
    for s in (0, 13, 31):
        sl = slice(8 * s, 8 * s + 8)
        y_ref, _ = O.gdn_recurrence(q[sl], k[sl], v[sl], g[sl], beta[sl], state[s])
        assert (y[sl].float().cpu() - y_ref.float()).abs().max() < 0.05 * y_ref.float().abs().max()
    st = dev[5].clone()
    one = torch.ones(32, dtype=torch.int32).cuda()
    ss = torch.arange(33, dtype=torch.int32).cuda()
    for t in range(8):
        sel = (torch.arange(32) * 8 + t).cuda()
        ys = lane_gdn.gated_delta_chain(dev[0][sel].contiguous(), dev[1][sel].contiguous(), dev[2][sel].contiguous(),
                                        dev[3][sel].contiguous(), dev[4][sel].contiguous(), st, ss)
        assert_same_bits(ys, y[sel], f"row {t}: window == serial")
        lane_gdn.replay(dev[1][sel].contiguous(), dev[2][sel].contiguous(), dev[3][sel].contiguous(), dev[4][sel].contiguous(), st, ss, one)
    full = dev[5].clone()
    lane_gdn.replay(dev[1], dev[2], dev[3], dev[4], full, dev[6], torch.full((32,), 8, dtype=torch.int32).cuda())
    assert torch.equal(full.view(torch.int32), st.view(torch.int32)), "replay(8) == eight serial steps"


def test_reference_call_shapes_tree_sdpa_and_gdn_cache(lib):
    """``lane_tree_sdpa`` for chain parents is ``lane_sdpa`` and refuses a branching tree; ``LaneGDNCache.step``
    advances every lane by one position with the bits of the chain kernel over the same rows."""

    from tensorfold_b200 import lane_attention as LA, lane_gdn

    gen = torch.Generator().manual_seed(8)
    l, t, h, hk, d = 90, 4, 4, 2, 128
    q = torch.randn((t, h, d), generator=gen).to(BF).cuda()
    k = torch.randn((l, hk, d), generator=gen).to(BF).cuda()
    v = torch.randn((l, hk, d), generator=gen).to(BF).cuda()
    assert_same_bits(LA.lane_tree_sdpa(q, k, v, d ** -0.5, [-1, 0, 1, 2]), LA.lane_sdpa(q, k, v, d ** -0.5), "chain tree")
    with pytest.raises(ValueError):
        LA.lane_tree_sdpa(q, k, v, d ** -0.5, [-1, 0, 0, 1])

    lanes, steps = 3, 4
    qq, kk, vv, g, beta, state, _ = gdn_inputs(6, [steps] * lanes)
    s0 = state[0].cuda()
    cache = lane_gdn.LaneGDNCache(s0, lanes)
    ys = []
    for i in range(steps):
        sel = torch.arange(lanes) * steps + i
        ys.append(cache.step(qq[sel].cuda(), kk[sel].cuda(), vv[sel].cuda(), torch.log(g[sel]).cuda(), beta[sel].cuda()))
    starts = torch.arange(0, lanes * steps + 1, steps, dtype=torch.int32).cuda()
    # the chain kernel takes g itself; the cache takes log g and exponentiates: feed the chain the same values
    gexp = torch.exp(torch.log(g).cuda().float())
    want = lane_gdn.gated_delta_chain(qq.cuda(), kk.cuda(), vv.cuda(), gexp, beta.cuda(), s0.unsqueeze(0).repeat(lanes, 1, 1, 1).contiguous(), starts)
    for i in range(steps):
        sel = (torch.arange(lanes) * steps + i).cuda()
        assert_same_bits(ys[i], want[sel], f"cache step {i}")
