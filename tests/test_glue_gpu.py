"""Glue kernels on the GPU: parity with the oracle within the bf16 tolerance, and rows alone == rows in a window.

Follows the reference's ``tests/cuda/test_qwen27_glue.py`` (``_rows_alone`` idea) and ``tests/test_lane_glue_norm.py``.
"""

import pytest
import torch

from oracle import lane_oracle as O
from tests.helpers import assert_close, assert_same_bits

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


@pytest.fixture(scope="module")
def mods(lib):
    from tensorfold_b200 import lane_glue, lane_qmm

    return lane_glue, lane_qmm


def unpack(packed, qmm_mod):
    """Rows and group sums back out of a packed buffer, by feeding identity-like probes is overkill: decode the layout."""

    m, k, g = packed.m, packed.k, packed.group
    mp = qmm_mod.padded_rows(m)
    gpt = 64 // g
    tile = mp * (128 + 4 * gpt)
    raw = packed.data.cpu().reshape(k // 64, tile)
    rows = raw[:, :mp * 128].reshape(k // 64, mp, 8, 16)
    out = torch.empty((k // 64, mp, 8, 16), dtype=torch.uint8)
    for r in range(mp):
        order = [c ^ (4 * (r & 1)) for c in range(8)]
        out[:, r] = rows[:, r][:, order]
    x = out.reshape(k // 64, mp, 128).view(BF).permute(1, 0, 2).reshape(mp, k)
    sums = raw[:, mp * 128:].contiguous().view(torch.float32).reshape(k // 64, gpt, mp).permute(2, 0, 1).reshape(mp, k // g)
    return x[:m], sums[:m], x[m:], sums[m:]


def test_pack_rows_layout_and_zero_padding(mods):
    glue, qmm = mods
    x = torch.randn((5, 512), generator=torch.Generator().manual_seed(0)).to(BF)
    for g in (64, 32):
        rows, sums, pad_rows, pad_sums = unpack(qmm.pack_rows(x.cuda(), g), qmm)
        assert_same_bits(rows, x)
        assert torch.allclose(sums, O.group_sums(x, g), atol=1e-5)
        assert not pad_rows.view(torch.int16).any() and not pad_sums.any()


@pytest.mark.parametrize("group", [64, 32])
@pytest.mark.parametrize("m", [1, 5, 8, 13, 128])
def test_norm_xs(mods, m, group):
    glue, qmm = mods
    gen = torch.Generator().manual_seed(m)
    d = 1024
    x = torch.randn((m, d), generator=gen).to(BF)
    r = torch.randn((m, d), generator=gen).to(BF)
    w = (1 + 0.05 * torch.randn(d, generator=gen)).to(BF)
    h, packed, rows = glue.norm_xs(x.cuda(), r.cuda(), w.cuda(), 1e-6, group=group, rows_out=True)
    h_ref, y_ref = O.add_rmsnorm(x, r, w, 1e-6)
    assert_same_bits(h.cpu(), h_ref, "residual add")
    assert_close(rows, y_ref, "norm rows")
    prow, psum, pad_rows, _ = unpack(packed, qmm)
    assert_same_bits(prow, rows.cpu(), "packed rows == plain rows")
    assert torch.allclose(psum, O.group_sums(rows.cpu(), group), atol=1e-4)
    assert not pad_rows.view(torch.int16).any()
    # no residual: h is the input itself
    h2, rows2 = glue.norm_xs(x.cuda(), None, w.cuda(), 1e-6, group=group, rows_out=True, packed_out=False)
    assert h2.data_ptr() != 0 and torch.equal(h2.cpu(), x)
    assert_close(rows2, O.add_rmsnorm(x, None, w, 1e-6)[1])
    # each row alone
    for i in (0, m - 1):
        _, one = glue.norm_xs(x[i:i + 1].cuda(), r[i:i + 1].cuda(), w.cuda(), 1e-6, group=group, rows_out=True, packed_out=False)
        assert_same_bits(one, rows[i:i + 1], f"row {i} alone")


def test_norm_xs_rank_partials_sum_in_rank_order(mods):
    glue, _ = mods
    gen = torch.Generator().manual_seed(3)
    x = torch.randn((6, 512), generator=gen).to(BF)
    parts = torch.randn((4, 6, 512), generator=gen)
    w = torch.ones(512).to(BF)
    h, rows = glue.norm_xs(x.cuda(), None, w.cuda(), 1e-6, partials=parts.cuda(), rows_out=True, packed_out=False)
    r = (((parts[0] + parts[1]) + parts[2]) + parts[3]).to(BF)
    assert_same_bits(h.cpu(), (x.float() + r.float()).to(BF), "rank-ordered sum, one rounding")
    # the reference's closed-form example (tests/cuda/test_qwen27_distributed.py:140-145): rounding happens once
    a = torch.full((1, 256), 1.0); b2 = torch.full((1, 256), 2.0 ** -9)
    h2, _ = glue.norm_xs(torch.zeros((1, 256), dtype=BF).cuda(), None, torch.ones(256, dtype=BF).cuda(), 1e-6,
                         partials=torch.stack([a, b2, b2]).cuda(), rows_out=True, packed_out=False)
    assert_same_bits(h2.cpu(), (a + b2 + b2).to(BF))


@pytest.mark.parametrize("group", [64, 32])
def test_mlp_act_gdn_post_gate_mul(mods, group):
    glue, qmm = mods
    gen = torch.Generator().manual_seed(5)
    m, inter = 9, 768
    gu = torch.randn((m, 2 * inter), generator=gen).to(BF)
    packed, rows = glue.mlp_act(gu.cuda()[:, :inter], gu.cuda()[:, inter:], group=group, rows_out=True)
    assert_close(rows, O.swiglu(gu[:, :inter], gu[:, inter:]), "swiglu")
    assert_same_bits(unpack(packed, qmm)[0], rows.cpu())
    one = glue.mlp_act(gu.cuda()[4:5, :inter], gu.cuda()[4:5, inter:], group=group, rows_out=True)[1]
    assert_same_bits(one, rows[4:5], "swiglu row alone")

    nv = 4
    y = torch.randn((m, nv, 128), generator=gen).to(BF)
    z = torch.randn((m, nv * 128 + 64), generator=gen).to(BF)
    w = (1 + 0.05 * torch.randn(128, generator=gen)).to(BF)
    packed, rows = glue.gdn_post(y.cuda(), z.cuda()[:, :nv * 128], w.cuda(), 1e-6, group=group, rows_out=True)
    assert_close(rows, O.gated_norm(y, z[:, :nv * 128].reshape(m, nv, 128), w, 1e-6), "gated norm")
    assert_same_bits(unpack(packed, qmm)[0], rows.cpu())
    assert torch.allclose(unpack(packed, qmm)[1], O.group_sums(rows.cpu(), group), atol=1e-4)

    for hd in (128, 256):
        h = 3
        o = torch.randn((m, h, hd), generator=gen).to(BF)
        qg = torch.randn((m, h * 2 * hd), generator=gen).to(BF)
        packed, rows = glue.gate_mul(o.cuda(), qg.cuda(), heads=h, head_dim=hd, group=group, rows_out=True)
        assert_close(rows, O.gate_mul(o, qg, heads=h, head_dim=hd), "gate_mul")
        assert_same_bits(unpack(packed, qmm)[0], rows.cpu())


@pytest.mark.parametrize("hd", [128, 256])
def test_attn_prep(mods, hd):
    glue, _ = mods
    gen = torch.Generator().manual_seed(7)
    m, h, hk = 7, 4, 2
    qg = torch.randn((m, h * 2 * hd), generator=gen).to(BF)
    k = torch.randn((m, hk * hd), generator=gen).to(BF)
    v = torch.randn((m, hk * hd), generator=gen).to(BF)
    qn = (1 + 0.05 * torch.randn(hd, generator=gen)).to(BF)
    kn = (1 + 0.05 * torch.randn(hd, generator=gen)).to(BF)
    pos = torch.tensor([0, 1, 2, 3, 1000, 32767, 65535], dtype=torch.int32)
    cfg = O.Config(hidden=256, intermediate=256, layers=1, heads=h, kv_heads=hk, head_dim=hd, vocab=8, k_heads=1, v_heads=1, dk=128, dv=128)
    inv = cfg.inv_freq()
    q, kk, vv = glue.attn_prep(qg.cuda(), k.cuda(), v.cuda(), qn.cuda(), kn.cuda(), pos.cuda(), inv.cuda(), 1e-6, heads=h,
                               kv_heads=hk, head_dim=hd)
    q_ref, k_ref = O.attn_prep(qg, k, qn, kn, pos, inv, 1e-6, heads=h, kv_heads=hk, head_dim=hd)
    # large positions: sin/cos of a float32 angle near 6e4 rad; both sides round the same product, tolerance unchanged
    assert_close(q, q_ref, "q", rel=2e-2, abs_=2e-2)
    assert_close(kk, k_ref, "k", rel=2e-2, abs_=2e-2)
    assert_close(q[:4], q_ref[:4], "q small positions")
    assert_same_bits(vv.cpu(), v.reshape(m, hk, hd))
    q1, k1, _ = glue.attn_prep(qg[5:6].cuda(), k[5:6].cuda(), v[5:6].cuda(), qn.cuda(), kn.cuda(), pos[5:6].cuda(), inv.cuda(),
                               1e-6, heads=h, kv_heads=hk, head_dim=hd)
    assert_same_bits(q1, q[5:6], "q row alone")
    assert_same_bits(k1, kk[5:6], "k row alone")


def test_gdn_pre_two_sequences(mods):
    glue, _ = mods
    gen = torch.Generator().manual_seed(9)
    nk, nv = 2, 4
    c = (2 * nk + nv) * 128
    widths = [5, 3]
    m = sum(widths)
    qkv = torch.randn((m, c), generator=gen).to(BF)
    conv_state = torch.randn((2, 3, c), generator=gen).to(BF)
    conv_w = (0.3 * torch.randn((c, 4), generator=gen)).to(BF)
    a = torch.randn((m, nv), generator=gen).to(BF)
    b = torch.randn((m, nv), generator=gen).to(BF)
    a_log, dt = 0.5 * torch.randn(nv, generator=gen), 0.5 * torch.randn(nv, generator=gen)
    row_seq = torch.tensor([0] * 5 + [1] * 3, dtype=torch.int32)
    row_idx = torch.tensor([0, 1, 2, 3, 4, 0, 1, 2], dtype=torch.int32)
    got = glue.gdn_pre(qkv.cuda(), conv_state.cuda(), conv_w.cuda(), row_seq.cuda(), row_idx.cuda(), a.cuda(), b.cuda(),
                       a_log.cuda(), dt.cuda(), nk=nk, nv=nv)
    r0 = 0
    for s, wd in enumerate(widths):
        want = O.gdn_pre(qkv[r0:r0 + wd], conv_state[s], conv_w, a[r0:r0 + wd], b[r0:r0 + wd], a_log, dt, kh=nk, vh=nv, dk=128, dv=128)
        for name, gt, wt in zip("qkvgb", got, want):
            if name in "qkv":
                assert_close(gt[r0:r0 + wd], wt, f"seq {s} {name}", rel=1e-2, abs_=2e-3)
            else:
                assert torch.allclose(gt[r0:r0 + wd].cpu(), wt, rtol=1e-5, atol=1e-6), name
        r0 += wd
    # serial form: the second sequence's last row alone, with the conv tail a commit of 2 rows leaves
    tail = torch.cat([conv_state[1], qkv[5:7]])[-3:]
    one = glue.gdn_pre(qkv[7:8].cuda(), tail[None].cuda(), conv_w.cuda(), torch.zeros(1, dtype=torch.int32).cuda(),
                       torch.zeros(1, dtype=torch.int32).cuda(), a[7:8].cuda(), b[7:8].cuda(), a_log.cuda(), dt.cuda(), nk=nk, nv=nv)
    for gt, o in zip(got, one):
        assert_same_bits(o, gt[7:8], "window row == serial step")


def test_embed(mods):
    glue, _ = mods
    gen = torch.Generator().manual_seed(11)
    for group in (64, 32):
        q = O.random_q4(gen, 300, 512, group)
        ids = torch.tensor([0, 299, 17, 17, 123], dtype=torch.int32)
        out = glue.embed(ids.cuda(), q.words.cuda(), q.scales.cuda(), q.biases.cuda(), 512, group)
        assert_same_bits(out.cpu(), O.embed(ids, q.words, q.scales, q.biases, group), "embed is exact")


def test_lane_fuse_stacks_and_reads_in_place(mods):
    """The reference's lane_fuse entry points (tests/test_lane_fuse.py: stacked output == members side by side,
    consumers read the stack in place): a stacked row has the bits of that row alone, every member's columns
    are within the matmul tolerance of the member projected by itself, and gdn_post / mlp_act on the stacked
    rows equal the kernels on separate tensors."""

    from tensorfold_b200 import lane_fuse, lane_qmm

    glue, qmm = mods
    gen = torch.Generator().manual_seed(9)
    nv, dv, d = 4, 128, 512
    layer = {"z": O.random_q4(gen, nv * dv, d, 64), "b": O.random_q4(gen, nv, d, 64), "a": O.random_q4(gen, nv, d, 64),
             "gate": O.random_q4(gen, 256, d, 64), "up": O.random_q4(gen, 256, d, 64)}
    model = {"config": O.Config(hidden=d, intermediate=256, layers=1, heads=2, kv_heads=1, head_dim=128, vocab=64, k_heads=2,
                                v_heads=nv, dk=128, dv=128), "layers": [layer]}
    assert lane_fuse.attn_kv(layer, torch.zeros((1, d), dtype=BF).cuda()) is None          # nothing stacked yet
    assert lane_fuse.build(model) == {"zba": 1, "kv": 0, "gu": 1}
    assert lane_fuse.stats(model)["groups"] == {"zba": 1, "kv": 0, "gu": 1}
    x = torch.randn((5, d), generator=gen).to(BF).cuda()
    zba = lane_fuse.gdn_in(layer, x)
    assert zba.shape == (5, nv * dv + 2 * nv)
    assert_same_bits(lane_fuse.gdn_in(layer, x[2:3]), zba[2:3], "stacked row alone")
    zq = layer["z"]
    z_alone = qmm.lane_matmul(x, qmm.tile_weight(zq.words.cuda(), zq.scales.cuda(), zq.biases.cuda(), 64))
    assert_close(zba[:, :nv * dv], z_alone.cpu(), "z member of the stack")
    y = torch.randn((5, nv, dv), generator=gen).to(BF).cuda()
    w = (1 + 0.05 * torch.randn(dv, generator=gen)).to(BF).cuda()
    a = lane_fuse.gdn_post(y, zba, w, 1e-6)
    b = glue.gdn_post(y, zba[:, :nv * dv].contiguous(), w, 1e-6)
    assert torch.equal(a.data, b.data)
    gu = lane_fuse.mlp_gate_up(layer, x)
    a = lane_fuse.mlp_act(gu)
    b = glue.mlp_act(gu[:, :256].contiguous(), gu[:, 256:].contiguous())
    assert torch.equal(a.data, b.data)
    lane_fuse.clear(model)
    assert lane_fuse.gdn_in(layer, x) is None


@pytest.mark.parametrize("group", [64, 32])
@pytest.mark.parametrize("rows", [1, 5, 8])
def test_swiglu_in_the_matmul_epilogue_has_the_bits_of_the_separate_kernel(mods, group, rows):
    """[gate; up] interleaved by 16-column tile: the lane matmul's SwiGLU epilogue writes the packed input of the down
    projection with the bits of matmul -> ``mlp_act_tiled``, which in turn equals ``mlp_act`` on the separated halves."""

    from tensorfold_b200 import forward as F

    glue, qmm = mods
    inter, k = 1280, 1024                       # 2 I = 2560 output columns = ten column blocks: K is cut, blocks have owners
    gen = torch.Generator().manual_seed(91 + rows)
    gate, up = O.random_q4(gen, inter, k, group), O.random_q4(gen, inter, k, group)
    mixed = F.interleave_gate_up(gate, up)
    w = qmm.tile_weight(mixed.words.cuda(), mixed.scales.cuda(), mixed.biases.cuda(), group)
    x = torch.randn((rows, k), generator=gen).to(BF).cuda()
    xp = qmm.pack_rows(x, group)
    gu = qmm.lane_matmul(xp, w)
    separate = glue.mlp_act_tiled(gu, inter, group=group)
    fused = qmm.lane_matmul(xp, w, act_out=qmm.new_packed(rows, inter, group, "cuda"))
    torch.cuda.synchronize()
    assert torch.equal(fused.data.cpu(), separate.data.cpu()), "fused SwiGLU epilogue differs from the separate kernel"
    tiles = gu.reshape(rows, inter // 16, 2, 16)
    halves = torch.cat([tiles[:, :, 0].reshape(rows, inter), tiles[:, :, 1].reshape(rows, inter)], dim=1).contiguous()
    plain = glue.mlp_act(halves[:, :inter], halves[:, inter:], group=group)
    assert torch.equal(plain.data.cpu(), separate.data.cpu()), "mlp_act_tiled differs from mlp_act on the separated halves"
    # and against the oracle's arithmetic
    want = O.swiglu(halves[:, :inter].cpu(), halves[:, inter:].cpu())
    _, got_rows = glue.mlp_act_tiled(gu, inter, group=group, rows_out=True)
    assert_close(got_rows, want, "tiled SwiGLU vs oracle")
