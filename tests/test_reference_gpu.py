"""The reference's own CUDA lane path (Triton + its gdn kernels) as the parity target on the GPU.

``oracle/make_ref.py`` copies the reference's lane-path sources into the git-ignored ``oracle/_ref``; where
that folder is absent (no reference checkout when the tree was prepared) these tests skip. On identical
seeded inputs: the lane matmul within rel 1e-2 / abs 1e-3 of ``qmm.lane_matmul`` and of the tiled
``qmm_fast.matmul``; a small dense hybrid forward with logits close to ``forward.tree_forward`` and the same
greedy tokens; the MoE router, selection and expert block against ``families/qwen4_exp/cuda/moe.py``.
The package under test never imports any of it.
"""

import sys
from pathlib import Path

import pytest
import torch

from oracle import lane_oracle as O
from tests.helpers import assert_close

pytestmark = pytest.mark.gpu
REF = Path(__file__).resolve().parents[1] / "oracle" / "_ref"
BF = torch.bfloat16


@pytest.fixture(scope="module")
def ref(lib):
    if not (REF / "tensorfold").is_dir():
        pytest.skip("oracle/_ref is absent: run `python oracle/make_ref.py` where the reference checkout exists")
    sys.path.insert(0, str(REF))
    try:
        import tensorfold.families.qwen3_5.cuda.qmm as rq       # noqa: F401  (Triton must be importable)
    except Exception as exc:                                     # pragma: no cover
        pytest.skip(f"the reference's Triton path does not import here: {exc}")
    yield sys.modules["tensorfold"]
    sys.path.remove(str(REF))


@pytest.mark.parametrize("n,k,rows,rtn", [(17408, 5120, 8, True), (5120, 6144, 13, False), (1024, 5120, 1, False)])
def test_lane_matmul_against_the_reference_kernels(ref, n, k, rows, rtn):
    from tensorfold.families.qwen3_5.cuda import qmm as rqmm, qmm_fast
    from tensorfold.families.qwen3_5.cuda.weights import QLinear
    from tensorfold_b200 import lane_qmm

    gen = torch.Generator().manual_seed(n + k)
    if rtn:
        words, scales, biases = O.rtn_quantize(0.02 * torch.randn((n, k), generator=gen), 64)
    else:
        q = O.random_q4(gen, n, k, 64)
        words, scales, biases = q.words, q.scales, q.biases
    x = torch.randn((rows, k), generator=gen).to(BF).cuda()
    wd, sd, bd = words.cuda(), scales.cuda(), biases.cuda()
    ours = lane_qmm.lane_matmul(x, lane_qmm.tile_weight(wd, sd, bd, 64))
    theirs = rqmm.lane_matmul(x, wd, sd, bd)
    assert_close(ours, theirs.cpu(), f"vs qmm.lane_matmul {n}x{k}", rel=1e-2, abs_=1e-3)
    tiled = qmm_fast.matmul(x, qmm_fast.tile(QLinear(wd, sd, bd)))
    assert_close(ours, tiled.cpu(), f"vs qmm_fast.matmul {n}x{k}", rel=1e-2, abs_=1e-3)


def _reference_weights(model, dev):
    from tensorfold.families.qwen3_5.cuda.weights import Attention, Config, GDN, Layer, QLinear, Weights

    c = model["config"]

    def ql(q):
        return QLinear(q.words.to(dev), q.scales.to(dev), q.biases.to(dev))

    layers = []
    for src in model["layers"]:
        t = lambda name: src[name].to(dev)
        if src["linear"]:
            gdn = GDN(ql(src["qkv"]), ql(src["z"]), ql(src["b"]), ql(src["a"]), ql(src["out"]), t("conv"), t("A_log").float(),
                      t("dt_bias").float(), t("norm"))
            layers.append(Layer(True, t("input_norm"), t("post_norm"), gdn, None, ql(src["gate"]), ql(src["up"]), ql(src["down"])))
        else:
            att = Attention(ql(src["q"]), ql(src["k"]), ql(src["v"]), ql(src["o"]), t("q_norm"), t("k_norm"))
            layers.append(Layer(False, t("input_norm"), t("post_norm"), None, att, ql(src["gate"]), ql(src["up"]), ql(src["down"])))
    rope_dims = getattr(c, "rope_dims", 0) or c.head_dim // 4
    theta = getattr(c, "rope_theta", 1e7)
    cfg = Config(hidden=c.hidden, intermediate=c.intermediate, layers=c.layers, heads=c.heads, kv_heads=c.kv_heads,
                 head_dim=c.head_dim, vocab=c.vocab, k_heads=c.k_heads, v_heads=c.v_heads, dk=c.dk, dv=c.dv, conv_kernel=4,
                 interval=getattr(c, "interval", 4), eps=getattr(c, "eps", 1e-6), rope_dims=rope_dims, rope_theta=theta, eos=(0,))
    half = rope_dims // 2
    inv_freq = (theta ** (-torch.arange(0, half, dtype=torch.float64) / half)).to(torch.float32).to(dev)
    return Weights(cfg, ql(model["embed"]), layers, model["norm"].to(dev), ql(model["head"]), inv_freq)


def test_dense_forward_against_the_reference_forward(ref):
    """4 layers (3 gated-DeltaNet + 1 attention): a 24-token prompt committed in windows, then an 8-row verify
    window; logits within 4 % of their range of the reference's ``tree_forward`` and identical greedy tokens."""

    from tensorfold.families.qwen3_5.cuda import forward as RF
    from tensorfold_b200 import forward as F

    cfg = O.Config(hidden=512, intermediate=1024, layers=4, heads=4, kv_heads=2, head_dim=256, vocab=2048, k_heads=2, v_heads=4,
                   dk=128, dv=128)
    model = O.random_model(cfg, seed=17)
    dev = torch.device("cuda")
    ours_w = F.load_weights(model, dev)
    ref_w = _reference_weights(model, dev)
    gen = torch.Generator().manual_seed(2)
    tokens = torch.randint(0, cfg.vocab, (32,), generator=gen).tolist()

    st = F.State(ours_w, 1, 128)
    rst = RF.State(ref_w)
    got, want = [], []
    for lo, hi in ((0, 16), (16, 24), (24, 32)):
        tk = torch.tensor(tokens[lo:hi], dtype=torch.int32, device=dev)
        n = hi - lo
        logits, rec = F.tree_forward(ours_w, tk, [n], st)
        F.commit(st, rec, [n])
        rl, rrec = RF.tree_forward(ref_w, tk, [-1] + list(range(n - 1)), rst)
        RF.commit(rst, rrec, list(range(n)))
        got.append(logits.float().cpu())
        want.append(rl.float().cpu())
    got, want = torch.cat(got), torch.cat(want)
    err = (got - want).abs().max() / want.abs().max()
    assert float(err) <= 0.04, float(err)
    # greedy tokens: identical wherever the reference's own top-2 margin exceeds the deviation
    top2 = want.topk(2, dim=-1).values
    clear = (top2[:, 0] - top2[:, 1]) > 2 * (got - want).abs().max(dim=-1).values
    assert int(clear.sum()) >= 24, "too few rows with a clear margin to compare greedy tokens"
    assert torch.equal(got.argmax(-1)[clear], want.argmax(-1)[clear]), "greedy tokens differ from the reference's lane path"
    print(f"REFERENCE_FORWARD max_dev_of_range={float(err):.5f} rows_compared={int(clear.sum())}/32 greedy_equal=1")


def test_moe_block_against_the_reference_moe(ref):
    """Router logits, the selection (ids and weights) and the combined expert outputs of
    ``families/qwen4_exp/cuda/moe.py`` + ``qmm.py`` on the same rows: this is what pins the MoE part of the oracle."""

    from types import SimpleNamespace

    from tensorfold.families.qwen4_exp.cuda import moe as RM, qmm as RQ
    from tensorfold_b200 import lane_moe

    d, inter, e, topk, g, rows = 512, 128, 16, 4, 32, 13
    gen = torch.Generator().manual_seed(31)
    gates = [O.random_q4(gen, inter, d, g) for _ in range(e + 1)]
    ups = [O.random_q4(gen, inter, d, g) for _ in range(e + 1)]
    downs = [O.random_q4(gen, d, inter, g) for _ in range(e + 1)]
    router_rows = (0.05 * torch.randn((e + 1, d), generator=gen)).to(BF)
    x = torch.randn((rows, d), generator=gen).to(BF)
    ex = lane_moe.make_experts(gates, ups, downs, g)
    buf = lane_moe.MoEBuffers(rows, e, topk, True, d, inter, g, "cuda")
    out = lane_moe.moe(x.cuda(), router_rows.cuda(), ex, buf)

    def stack(qs):
        return (torch.stack([q.words for q in qs]).cuda(), torch.stack([q.scales for q in qs]).cuda(), torch.stack([q.biases for q in qs]).cuda())

    one = lambda q: (q.words.cuda(), q.scales.cuda(), q.biases.cuda())
    rex = RQ.make_experts(stack(gates[:e]), stack(ups[:e]), stack(downs[:e]), (one(gates[e]), one(ups[e]), one(downs[e])))
    rcfg = SimpleNamespace(num_experts_per_tok=topk, num_experts=e, moe_intermediate_size=inter, hidden_size=d)
    rbuf = RM.MoEBuffers(rows, rcfg, "cuda")
    xd = x.cuda()
    RM.moe(xd, RQ.group_sums(xd), router_rows.cuda(), rex, rbuf, rcfg)
    torch.cuda.synchronize()
    assert torch.allclose(buf.logits.cpu(), rbuf.logits.cpu(), rtol=1e-4, atol=1e-4), "router logits"
    assert torch.equal(buf.pick.cpu(), rbuf.pick.cpu()), "picked experts"
    assert (buf.wts.cpu() - rbuf.wts.cpu()).abs().max() <= 2 ** -8, "slot weights"
    want = (rbuf.y * rbuf.wts[..., None]).sum(1).to(BF)              # the reference's combine: slots in order, one rounding
    # the reference's own bound for this block: max|y| * 2^-5 + 1e-3 per element (tests/cuda/test_flashnext_kernels.py:124-144);
    # half of it here, both sides being bf16 roundings of the same fp32 sums
    bound = float(want.float().abs().max()) * 2 ** -6 + 1e-3
    assert float((out.float().cpu() - want.float().cpu()).abs().max()) <= bound, "combined expert outputs"
    # and the oracle's MoE functions against the same reference outputs (the pin)
    pick, wts = O.moe_select(O.moe_router(x, router_rows), e, topk, True)
    assert torch.equal(pick, rbuf.pick.cpu())
    oy = O.moe_experts(x, pick, wts, gates, ups, downs, g)
    assert float((oy.float() - want.float().cpu()).abs().max()) <= bound, "oracle MoE vs reference"
    print("REFERENCE_MOE router=ok pick=equal out=close oracle=close")
