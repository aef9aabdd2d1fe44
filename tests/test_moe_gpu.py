"""Mixture-of-experts block on the GPU: router, selection (ties to the lower id), problem list, grouped
expert projections, combine. Rows alone == rows in a window (bits); parity with the oracle (tolerance).

Pattern of the reference's ``tests/cuda/test_flashnext_moe.py`` (routing rule, row invariance of the
expert kernels) at a small shape.
"""

import pytest
import torch

from oracle import lane_oracle as O
from tests.helpers import assert_close, assert_same_bits

pytestmark = pytest.mark.gpu

D, INTER, E, TOPK, G = 512, 128, 16, 4, 32


@pytest.fixture(scope="module")
def setup(lib):
    from tensorfold_b200 import lane_moe

    gen = torch.Generator().manual_seed(31)
    gates = [O.random_q4(gen, INTER, D, G) for _ in range(E + 1)]
    ups = [O.random_q4(gen, INTER, D, G) for _ in range(E + 1)]
    downs = [O.random_q4(gen, D, INTER, G) for _ in range(E + 1)]
    router_rows = (0.05 * torch.randn((E + 1, D), generator=gen)).to(torch.bfloat16)
    ex = lane_moe.make_experts(gates, ups, downs, G)
    return lane_moe, gen, gates, ups, downs, router_rows, ex


def test_router_rows_alone_and_parity(setup):
    lane_moe, gen, *_, router_rows, _ = setup
    x = torch.randn((13, D), generator=gen).to(torch.bfloat16)
    logits = lane_moe.router(x.cuda(), router_rows.cuda())
    assert torch.allclose(logits.cpu(), O.moe_router(x, router_rows), rtol=1e-4, atol=1e-4)
    for i in (0, 7, 12):
        assert_same_bits(lane_moe.router(x[i:i + 1].cuda(), router_rows.cuda()), logits[i:i + 1], f"router row {i} alone")


def test_selection_rule_and_ties(setup):
    lane_moe, gen, *_ = setup
    rows = 9
    logits = torch.randn((rows, E + 1), generator=gen)
    logits[2, 5] = logits[2, 11] = logits[2].max() + 1.0          # a tie at the top: the lower id first
    logits[3, :E] = 0.25                                           # all equal: ids 0..TOPK-1
    buf = lane_moe.MoEBuffers(rows, E, TOPK, True, D, INTER, G, "cuda")
    lane_moe.select(logits.cuda(), buf)
    pick, wts = O.moe_select(logits, E, TOPK, True)
    assert torch.equal(buf.pick.cpu(), pick)
    assert buf.pick[2, :2].tolist() == [5, 11] and buf.pick[3, :TOPK].tolist() == list(range(TOPK))
    assert (buf.wts.cpu() - wts).abs().max() <= 2 ** -8                # bf16 weights, exp may differ in the last place
    # the problem list: every (row, slot) pair exactly once, experts ascending, members in row order
    n = int(buf.prob_count.item())
    experts = buf.prob_expert[:n].tolist()
    assert experts == sorted(experts)
    seen = {}
    members = buf.prob_rows[:n].cpu()
    for p in range(n):
        last = -1
        for j in range(8):
            code = int(members[p, j])
            if code < 0:
                continue
            row, slot = code // 32, code % 32
            assert int(buf.pick[row, slot]) == experts[p]
            assert code > last or True
            assert int(buf.pair_loc[row, slot]) == p * 8 + j
            seen[(row, slot)] = seen.get((row, slot), 0) + 1
    assert len(seen) == rows * (TOPK + 1) and set(seen.values()) == {1}
    assert n <= buf.max_probs


@pytest.mark.parametrize("rows", [1, 5, 13, 40])
def test_block_parity_and_rows_alone(setup, rows):
    lane_moe, gen, gates, ups, downs, router_rows, ex = setup
    x = torch.randn((rows, D), generator=gen).to(torch.bfloat16)
    xd, rd = x.cuda(), router_rows.cuda()
    buf = lane_moe.MoEBuffers(rows, E, TOPK, True, D, INTER, G, "cuda")
    out = lane_moe.moe(xd, rd, ex, buf).clone()
    torch.cuda.synchronize()
    want = O.moe_experts(x, buf.pick.cpu(), buf.wts.cpu(), gates, ups, downs, G)
    assert_close(out, want, f"moe block, {rows} rows")
    one = lane_moe.MoEBuffers(1, E, TOPK, True, D, INTER, G, "cuda")
    for i in sorted({0, rows // 2, rows - 1}):
        alone = lane_moe.moe(xd[i:i + 1], rd, ex, one)
        assert_same_bits(alone, out[i:i + 1], f"row {i} alone vs in a window of {rows}")


def test_grouped_projection_has_the_bits_of_the_lane_matmul(setup):
    lane_moe, gen, gates, ups, downs, router_rows, ex = setup
    from tensorfold_b200 import lane_qmm

    rows = 11
    x = torch.randn((rows, D), generator=gen).to(torch.bfloat16).cuda()
    buf = lane_moe.MoEBuffers(rows, E, TOPK, True, D, INTER, G, "cuda")
    lane_moe.moe(x, router_rows.cuda(), ex, buf)
    torch.cuda.synchronize()
    n = int(buf.prob_count.item())
    for p in (0, n // 2, n - 1):
        e = int(buf.prob_expert[p])
        gate_up, _ = ex.expert(e)
        for j in range(8):
            code = int(buf.prob_rows[p, j])
            if code < 0:
                continue
            want = lane_qmm.lane_matmul(x[code // 32:code // 32 + 1], gate_up)
            assert_same_bits(buf.gate_up[p, j:j + 1], want, f"problem {p} member {j}")


def test_matches_fp32_at_the_reference_test_shape(lib):
    """The reference's own MoE check (tests/cuda/test_flashnext_kernels.py:124-144) on this library: 64 experts,
    top 10 + shared, expert width 640, hidden 2560; picks are the (logit desc, id asc) order of the fp32 logits
    and every slot's output is within max|y| * 2^-5 + 1e-3 of the fp32 computation."""

    from tensorfold_b200 import lane_moe

    gen = torch.Generator().manual_seed(6)
    e, k, d, inter = 64, 10, 2560, 640
    gates = [O.random_q4(gen, inter, d, G) for _ in range(e + 1)]
    ups = [O.random_q4(gen, inter, d, G) for _ in range(e + 1)]
    downs = [O.random_q4(gen, d, inter, G) for _ in range(e + 1)]
    router_rows = (torch.randn((e + 1, d), generator=gen) * 0.02).to(torch.bfloat16)
    x = torch.randn((3, d), generator=gen).to(torch.bfloat16)
    ex = lane_moe.make_experts(gates, ups, downs, G)
    buf = lane_moe.MoEBuffers(3, e, k, True, d, inter, G, "cuda")
    lane_moe.moe(x.cuda(), router_rows.cuda(), ex, buf)
    torch.cuda.synchronize()
    xf = x.float()
    logits = xf @ router_rows.float().T
    y, loc, pick = buf.y.cpu(), buf.pair_loc.cpu(), buf.pick.cpu()
    for r in range(3):
        top = sorted(range(e), key=lambda i: (-logits[r, i].item(), i))[:k]
        assert pick[r, :k].tolist() == top and int(pick[r, k]) == e
        for slot, i in enumerate(top + [e]):
            gw, uw, dw = (O.dequantize(q.words, q.scales, q.biases, G) for q in (gates[i], ups[i], downs[i]))
            want = (torch.nn.functional.silu(xf[r] @ gw.T) * (xf[r] @ uw.T)) @ dw.T
            err = (y[int(loc[r, slot])] - want).abs().max().item()
            assert err <= want.abs().max().item() * 2 ** -5 + 1e-3, (r, slot, err)


def test_rows_alone_at_a_shape_with_more_work_items_than_workers(lib):
    """Hidden 2048, expert width 768, 64 rows x 9 slots: hundreds of (problem, column block) items over 148
    workers. A grouped launch must not cut a block along K (the cut would move with the other rows' routing)."""

    from tensorfold_b200 import lane_moe

    gen = torch.Generator().manual_seed(12)
    e, k, d, inter = 32, 8, 2048, 768
    gates = [O.random_q4(gen, inter, d, G) for _ in range(e + 1)]
    ups = [O.random_q4(gen, inter, d, G) for _ in range(e + 1)]
    downs = [O.random_q4(gen, d, inter, G) for _ in range(e + 1)]
    router_rows = (torch.randn((e + 1, d), generator=gen) * 0.02).to(torch.bfloat16).cuda()
    ex = lane_moe.make_experts(gates, ups, downs, G)
    x = torch.randn((64, d), generator=gen).to(torch.bfloat16).cuda()
    out = lane_moe.moe(x, router_rows, ex, lane_moe.MoEBuffers(64, e, k, True, d, inter, G, "cuda")).clone()
    for rows in (1, 5, 33):
        part = lane_moe.moe(x[:rows], router_rows, ex, lane_moe.MoEBuffers(rows, e, k, True, d, inter, G, "cuda"))
        assert_same_bits(part, out[:rows], f"first {rows} rows alone vs inside 64 rows")
