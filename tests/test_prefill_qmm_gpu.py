"""Wide-row matmul (tcgen05): parity with the oracle within the dense bf16 GEMM bound, rows independent of
their companions (across row buckets too), tile layout keeps every bit. The reference has no wide-row
kernel; its dense accuracy bound (``tests/cuda/test_qwen27_qmm.py:41-49``) is applied here too."""

import pytest
import torch

from oracle import lane_oracle as O
from tests.helpers import assert_close, assert_same_bits

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def pq(lib):
    from tensorfold_b200 import prefill_qmm

    return prefill_qmm


def make(n, k, group, seed, rows):
    gen = torch.Generator().manual_seed(seed)
    q = O.random_q4(gen, n, k, group)
    x = torch.randn((rows, k), generator=gen).to(torch.bfloat16)
    return x, q.words, q.scales, q.biases


@pytest.mark.parametrize("group", [64, 32])
@pytest.mark.parametrize("n,k", [(48, 256), (100, 192), (1024, 5120)])
def test_tile_roundtrip_keeps_every_bit(pq, n, k, group):
    _, words, scales, biases = make(n, k, group, n + k, 1)
    q = pq.tile_weight(words.cuda(), scales.cuda(), biases.cuda(), group)
    w2, s2, b2 = pq.untile_weight(q)
    assert torch.equal(w2.cpu(), words)
    assert torch.equal(s2.cpu().view(torch.int16), scales.view(torch.int16))
    assert torch.equal(b2.cpu().view(torch.int16), biases.view(torch.int16))


@pytest.mark.parametrize("group", [64, 32])
@pytest.mark.parametrize("n,k,rows", [(48, 256, 5), (272, 1088, 13), (1024, 5120, 128), (5120, 6144, 300)])
def test_parity_with_oracle(pq, n, k, rows, group):
    x, words, scales, biases = make(n, k, group, 3 * n + k, rows)
    q = pq.tile_weight(words.cuda(), scales.cuda(), biases.cuda(), group)
    y = pq.prefill_matmul(x.cuda(), q)
    torch.cuda.synchronize()
    # weights are rounded to bf16 before the product (2^-9 relative each), the output once more: elementwise
    # |err| <= rel 1e-2 of the value + 2^-8 of the sum of |w x| behind it (the dense bf16 GEMM bound); against the
    # lane arithmetic of the oracle the same bound holds
    w = O.dequantize(words, scales, biases, group)
    ref32 = x.float() @ w.T
    bound = 1e-2 * ref32.abs() + 2.0 ** -8 * (x.float().abs() @ w.abs().T)
    for want, name in ((ref32, "fp32 product"), (O.qmm(x, words, scales, biases, group).float(), "lane oracle")):
        err = (y.float().cpu() - want).abs()
        assert bool((err <= bound).all()), f"{name} {n}x{k} g{group}: worst excess {float((err - bound).max()):.4g}"
    assert float((y.float().cpu() - ref32).abs().max()) <= float(ref32.abs().max()) * 2 ** -7


@pytest.mark.parametrize("group", [64, 32])
def test_rows_do_not_depend_on_their_companions(pq, group):
    n, k = 1024, 5120
    x, words, scales, biases = make(n, k, group, 11, 128)
    q = pq.tile_weight(words.cuda(), scales.cuda(), biases.cuda(), group)
    xd = x.cuda()
    full = pq.prefill_matmul(xd, q)
    for rows in (1, 8, 16, 17, 33, 64, 100):
        part = pq.prefill_matmul(xd[:rows], q)
        assert_same_bits(part, full[:rows], f"{rows} rows vs 128 rows, group {group}")
    perm = torch.randperm(128, generator=torch.Generator().manual_seed(5)).cuda()
    assert_same_bits(pq.prefill_matmul(xd[perm], q), full[perm], "row permutation")


@pytest.mark.parametrize("group", [64, 32])
@pytest.mark.parametrize("rows", [5, 40, 128])
def test_rows_packed_by_the_lane_kernels_give_the_same_bits(pq, group, rows):
    from tensorfold_b200 import lane_qmm

    n, k = 512, 1024
    x, words, scales, biases = make(n, k, group, 23, rows)
    q = pq.tile_weight(words.cuda(), scales.cuda(), biases.cuda(), group)
    xd = x.cuda()
    direct = pq.prefill_matmul(xd, q)
    staged = pq.prefill_matmul(lane_qmm.pack_rows(xd, group), q,
                               staging=torch.empty(pq.packed_bytes(rows, k, group), dtype=torch.uint8, device="cuda"))
    assert_same_bits(staged, direct, f"packed input, {rows} rows, group {group}")


def test_weights_are_dequantised_to_bf16_with_one_rounding(pq):
    """The kernel's arithmetic, stated: w = bf16(s * q + b), products summed in fp32. Against that statement in
    fp64 the result is within fp32 accumulation error of the exact sum (far tighter than the oracle bound)."""

    n, k, group, rows = 256, 2048, 64, 32
    x, words, scales, biases = make(n, k, group, 77, rows)
    q = pq.tile_weight(words.cuda(), scales.cuda(), biases.cuda(), group)
    y = pq.prefill_matmul(x.cuda(), q, f32=True).cpu().double()
    codes = torch.stack([(words >> (4 * i)) & 0xF for i in range(8)], dim=-1).reshape(n, k).float()
    w = (codes * scales.float().repeat_interleave(group, 1) + biases.float().repeat_interleave(group, 1)).to(torch.bfloat16)
    want = x.double() @ w.double().T
    bound = (x.double().abs() @ w.double().abs().T).max() * 2.0 ** -18
    assert float((y - want).abs().max()) <= float(bound)
