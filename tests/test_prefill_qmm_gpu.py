"""Prefill-width matmul (tcgen05): parity with the oracle, rows independent of their companions,
tile layout keeps every bit. The reference has no test of its own for this phase beyond the dense
GEMM accuracy bound of ``tests/cuda/test_qwen27_qmm.py:41-49``, which is applied here too."""

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
    assert_close(y, O.qmm(x, words, scales, biases, group), f"prefill qmm {n}x{k} g{group}")
    ref32 = x.float() @ O.dequantize(words, scales, biases, group).T
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
