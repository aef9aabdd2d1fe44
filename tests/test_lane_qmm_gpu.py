"""Lane matmul on the GPU: rows alone == rows in a window (bits), parity with the oracle (tolerance).

Test ideas follow the reference's ``tests/cuda/test_qwen27_qmm.py`` (rows 1..128 and a row
permutation, accuracy bound, tiled layout keeps bits) and ``tests/test_lane_qmm.py`` (shape list).
"""

import pytest
import torch

from oracle import lane_oracle as O
from tests.helpers import assert_close, assert_same_bits

pytestmark = pytest.mark.gpu

SHAPES_27B = [(48, 5120), (1024, 5120), (5120, 6144), (10240, 5120), (5120, 17408), (17408, 5120)]
ROWS = [1, 2, 3, 7, 8, 9, 15, 16, 17, 31, 32, 33, 63, 64, 65, 100, 127, 128]


def make(n, k, group, seed, rows=8, rtn=False):
    gen = torch.Generator().manual_seed(seed)
    if rtn:
        words, scales, biases = O.rtn_quantize(0.02 * torch.randn((n, k), generator=gen), group)
    else:
        q = O.random_q4(gen, n, k, group)
        words, scales, biases = q.words, q.scales, q.biases
    x = torch.randn((rows, k), generator=gen).to(torch.bfloat16)
    return x, words, scales, biases


@pytest.fixture(scope="module")
def qmm(lib):
    from tensorfold_b200 import lane_qmm

    return lane_qmm


@pytest.mark.parametrize("group", [64, 32])
@pytest.mark.parametrize("n,k", [(48, 256), (40, 64), (100, 192), (1024, 5120), (768, 2048)])
def test_tile_roundtrip_keeps_every_bit(qmm, n, k, group):
    _, words, scales, biases = make(n, k, group, seed=n + k)
    q = qmm.tile_weight(words.cuda(), scales.cuda(), biases.cuda(), group)
    assert q.tiled.numel() == (-(-n // 256)) * 16 * (k // 64) * (576 if group == 64 else 640)
    w2, s2, b2 = qmm.untile_weight(q)
    assert torch.equal(w2.cpu(), words) and torch.equal(s2.cpu().view(torch.int16), scales.view(torch.int16))
    assert torch.equal(b2.cpu().view(torch.int16), biases.view(torch.int16))


def test_group_sums(qmm):
    gen = torch.Generator().manual_seed(1)
    x = torch.randn((9, 5120), generator=gen).to(torch.bfloat16)
    for group in (64, 32):
        xs = qmm.group_sums(x.cuda(), group).cpu()
        assert torch.allclose(xs, O.group_sums(x, group), rtol=1e-5, atol=1e-5)
        one = torch.cat([qmm.group_sums(x[i:i + 1].cuda(), group) for i in range(9)]).cpu()
        assert_same_bits(xs, one, "group sums alone vs together")


@pytest.mark.parametrize("group", [64, 32])
@pytest.mark.parametrize("n,k", [(48, 256), (40, 64), (100, 192), (272, 1088), (1024, 5120), (5120, 6144)])
def test_parity_with_oracle(qmm, n, k, group):
    x, words, scales, biases = make(n, k, group, seed=7 * n + k, rows=13)
    q = qmm.tile_weight(words.cuda(), scales.cuda(), biases.cuda(), group)
    y = qmm.lane_matmul(x.cuda(), q)
    torch.cuda.synchronize()
    want = O.qmm(x, words, scales, biases, group)
    assert_close(y, want, f"qmm {n}x{k} g{group}")
    # the reference's own accuracy bound: err <= max|ref| * 2^-7 (tests/cuda/test_qwen27_qmm.py:41-49)
    ref32 = x.float() @ O.dequantize(words, scales, biases, group).T
    assert float((y.float().cpu() - ref32).abs().max()) <= float(ref32.abs().max()) * 2 ** -7


def test_config1_shape_rtn_weights(qmm):
    # x ~ N(0,1) [8, 5120]; W ~ N(0, 0.02) [17408, 5120] RTN 4-bit group 64
    x, words, scales, biases = make(17408, 5120, 64, seed=0, rows=8, rtn=True)
    q = qmm.tile_weight(words.cuda(), scales.cuda(), biases.cuda(), 64)
    xc = x.cuda()
    y = qmm.lane_matmul(xc, q)
    assert_close(y, O.qmm(x, words, scales, biases, 64), "config 1")
    for i in range(8):
        assert_same_bits(y[i:i + 1], qmm.lane_matmul(xc[i:i + 1], q), f"row {i} alone")
    assert_same_bits(y, qmm.lane_matmul(xc, q), "second run")


@pytest.mark.parametrize("n,k,group", [(n, k, 64) for n, k in SHAPES_27B] + [(768, 2048, 32), (2048, 768, 32), (512, 2048, 32), (2048, 512, 32), (100, 192, 32)])
def test_rows_alone_equal_rows_in_window(qmm, n, k, group):
    x, words, scales, biases = make(n, k, group, seed=n ^ k, rows=128)
    q = qmm.tile_weight(words.cuda(), scales.cuda(), biases.cuda(), group)
    xc = x.cuda()
    full = qmm.lane_matmul(xc, q)
    single = torch.cat([qmm.lane_matmul(xc[i:i + 1], q) for i in (0, 1, 7, 8, 64, 127)])
    assert_same_bits(full[[0, 1, 7, 8, 64, 127]], single, "rows alone")
    for m in ROWS:
        assert_same_bits(qmm.lane_matmul(xc[:m], q), full[:m], f"{m} rows")
    perm = torch.randperm(128, generator=torch.Generator().manual_seed(5)).cuda()
    assert_same_bits(qmm.lane_matmul(xc[perm], q), full[perm], "row permutation")
    big = qmm.lane_matmul(torch.cat([xc, xc[:70]]), q)            # more than one launch
    assert_same_bits(big, torch.cat([full, full[:70]]), "198 rows")
    torch.cuda.synchronize()
    from tensorfold_b200 import _lib
    _lib.status(xc.device).raise_if_set()


def test_fp32_partial_rounds_to_the_bf16_output(qmm):
    x, words, scales, biases = make(5120, 6144, 64, seed=3, rows=12)
    q = qmm.tile_weight(words.cuda(), scales.cuda(), biases.cuda(), 64)
    y = qmm.lane_matmul(x.cuda(), q)
    p = qmm.lane_matmul(x.cuda(), q, f32=True)
    assert p.dtype == torch.float32
    assert_same_bits(p.to(torch.bfloat16), y, "fp32 partial")


def test_rows_packed_by_the_caller_and_launch_numbers_in_step(qmm):
    x, words, scales, biases = make(1024, 5120, 64, seed=4, rows=8)
    q = qmm.tile_weight(words.cuda(), scales.cuda(), biases.cuda(), 64)
    xc = x.cuda()
    packed = qmm.pack_rows(xc)
    assert_same_bits(qmm.lane_matmul(packed, q), qmm.lane_matmul(xc, q), "rows packed by the caller")
    torch.cuda.synchronize()
    # every worker advanced its launch number once per call: they stay equal (what the K-segment tags rely on)
    scratch = qmm.scratch_for(xc.device)
    off = 16384 + 2 * 148 * 128 * 256 * 4
    epochs = scratch[off:off + 148 * 4].view(torch.int32).cpu()
    assert int(epochs.min()) == int(epochs.max()) and int(epochs[0]) > 0
    assert int(scratch[:16384].view(torch.int32).abs().sum()) == 0         # the prefill kernel's ticket words


def test_reference_call_shape_with_stored_weights(qmm):
    """``lane_matmul(x, weight, scales, biases, xs=..., sk=...)`` as the reference calls it (families/qwen3_5/cuda/qmm.py:117-144)."""

    x, words, scales, biases = make(1024, 5120, 64, seed=12, rows=8)
    wd, sd, bd = words.cuda(), scales.cuda(), biases.cuda()
    tiled = qmm.lane_matmul(x.cuda(), qmm.tile_weight(wd, sd, bd, 64))
    xs = qmm.group_sums(x.cuda())
    assert_same_bits(qmm.lane_matmul(x.cuda(), wd, sd, bd, xs=xs, sk=qmm.split_k(1024, 5120)), tiled, "stored call shape")
    with pytest.raises(ValueError):
        qmm.lane_matmul(x.cuda(), wd, sd, bd, sk=qmm.split_k(1024, 5120) + 1)
    with pytest.raises(ValueError):
        qmm.lane_matmul(x.cuda(), wd)


def test_wrong_arguments_raise(qmm):
    x, words, scales, biases = make(64, 128, 64, seed=2)
    q = qmm.tile_weight(words.cuda(), scales.cuda(), biases.cuda(), 64)
    with pytest.raises(ValueError):
        qmm.lane_matmul(x.cuda().float(), q)
    with pytest.raises(ValueError):
        qmm.lane_matmul(x.cuda()[:, :64], q)
    with pytest.raises(ValueError):
        qmm.lane_matmul(x, q)                      # CPU tensor: there is no CPU path
    with pytest.raises(ValueError):
        qmm.tile_weight(words.cuda(), scales.cuda().float(), biases.cuda())


def test_head_shape_248320_by_5120(qmm):
    """The vocabulary head of the 27B-class model (the largest matmul of a step, 715 MB of weights): a row alone has
    the bits of the row in an 8-row window, and 4096 sampled output columns agree with the oracle."""

    n, k, group, rows = 248320, 5120, 64, 8
    gen = torch.Generator(device="cuda").manual_seed(77)
    words = torch.randint(-2 ** 31, 2 ** 31 - 1, (n, k // 8), generator=gen, dtype=torch.int64, device="cuda").to(torch.int32)
    scales = ((torch.rand((n, k // group), generator=gen, device="cuda") / 8 + 1 / 64) * (4.0 / k ** 0.5)).to(torch.bfloat16)
    biases = (-7.5 * scales.float()).to(torch.bfloat16)
    x = torch.randn((rows, k), generator=gen, device="cuda").to(torch.bfloat16)
    q = qmm.tile_weight(words, scales, biases, group)
    full = qmm.lane_matmul(x, q)
    for r in (0, 3, 7):
        assert_same_bits(qmm.lane_matmul(x[r:r + 1], q), full[r:r + 1], f"head: row {r} alone")
    cols = torch.randperm(n, generator=torch.Generator().manual_seed(5))[:4096].sort().values
    want = O.qmm(x.cpu(), words[cols.cuda()].cpu(), scales[cols.cuda()].cpu(), biases[cols.cuda()].cpu(), group)
    assert_close(full[:, cols.cuda()], want, "head columns vs oracle")
