"""The allocation-free attention entry point against the ordinary one.

Some callers of this library cannot allocate device memory while serving (their memory was handed out
once at start-up, or the runtime hosting them forbids cudaMalloc on the hot path), so they cannot give
the attention kernel its scratch buffer. ``tf_lane_attention_paged_static`` keeps the chunk partials in
a fixed array inside the library instead. This test calls both entry points through the C ABI on the
same inputs, twice in a row with different shapes (the second call must not be disturbed by what the
first left in the shared array), and expects identical bits. It runs last so that a failure here
cannot hide the other tests' results.
"""

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
BF = torch.bfloat16
STATIC_BYTES = 8 << 20


def _case(seed, lens, widths, h, hk, d):
    from tensorfold_b200 import lane_attention as LA

    gen = torch.Generator().manual_seed(seed)
    s = len(lens)
    pages = sum(-(-(l + w) // 16) for l, w in zip(lens, widths))
    kv = LA.PagedKV(1, s, pages, hk, d, max(-(-(l + w) // 16) for l, w in zip(lens, widths)), "cuda")
    for i in range(s):
        kv.reserve(i, lens[i] + widths[i])
    kv.sync_table()
    kv.k.copy_(torch.randn(kv.k.shape, generator=gen).to(BF))
    kv.v.copy_(torch.randn(kv.v.shape, generator=gen).to(BF))
    r = sum(widths)
    q = torch.randn((r, h, d), generator=gen).to(BF).cuda()
    k_new = torch.randn((r, hk, d), generator=gen).to(BF).cuda()
    v_new = torch.randn((r, hk, d), generator=gen).to(BF).cuda()
    i32 = lambda v: torch.tensor(v, dtype=torch.int32).cuda()
    starts = i32([0] + list(np.cumsum(widths)))
    nkeys = i32([lens[i] + t + 1 for i in range(s) for t in range(widths[i])])
    from tensorfold_b200 import lane_attention as LA

    chunks = max(LA.chunks_for(l + w) for l, w in zip(lens, widths))
    return kv, q, k_new, v_new, i32(lens), starts, nkeys, r, s, max(widths), chunks


def _both(lib, case, h, hk, d):
    from tensorfold_b200 import _lib

    kv, q, k_new, v_new, lens, starts, nkeys, r, s, maxw, chunks = case
    stream = _lib.stream()
    need = lib.tf_attention_scratch_bytes(r, h, d, chunks)
    scratch = torch.empty(need, dtype=torch.uint8, device="cuda")
    want = torch.empty_like(q)
    got = torch.full_like(q, float("nan"))
    common = (q.data_ptr(), k_new.data_ptr(), v_new.data_ptr(), kv.k[0].data_ptr(), kv.v[0].data_ptr(), kv.table.data_ptr(),
              kv.max_pages, lens.data_ptr(), starts.data_ptr(), nkeys.data_ptr())
    tail = (r, s, maxw, chunks, h, hk, d, float(d ** -0.5), stream)
    assert lib.tf_lane_attention_paged(*common, want.data_ptr(), scratch.data_ptr(), need, *tail) == 0
    assert lib.tf_lane_attention_paged_static(*common, got.data_ptr(), *tail) == 0
    torch.cuda.synchronize()
    return got, want, common, tail


def test_static_scratch_attention_equals_the_ordinary_entry_point(lib):
    from tensorfold_b200 import _lib

    # first call: three sequences, several chunks; second call: other shapes, fewer chunks, other head size
    first = _case(1, [1500, 17, 600], [8, 3, 5], 8, 2, 128)
    got, want, _, _ = _both(lib, first, 8, 2, 128)
    assert torch.equal(got.view(torch.int16), want.view(torch.int16)), "first call differs"
    second = _case(2, [40, 700], [4, 8], 6, 1, 256)
    got, want, common, tail = _both(lib, second, 6, 1, 256)
    assert torch.equal(got.view(torch.int16), want.view(torch.int16)), "second call differs"
    # a request that would need more than the fixed array is refused and nothing is written
    out = torch.zeros_like(got)
    rows, heads, d = tail[0], tail[4], tail[6]
    too_many = STATIC_BYTES // (rows * heads * (d + 2) * 4) + 1
    big = tail[:3] + (too_many,) + tail[4:]
    assert lib.tf_attention_scratch_bytes(rows, heads, d, too_many) > STATIC_BYTES
    assert lib.tf_lane_attention_paged_static(*common, out.data_ptr(), *big) == _lib.TF_ESCRATCH
    torch.cuda.synchronize()
    assert not out.any()
