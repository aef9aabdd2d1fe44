"""The CPU oracle against the golden outputs of the reference's own Python code (tests/golden)."""

from pathlib import Path

import numpy as np
import torch

from oracle import lane_oracle as O

GOLD = Path(__file__).parent / "golden"


def test_dequantize_matches_reference_both_groups():
    z = np.load(GOLD / "qmm_dequantize.npz")
    gen = torch.Generator().manual_seed(int(z["seed"]))
    wf = 0.02 * torch.randn((48, 256), generator=gen)
    x = torch.randn((5, 256), generator=gen).to(torch.bfloat16)
    for group in (64, 32):
        words, scales, biases = O.rtn_quantize(wf, group)
        deq = O.dequantize(words, scales, biases, group)
        assert np.array_equal(deq.numpy(), z[f"deq{group}"])
        assert np.array_equal(O.qmm(x, words, scales, biases, group).float().numpy(), z[f"y{group}"])
        # the RTN harness itself: codes reproduce the weight to within half a step
        assert float((deq - wf).abs().max()) <= float(scales.float().max()) * 0.51 + 1e-3
        # ordered-group form agrees with the plain product to fp32 rounding
        yo = O.qmm_ordered(x, words, scales, biases, group, f32=True)
        assert torch.allclose(yo, x.float() @ deq.T, rtol=1e-4, atol=1e-4)


def test_pack_unpack_roundtrip():
    gen = torch.Generator().manual_seed(3)
    q = torch.randint(0, 16, (7, 128), generator=gen)
    assert torch.equal(O.unpack_nibbles(O.pack_nibbles(q)), q)


def test_dense_forward_matches_reference():
    z = np.load(GOLD / "dense_forward_tiny.npz", allow_pickle=True)
    cfg = O.Config(**{k: (float(v) if k in ("eps", "rope_theta") else int(v)) for k, v in z["config"]})
    model = O.random_model(cfg, seed=int(z["model_seed"]))
    tokens = torch.from_numpy(z["tokens"])
    st = O.State.fresh(model)
    torch.set_num_threads(1)
    logits = [O.forward(model, tokens[:6], st)]
    for i in range(6, 9):
        logits.append(O.forward(model, tokens[i:i + 1], st))
    got = torch.cat(logits).numpy()
    want = z["logits"]
    # same torch ops in the same order: equal up to BLAS blocking differences
    assert np.allclose(got, want, rtol=2e-3, atol=2e-3), float(np.abs(got - want).max())
    assert (got.argmax(-1) == want.argmax(-1)).all()
    rec = torch.stack([r for r in st.rec if r is not None]).numpy()
    assert np.allclose(rec, z["rec"], rtol=2e-3, atol=2e-4)
    assert np.allclose(st.kv[3][0].float().numpy(), z["k_cache"], rtol=1e-2, atol=1e-2)
    assert np.allclose(st.conv[0].float().numpy(), z["conv"], rtol=1e-2, atol=1e-2)


def test_keyed_sampling_matches_reference():
    z = np.load(GOLD / "exact_sampling.npz")
    vals, ids, positions = z["vals"], z["ids"], z["positions"]
    assert np.array_equal(O.uniform_rows(1234, positions[:8], ids[:8]), z["u"])
    for name, s in (("default", O.Sampling(seed=1234)), ("hot", O.Sampling(seed=99, temperature=1.7, top_k=10, top_p=0.8)),
                    ("all", O.Sampling(seed=5, temperature=0.7, top_k=0, top_p=1.0))):
        assert O.choose_rows(vals, ids, positions, s) == z["pick_" + name].tolist()


def test_topk_rule_ties_by_lower_id():
    x = np.array([[1.0, 3.0, 3.0, 2.0, 3.0], [0.0, 0.0, 0.0, 0.0, 0.0]], dtype=np.float32)
    idx, val = O.topk_rows(x, 3)
    assert idx.tolist() == [[1, 2, 4], [0, 1, 2]]
    assert val.tolist() == [[3.0, 3.0, 3.0], [0.0, 0.0, 0.0]]
