"""Generate the golden fixtures that pin ``oracle/lane_oracle.py`` to the TensorFold reference.

Run once in a container that holds the reference checkout (it cannot travel to the GPU box):

    PYTHONPATH=/path/to/reference/src python tests/golden/make_golden.py

It imports the reference's own Python code — ``families/qwen3_5/cuda/reference.py`` (plain fp32
forward), ``qmm.dequantize`` (group 64), ``families/qwen4_exp/cuda/qmm.dequantize`` (group 32),
``engine/exact_sampling.py`` — runs it on seeded inputs and stores inputs' seeds plus outputs as
small ``.npz`` files next to this script. The random inputs come from ``oracle.lane_oracle``'s
generators, so a test can rebuild the same inputs from the seed and compare outputs.
"""

from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))

from oracle import lane_oracle as O  # noqa: E402

from tensorfold.engine import exact_sampling as ref_sampling  # noqa: E402
from tensorfold.families.qwen3_5.cuda import qmm as ref_qmm  # noqa: E402
from tensorfold.families.qwen3_5.cuda import reference as ref_model  # noqa: E402
from tensorfold.families.qwen3_5.cuda import weights as ref_weights  # noqa: E402
from tensorfold.families.qwen4_exp.cuda import qmm as ref_qmm32  # noqa: E402

TINY = dict(hidden=256, intermediate=512, layers=4, heads=4, kv_heads=2, head_dim=64, vocab=512, k_heads=2, v_heads=4,
            dk=64, dv=64, conv_kernel=4, interval=4, eps=1e-6, rope_dims=16, rope_theta=1e7)


def to_reference(model: dict) -> ref_weights.Weights:
    """The oracle's random model as the reference's own dataclasses (same tensors)."""

    c = model["config"]
    cfg = ref_weights.Config(hidden=c.hidden, intermediate=c.intermediate, layers=c.layers, heads=c.heads,
                             kv_heads=c.kv_heads, head_dim=c.head_dim, vocab=c.vocab, k_heads=c.k_heads,
                             v_heads=c.v_heads, dk=c.dk, dv=c.dv, conv_kernel=c.conv_kernel, interval=c.interval,
                             eps=c.eps, rope_dims=c.rope_dims, rope_theta=c.rope_theta, eos=(0,))

    def ql(q):
        return ref_weights.QLinear(q.words, q.scales, q.biases)

    layers = []
    for layer in model["layers"]:
        gdn = attn = None
        if layer["linear"]:
            gdn = ref_weights.GDN(qkv=ql(layer["qkv"]), z=ql(layer["z"]), b=ql(layer["b"]), a=ql(layer["a"]),
                                  out=ql(layer["out"]), conv=layer["conv"], A_log=layer["A_log"],
                                  dt_bias=layer["dt_bias"], norm=layer["norm"])
        else:
            attn = ref_weights.Attention(q=ql(layer["q"]), k=ql(layer["k"]), v=ql(layer["v"]), o=ql(layer["o"]),
                                         q_norm=layer["q_norm"], k_norm=layer["k_norm"])
        layers.append(ref_weights.Layer(linear=layer["linear"], input_norm=layer["input_norm"],
                                        post_norm=layer["post_norm"], gdn=gdn, attn=attn, gate=ql(layer["gate"]),
                                        up=ql(layer["up"]), down=ql(layer["down"])))
    return ref_weights.Weights(config=cfg, embed=ql(model["embed"]), layers=layers, norm=model["norm"],
                               head=ql(model["head"]), inv_freq=model["inv_freq"])


def main() -> None:
    torch.manual_seed(0)
    torch.set_num_threads(1)          # the stored values are compared tightly: keep the reduction order fixed
    # 1. dequantize, both group sizes, and the reference projection
    gen = torch.Generator().manual_seed(11)
    wf = 0.02 * torch.randn((48, 256), generator=gen)
    x = torch.randn((5, 256), generator=gen).to(torch.bfloat16)
    out = {}
    for group, mod in ((64, ref_qmm), (32, ref_qmm32)):
        words, scales, biases = O.rtn_quantize(wf, group)
        deq = mod.dequantize(words, scales, biases)
        out[f"deq{group}"] = deq.numpy()
        out[f"y{group}"] = (x.float() @ deq.T).to(torch.bfloat16).float().numpy()
    np.savez_compressed(HERE / "qmm_dequantize.npz", seed=11, **out)

    # 2. the reference forward on a tiny hybrid model: a 6-token prompt, then 3 serial steps
    cfg = O.Config(**TINY)
    model = O.random_model(cfg, seed=5)
    w = to_reference(model)
    st = ref_model.State(w)
    gen = torch.Generator().manual_seed(6)
    tokens = torch.randint(0, cfg.vocab, (9,), generator=gen)
    logits = [ref_model.forward(w, tokens[:6], st)]
    for i in range(6, 9):
        logits.append(ref_model.forward(w, tokens[i:i + 1], st))
    rec = torch.stack([r for r in st.rec if r is not None])
    np.savez_compressed(HERE / "dense_forward_tiny.npz", model_seed=5, token_seed=6, tokens=tokens.numpy(),
                        logits=torch.cat(logits).numpy(), rec=rec.numpy(),
                        k_cache=st.kv[3][0].float().numpy(), conv=st.conv[0].float().numpy(),
                        config=np.array(list(TINY.items()), dtype=object))

    # 3. keyed sampling: choose_rows on random candidate rows, ties included
    rng = np.random.default_rng(7)
    vals = np.round(rng.normal(size=(64, 28)) * 4) / 4          # quarter steps: many exact ties
    ids = np.stack([rng.permutation(5000)[:28] for _ in range(64)]).astype(np.int64)
    positions = rng.integers(0, 100000, size=64)
    picks = {}
    for name, s in (("default", ref_sampling.Sampling(seed=1234)),
                    ("hot", ref_sampling.Sampling(seed=99, temperature=1.7, top_k=10, top_p=0.8)),
                    ("all", ref_sampling.Sampling(seed=5, temperature=0.7, top_k=0, top_p=1.0))):
        picks[name] = np.array(ref_sampling.choose_rows(vals.astype(np.float32), ids, positions, s))
    u = ref_sampling.uniform_rows(1234, positions[:8], ids[:8])
    np.savez_compressed(HERE / "exact_sampling.npz", vals=vals.astype(np.float32), ids=ids, positions=positions, u=u,
                        **{"pick_" + k: v for k, v in picks.items()})
    print("wrote", sorted(p.name for p in HERE.glob("*.npz")))


if __name__ == "__main__":
    main()
