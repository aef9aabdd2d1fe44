"""CPU oracle for the lane-verify forward. TEST INFRASTRUCTURE ONLY.

A plain restatement, in fp32 PyTorch/numpy on the CPU, of the arithmetic the TensorFold reference
defines for this path. Only ``tests/``, ``__graft_entry__.smoke()`` and ``bench.py``'s CPU-baseline
legs may import it; the product package never does (it has no CPU path at all).

Each function cites the reference file (path inside the TensorFold project) it follows. The oracle
is pinned by ``tests/golden/*.npz``: outputs of the reference's own Python code
(``families/qwen3_5/cuda/reference.py``, ``qmm.dequantize``, ``families/qwen4_exp/cuda/qmm.dequantize``,
``engine/exact_sampling.py``) run in the build container by ``tests/golden/make_golden.py``;
``tests/test_oracle.py`` checks the oracle against them.

Where the reference rounds to bf16 (values the model stores) the oracle rounds too; everything
else is fp32, as in ``reference.py``. The CUDA kernels are compared with this oracle within the
tolerance the path states (bf16 outputs: rel 1e-2 / abs 1e-3); bit-exactness is a property of the
kernels against themselves (row alone == row in a window), never against this file.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch

BF16 = torch.bfloat16


# ------------------------------------------------------------------------------------------------
# 4-bit group-affine weights
# ------------------------------------------------------------------------------------------------

def rtn_quantize(wf: torch.Tensor, group: int = 64):
    """Harness-defined round-to-nearest affine 4-bit quantisation (the reference takes packed
    weights as given; its tests draw random words, ``tests/cuda/test_qwen27_qmm.py:17-24``).

    Per (row, group): scale = (max-min)/15 (1 when zero), bias = min, q = clamp(round((w-bias)/scale)),
    scale and bias rounded to bf16; 8 nibbles per uint32, element i at bits 4*(i%8) of word i//8
    (``families/qwen3_5/cuda/qmm.py:11-12``). Returns (words int32 (N,K/8), scales, biases bf16 (N,K/group)).
    """

    n, k = wf.shape
    g = wf.float().reshape(n, k // group, group)
    lo, hi = g.min(-1).values, g.max(-1).values
    scale = (hi - lo) / 15.0
    scale = torch.where(scale == 0, torch.ones_like(scale), scale)
    q = torch.clamp(torch.round((g - lo[..., None]) / scale[..., None]), 0, 15).to(torch.int64).reshape(n, k)
    return pack_nibbles(q), scale.to(BF16), lo.to(BF16)


def pack_nibbles(q: torch.Tensor) -> torch.Tensor:
    """(N, K) integers 0..15 -> (N, K/8) int32 words, little-nibble-first."""

    n, k = q.shape
    shifts = torch.arange(8, dtype=torch.int64) * 4
    words = (q.reshape(n, k // 8, 8).to(torch.int64) << shifts).sum(-1)
    words = torch.where(words >= 2 ** 31, words - 2 ** 32, words)
    return words.to(torch.int32)


def unpack_nibbles(words: torch.Tensor) -> torch.Tensor:
    """(N, K/8) int32 words -> (N, K) integers 0..15 (``qmm.py:147-156``)."""

    n, k8 = words.shape
    w = words.view(torch.int32).to(torch.int64) & 0xFFFFFFFF
    shifts = torch.arange(8, dtype=torch.int64) * 4
    return ((w[:, :, None] >> shifts) & 0xF).reshape(n, k8 * 8)


def dequantize(words: torch.Tensor, scales: torch.Tensor, biases: torch.Tensor, group: int | None = None) -> torch.Tensor:
    """(N, K) fp32 values s*q + b. ``families/qwen3_5/cuda/qmm.py:147-156`` (group 64) and
    ``families/qwen4_exp/cuda/qmm.py:100-109`` (group 32)."""

    q = unpack_nibbles(words).float()
    k = q.shape[1]
    group = group or k // scales.shape[1]
    s = scales.float().repeat_interleave(group, dim=1)
    b = biases.float().repeat_interleave(group, dim=1)
    return q * s + b


def qmm(x: torch.Tensor, words, scales, biases, group: int | None = None) -> torch.Tensor:
    """bf16( x.float() @ dequantize(W).T ): the fp32 reference projection (``reference.py:19-23``)."""

    return (x.float() @ dequantize(words, scales, biases, group).T).to(BF16)


def group_sums(x: torch.Tensor, group: int = 64) -> torch.Tensor:
    """fp32 sum of each input group (``qmm.py:49-59``)."""

    m, k = x.shape
    return x.float().reshape(m, k // group, group).sum(-1)


def qmm_ordered(x: torch.Tensor, words, scales, biases, group: int | None = None, f32: bool = False) -> torch.Tensor:
    """The lane form: y = sum over groups, in order, of s*(x_g . q_g) + b*xs_g, fp32, one rounding
    (``qmm.py:1-17,62-93``; Metal ``lane_qmm.py:9-20``). Used for the timed CPU baseline too."""

    q = unpack_nibbles(words).float()
    m, k = x.shape
    n = q.shape[0]
    group = group or k // scales.shape[1]
    kg = k // group
    xf = x.float().reshape(m, kg, group)
    xs = xf.sum(-1)
    qg = q.reshape(n, kg, group)
    s, b = scales.float(), biases.float()
    acc = torch.zeros((m, n), dtype=torch.float32)
    for g in range(kg):
        p = xf[:, g] @ qg[:, g].T
        acc = acc + p * s[:, g][None, :] + xs[:, g][:, None] * b[:, g][None, :]
    return acc if f32 else acc.to(BF16)


# ------------------------------------------------------------------------------------------------
# mixture-of-experts block (``families/qwen4_exp/cuda/moe.py``, ``qmm.py:421-602``, ``glue.py:85-91``)
# ------------------------------------------------------------------------------------------------

def moe_router(x: torch.Tensor, router_rows: torch.Tensor) -> torch.Tensor:
    """fp32 logits = bf16 x . bf16 rows (``moe.py:25-41``)."""

    return x.float() @ router_rows.float().T


def moe_select(logits: torch.Tensor, experts: int, top_k: int, shared: bool):
    """Per row: the top_k routed experts by (logit descending, id ascending), weights
    bf16(exp(l_k - l_0) / sum) with the sum in slot order, then the shared expert (id ``experts``) with
    weight bf16(sigmoid(bf16(gate logit))) (``moe.py:64-97``). Returns (pick int32, wts fp32)."""

    rows = logits.shape[0]
    slots = top_k + (1 if shared else 0)
    pick = torch.zeros((rows, slots), dtype=torch.int32)
    wts = torch.zeros((rows, slots), dtype=torch.float32)
    for r in range(rows):
        v = logits[r, :experts].clone()
        chosen, exs = [], []
        top = v.max()
        for _ in range(top_k):
            m = v.max()
            idx = int((v == m).nonzero()[0])
            chosen.append(idx)
            exs.append(torch.exp(m - top))
            v[idx] = float("-inf")
        total = torch.zeros((), dtype=torch.float32)
        for e in exs:
            total = total + e
        for k in range(top_k):
            pick[r, k] = chosen[k]
            wts[r, k] = (exs[k] / total).to(BF16).float()
        if shared:
            sg = logits[r, experts].to(BF16).float()
            pick[r, top_k] = experts
            wts[r, top_k] = (1.0 / (1.0 + torch.exp(-sg))).to(BF16).float()
    return pick, wts


def moe_experts(x: torch.Tensor, pick: torch.Tensor, wts: torch.Tensor, gates, ups, downs, group: int = 32) -> torch.Tensor:
    """Every (row, expert) pair alone: act = bf16(silu(bf16 gate) * bf16 up), y = fp32 down(act); a row's
    result is bf16(sum_k w_k y_k) in slot order (``qmm.py:517-526``, ``glue.py:85-91``)."""

    rows, slots = pick.shape
    dq = {}
    out = torch.zeros((rows, x.shape[1]), dtype=torch.float32)
    for r in range(rows):
        acc = torch.zeros(x.shape[1], dtype=torch.float32)
        for k in range(slots):
            e = int(pick[r, k])
            if e not in dq:
                dq[e] = tuple(dequantize(q.words, q.scales, q.biases, group) for q in (gates[e], ups[e], downs[e]))
            wg, wu, wd = dq[e]
            xr = x[r:r + 1].float()
            act = swiglu((xr @ wg.T).to(BF16), (xr @ wu.T).to(BF16))
            acc = acc + wts[r, k] * (act.float() @ wd.T)[0]
        out[r] = acc
    return out.to(BF16)


# ------------------------------------------------------------------------------------------------
# glue (``families/qwen3_5/cuda/glue.py``; fp32 forms as in ``reference.py``)
# ------------------------------------------------------------------------------------------------

def rms(x: torch.Tensor, w: torch.Tensor | None, eps: float) -> torch.Tensor:
    """``reference.py:26-29``."""

    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return y * w.float() if w is not None else y


def add_rmsnorm(x: torch.Tensor, r: torch.Tensor | None, w: torch.Tensor, eps: float):
    """h = bf16(x + r); y = bf16(rmsnorm(h) * w); xs = y's group sums (``glue.py:15-45``)."""

    h = x if r is None else (x.float() + r.float()).to(BF16)
    y = rms(h, w, eps).to(BF16)
    return h, y


def embed(ids: torch.Tensor, words, scales, biases, group: int = 64) -> torch.Tensor:
    """Dequantise one 4-bit row per token, bf16(q*s + b) (``glue.py:229-246``; ``reference.py:137-140``)."""

    i = ids.long()
    return dequantize(words[i], scales[i], biases[i], group).to(BF16)


def conv_silu(qkv: torch.Tensor, conv_state: torch.Tensor, conv_w: torch.Tensor) -> torch.Tensor:
    """Depthwise causal conv (taps = conv_w.shape[1]) over [conv_state; qkv], SiLU, rounded to bf16
    (``reference.py:75-79``). qkv (T, C) bf16, conv_state (taps-1, C), conv_w (C, taps)."""

    t = qkv.shape[0]
    taps = conv_w.shape[1]
    inp = torch.cat([conv_state, qkv], 0).float()
    w = conv_w.float()
    conv = sum(inp[j:j + t] * w[:, j] for j in range(taps))
    return torch.nn.functional.silu(conv).to(BF16)


def gdn_pre(qkv, conv_state, conv_w, a, b, a_log, dt_bias, *, kh: int, vh: int, dk: int, dv: int):
    """conv + SiLU, q/k RMS-normalised and scaled (q * 1/dk, k * dk^-1/2), g, beta
    (``reference.py:75-87``; ``glue.py:48-105``). Returns q,k (T,kh,dk) bf16, v (T,vh,dv) bf16, g, beta (T,vh) fp32."""

    t = qkv.shape[0]
    conv = conv_silu(qkv, conv_state, conv_w).float()
    kd = kh * dk
    q = conv[:, :kd].reshape(t, kh, dk)
    k = conv[:, kd:2 * kd].reshape(t, kh, dk)
    v = conv[:, 2 * kd:].reshape(t, vh, dv)
    q = (rms(q, None, 1e-6) * (1.0 / dk)).to(BF16)
    k = (rms(k, None, 1e-6) * (dk ** -0.5)).to(BF16)
    beta = torch.sigmoid(b.float())
    g = torch.exp(-torch.exp(a_log.float()) * torch.nn.functional.softplus(a.float() + dt_bias.float()))
    return q, k, v.to(BF16), g, beta


def gdn_recurrence(q, k, v, g, beta, state):
    """The gated delta rule, rows in order (``reference.py:88-101``; ``gdn_tree.cu:58-86``).

    q,k (T,kh,dk) bf16; v (T,vh,dv) bf16; g,beta (T,vh) fp32; state (vh,dv,dk) fp32.
    Returns y (T,vh,dv) bf16 and the state after the last row (fp32)."""

    t, kh, dk = q.shape
    vh = v.shape[1]
    rep = vh // kh
    s = state.float().clone()
    qf, kf, vf = q.float(), k.float(), v.float()
    ys = []
    for i in range(t):
        qt = qf[i].repeat_interleave(rep, 0)
        kt = kf[i].repeat_interleave(rep, 0)
        s = s * g[i][:, None, None]
        mem = (s * kt[:, None, :]).sum(-1)
        delta = (vf[i] - mem) * beta[i][:, None]
        s = s + kt[:, None, :] * delta[:, :, None]
        ys.append((s * qt[:, None, :]).sum(-1))
    return torch.stack(ys).to(BF16), s


def gated_norm(y, z, w, eps: float) -> torch.Tensor:
    """bf16( silu(z) * rmsnorm(y) * w ) per head, flattened (``reference.py:101-103``; ``glue.py:108-130``)."""

    t = y.shape[0]
    yn = rms(y, w, eps)
    return (torch.nn.functional.silu(z.float().reshape(y.shape)) * yn).to(BF16).reshape(t, -1)


def swiglu(gate, up) -> torch.Tensor:
    """bf16( silu(gate) * up ) (``reference.py:149``; ``glue.py:133-154``)."""

    return (torch.nn.functional.silu(gate.float()) * up.float()).to(BF16)


def rope(x: torch.Tensor, pos: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
    """Rotate-half over the first 2*len(inv_freq) dims; x (T,H,D) fp32 (``reference.py:32-42``)."""

    half = inv_freq.numel()
    ang = pos.float()[:, None] * inv_freq.float()[None, :]
    cos, sin = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    x1, x2 = x[..., :half], x[..., half:2 * half]
    out = x.clone()
    out[..., :half] = x1 * cos - x2 * sin
    out[..., half:2 * half] = x2 * cos + x1 * sin
    return out


def attn_prep(qg, k, q_norm, k_norm, pos, inv_freq, eps, *, heads, kv_heads, head_dim):
    """Per-head RMSNorm (bf16) then partial RoPE (bf16) of q (from [q_h | gate_h] rows) and k
    (``reference.py:109-116``; ``glue.py:157-203``)."""

    t = qg.shape[0]
    q = qg.reshape(t, heads, 2 * head_dim)[..., :head_dim]
    kk = k.reshape(t, kv_heads, head_dim)
    q = rope(rms(q, q_norm, eps).to(BF16).float(), pos, inv_freq).to(BF16)
    kk = rope(rms(kk, k_norm, eps).to(BF16).float(), pos, inv_freq).to(BF16)
    return q, kk


def attention(q, k_all, v_all, n_keys: torch.Tensor, scale: float) -> torch.Tensor:
    """Causal GQA for T query rows: row t attends to keys [0, n_keys[t]) of k_all/v_all (L,HK,D)
    (``reference.py:117-126``). q (T,H,D) bf16 -> (T,H,D) bf16."""

    t, h, d = q.shape
    l, hk, _ = k_all.shape
    rep = h // hk
    kf = k_all.float().repeat_interleave(rep, 1)
    vf = v_all.float().repeat_interleave(rep, 1)
    s = torch.einsum("thd,lhd->htl", q.float(), kf) * scale
    mask = torch.arange(l)[None, :] >= n_keys.long()[:, None]
    s = s.masked_fill(mask[None], float("-inf"))
    return torch.einsum("htl,lhd->thd", torch.softmax(s, -1), vf).to(BF16)


def gate_mul(o, qg, *, heads, head_dim) -> torch.Tensor:
    """bf16( o * sigmoid(gate) ), gate = second half of each head's [q | gate] row
    (``reference.py:127``; ``glue.py:206-226``)."""

    t = o.shape[0]
    gate = qg.reshape(t, heads, 2 * head_dim)[..., head_dim:]
    return (o.float() * torch.sigmoid(gate.float())).to(BF16).reshape(t, -1)


# ------------------------------------------------------------------------------------------------
# the dense hybrid model (``families/qwen3_5/cuda/reference.py:45-157``, ``weights.py``)
# ------------------------------------------------------------------------------------------------

@dataclass
class Config:
    """``weights.py:38-59`` (the fields the forward uses)."""

    hidden: int
    intermediate: int
    layers: int
    heads: int
    kv_heads: int
    head_dim: int
    vocab: int
    k_heads: int
    v_heads: int
    dk: int
    dv: int
    conv_kernel: int = 4
    interval: int = 4
    eps: float = 1e-6
    rope_dims: int = 0
    rope_theta: float = 1e7
    group: int = 64
    experts: int = 0                  # mixture-of-experts MLP when > 0 (``families/qwen4_exp/model.py``)
    top_k: int = 0
    moe_intermediate: int = 0
    shared_expert: bool = True

    def __post_init__(self):
        if not self.rope_dims:
            self.rope_dims = self.head_dim // 4

    def is_linear(self, layer: int) -> bool:
        return (layer + 1) % self.interval != 0

    def inv_freq(self) -> torch.Tensor:
        """``weights.py:188-190``."""

        half = self.rope_dims // 2
        return (self.rope_theta ** (-torch.arange(0, half, dtype=torch.float64) / half)).to(torch.float32)


@dataclass
class Q4:
    words: torch.Tensor
    scales: torch.Tensor
    biases: torch.Tensor


def random_q4(gen: torch.Generator, n: int, k: int, group: int = 64, spread: float = 1.0) -> Q4:
    """Random packed words with centred scales so activations stay O(1) through many layers
    (``tests/cuda/test_flashnext_forward.py:35-40``): scales = (U(0,1)/8 + 1/64) * spread/sqrt(k),
    biases = -7.5 * scales."""

    words = torch.randint(-2 ** 31, 2 ** 31 - 1, (n, k // 8), generator=gen, dtype=torch.int64).to(torch.int32)
    s = (torch.rand((n, k // group), generator=gen) / 8 + 1 / 64) * (spread * 4.0 / k ** 0.5)
    scales = s.to(BF16)
    biases = (-7.5 * scales.float()).to(BF16)
    return Q4(words, scales, biases)


def random_model(cfg: Config, seed: int) -> dict:
    """Random weights of the dense hybrid architecture, as plain tensors in a dict."""

    gen = torch.Generator().manual_seed(seed)
    g = cfg.group

    def norm(n):
        return (1 + 0.05 * torch.randn(n, generator=gen)).to(BF16)

    kd, vd = cfg.k_heads * cfg.dk, cfg.v_heads * cfg.dv
    layers = []
    for i in range(cfg.layers):
        layer = {"linear": cfg.is_linear(i), "input_norm": norm(cfg.hidden), "post_norm": norm(cfg.hidden)}
        if cfg.experts:
            ne = cfg.experts + (1 if cfg.shared_expert else 0)
            layer["router"] = (0.05 * torch.randn((ne, cfg.hidden), generator=gen)).to(BF16)
            layer["experts"] = {"gate": [random_q4(gen, cfg.moe_intermediate, cfg.hidden, g) for _ in range(ne)],
                                "up": [random_q4(gen, cfg.moe_intermediate, cfg.hidden, g) for _ in range(ne)],
                                "down": [random_q4(gen, cfg.hidden, cfg.moe_intermediate, g) for _ in range(ne)]}
        else:
            layer.update(gate=random_q4(gen, cfg.intermediate, cfg.hidden, g), up=random_q4(gen, cfg.intermediate, cfg.hidden, g),
                         down=random_q4(gen, cfg.hidden, cfg.intermediate, g))
        if layer["linear"]:
            layer.update(qkv=random_q4(gen, 2 * kd + vd, cfg.hidden, g), z=random_q4(gen, vd, cfg.hidden, g),
                         b=random_q4(gen, cfg.v_heads, cfg.hidden, g), a=random_q4(gen, cfg.v_heads, cfg.hidden, g),
                         out=random_q4(gen, cfg.hidden, vd, g),
                         conv=(0.3 * torch.randn((2 * kd + vd, cfg.conv_kernel), generator=gen)).to(BF16),
                         A_log=0.5 * torch.randn(cfg.v_heads, generator=gen), dt_bias=0.5 * torch.randn(cfg.v_heads, generator=gen),
                         norm=norm(cfg.dv))
        else:
            layer.update(q=random_q4(gen, cfg.heads * cfg.head_dim * 2, cfg.hidden, g),
                         k=random_q4(gen, cfg.kv_heads * cfg.head_dim, cfg.hidden, g),
                         v=random_q4(gen, cfg.kv_heads * cfg.head_dim, cfg.hidden, g),
                         o=random_q4(gen, cfg.hidden, cfg.heads * cfg.head_dim, g),
                         q_norm=norm(cfg.head_dim), k_norm=norm(cfg.head_dim))
        layers.append(layer)
    embed_w = random_q4(gen, cfg.vocab, cfg.hidden, g, spread=2.0)
    return {"config": cfg, "layers": layers, "embed": embed_w, "norm": norm(cfg.hidden),
            "head": random_q4(gen, cfg.vocab, cfg.hidden, g), "inv_freq": cfg.inv_freq()}


@dataclass
class State:
    """One sequence's committed state (``reference.py:45-65``)."""

    pos: int = 0
    kv: list = field(default_factory=list)
    conv: list = field(default_factory=list)
    rec: list = field(default_factory=list)

    @classmethod
    def fresh(cls, model: dict) -> "State":
        c = model["config"]
        st = cls()
        for layer in model["layers"]:
            if layer["linear"]:
                cd = 2 * c.k_heads * c.dk + c.v_heads * c.dv
                st.conv.append(torch.zeros((c.conv_kernel - 1, cd), dtype=BF16))
                st.rec.append(torch.zeros((c.v_heads, c.dv, c.dk), dtype=torch.float32))
                st.kv.append(None)
            else:
                st.conv.append(None)
                st.rec.append(None)
                st.kv.append((torch.zeros((0, c.kv_heads, c.head_dim), dtype=BF16),
                              torch.zeros((0, c.kv_heads, c.head_dim), dtype=BF16)))
        return st


def _lin(x, w: Q4, group):
    return qmm(x, w.words, w.scales, w.biases, group)


def forward(model: dict, tokens: torch.Tensor, st: State, *, head: bool = True) -> torch.Tensor:
    """Logits (T, V) fp32 for ``tokens`` continuing ``st`` (which is advanced): ``reference.py:131-157``."""

    c = model["config"]
    g = c.group
    t = tokens.shape[0]
    e = model["embed"]
    x = embed(tokens, e.words, e.scales, e.biases, g)
    pos = torch.arange(st.pos, st.pos + t)
    for i, layer in enumerate(model["layers"]):
        _, h = add_rmsnorm(x, None, layer["input_norm"], c.eps)
        if layer["linear"]:
            qkv = _lin(h, layer["qkv"], g)
            z = _lin(h, layer["z"], g)
            b = _lin(h, layer["b"], g)
            a = _lin(h, layer["a"], g)
            q, k, v, gg, beta = gdn_pre(qkv, st.conv[i], layer["conv"], a, b, layer["A_log"], layer["dt_bias"],
                                        kh=c.k_heads, vh=c.v_heads, dk=c.dk, dv=c.dv)
            st.conv[i] = torch.cat([st.conv[i], qkv], 0)[-(c.conv_kernel - 1):].clone()
            y, st.rec[i] = gdn_recurrence(q, k, v, gg, beta, st.rec[i])
            out = gated_norm(y, z.reshape(t, c.v_heads, c.dv), layer["norm"], c.eps)
            r = _lin(out, layer["out"], g)
        else:
            qg = _lin(h, layer["q"], g)
            kk = _lin(h, layer["k"], g)
            vv = _lin(h, layer["v"], g).reshape(t, c.kv_heads, c.head_dim)
            q, kk = attn_prep(qg, kk, layer["q_norm"], layer["k_norm"], pos, model["inv_freq"], c.eps,
                              heads=c.heads, kv_heads=c.kv_heads, head_dim=c.head_dim)
            k0, v0 = st.kv[i]
            k_all, v_all = torch.cat([k0, kk]), torch.cat([v0, vv])
            st.kv[i] = (k_all, v_all)
            o = attention(q, k_all, v_all, pos + 1, c.head_dim ** -0.5)
            r = _lin(gate_mul(o, qg, heads=c.heads, head_dim=c.head_dim), layer["o"], g)
        x = (x.float() + r.float()).to(BF16)
        _, h = add_rmsnorm(x, None, layer["post_norm"], c.eps)
        if "router" in layer:
            e = layer["experts"]
            pick, wts = moe_select(moe_router(h, layer["router"]), c.experts, c.top_k, c.shared_expert)
            x = (x.float() + moe_experts(h, pick, wts, e["gate"], e["up"], e["down"], g).float()).to(BF16)
            continue
        act = swiglu(_lin(h, layer["gate"], g), _lin(h, layer["up"], g))
        x = (x.float() + _lin(act, layer["down"], g).float()).to(BF16)
    st.pos += t
    _, h = add_rmsnorm(x, None, model["norm"], c.eps)
    if not head:
        return h
    hd = model["head"]
    return h.float() @ dequantize(hd.words, hd.scales, hd.biases, g).T


# ------------------------------------------------------------------------------------------------
# exact top-k and keyed sampling (``engine/topk.py``, ``engine/exact_sampling.py``)
# ------------------------------------------------------------------------------------------------

def topk_rows(x: np.ndarray, k: int):
    """Each row's k largest by (value desc, id asc): ``tests/test_topk.py:11-13`` states the rule as
    ``np.lexsort((ids, -row))[:k]``. Returns (idx int32 (R,k), val fp32 (R,k))."""

    x = np.asarray(x, dtype=np.float32)
    ids = np.arange(x.shape[1])
    idx = np.stack([np.lexsort((ids, -row))[:k] for row in x]).astype(np.int32)
    return idx, np.take_along_axis(x, idx.astype(np.int64), axis=1)


@dataclass(frozen=True)
class Sampling:
    """``exact_sampling.py:34-39``."""

    seed: int
    temperature: float = 1.0
    top_k: int = 20
    top_p: float = 0.95


def _mix(x: np.ndarray) -> np.ndarray:
    """splitmix64 finaliser (``exact_sampling.py:49-54``)."""

    x = x ^ (x >> np.uint64(30))
    x = x * np.uint64(0xBF58476D1CE4E5B9)
    x = x ^ (x >> np.uint64(27))
    x = x * np.uint64(0x94D049BB133111EB)
    return x ^ (x >> np.uint64(31))


def uniform_rows(seed: int, positions: np.ndarray, ids: np.ndarray) -> np.ndarray:
    """Uniform (0,1) doubles from a hash of (seed, position, token id) (``exact_sampling.py:57-74``)."""

    with np.errstate(over="ignore"):
        x = _mix(np.uint64(seed & 0xFFFFFFFFFFFFFFFF) + np.uint64(0x9E3779B97F4A7C15))
        x = _mix(x ^ (np.asarray(positions).astype(np.uint64)[:, None] * np.uint64(0xD1B54A32D192ED03)))
        x = _mix(x ^ ids.astype(np.uint64))
    return (x >> np.uint64(11)).astype(np.float64) * 2.0 ** -53 + 2.0 ** -54


def choose_rows(values: np.ndarray, ids: np.ndarray, positions, s: Sampling) -> list[int]:
    """Keyed Gumbel-max over the top-k/top-p candidates of each row (``exact_sampling.py:93-109``)."""

    rows, width = ids.shape
    order = np.lexsort((ids, -values), axis=-1)
    k = max(1, min(int(s.top_k) if s.top_k else width, width))
    ids = np.take_along_axis(ids, order, axis=-1)[:, :k]
    scaled = np.take_along_axis(values, order, axis=-1)[:, :k].astype(np.float64) / max(float(s.temperature), 1e-6)
    score = scaled - np.log(-np.log(uniform_rows(s.seed, np.asarray(positions), ids)))
    if 0.0 < s.top_p < 1.0:
        probs = np.exp(scaled - scaled.max(axis=-1, keepdims=True))
        probs /= probs.sum(axis=-1, keepdims=True)
        keep = (np.cumsum(probs, axis=-1) < s.top_p).sum(axis=-1) + 1
        score[np.arange(k)[None, :] >= keep[:, None]] = -np.inf
    return [int(t) for t in ids[np.arange(rows), np.argmax(score, axis=-1)]]


def sample_rows(logits: np.ndarray, positions, s: Sampling | None) -> list[int]:
    """Greedy = first maximum; else candidates = the whole row (``families/qwen3_5/cuda/sampling.py:13-34``
    reads top_k + 8 from the GPU, which selects the same set)."""

    logits = np.asarray(logits, dtype=np.float32)
    if s is None or s.temperature <= 0:
        return [int(i) for i in logits.argmax(-1)]
    ids = np.broadcast_to(np.arange(logits.shape[1], dtype=np.int64), logits.shape)
    return choose_rows(logits, ids, positions, s)
