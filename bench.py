"""Lane-verify throughput of the 27B-class 4-bit dense hybrid decoder on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--seqs S] [--ctx C] [--width 8] [--impl ours|reference]

A step is one verify forward (all 64 layers + head + token choice) over S sequences x W drafted rows
with C committed tokens of context each; weights are random 4-bit group-64 of the 27B-class
architecture, prompts random token ids, the context built by real prefill through
the same kernels. Prints ONE JSON line (rank 0). With N > 1 the model is tensor-parallel over N ranks
(launch under torchrun). ``--impl reference`` times the CPU restatement of the reference arithmetic
(``oracle/``) on the host cores for the same workload, on a bounded sample.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.samples, self.proc, self.index = [], None, index

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append([x.strip() for x in line.split(",")])

    def __exit__(self, *exc):
        if self.proc:
            time.sleep(0.15)
            self.proc.terminate()
            self.thread.join(timeout=2)

    def summary(self):
        sm = sorted(int(s[0]) for s in self.samples if s and s[0].isdigit())
        reasons = set()
        for s in self.samples:
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), s[2:6]):
                if v == "Active":
                    reasons.add(name)
        mx = max((int(s[1]) for s in self.samples if len(s) > 1 and s[1].isdigit()), default=None)
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons), "samples": len(sm)}


def cpu_reference(args, rows: int):
    """The reference arithmetic on the host cores (oracle port): one GDN layer and one attention layer of
    the 27B-class shapes over the step's rows, scaled to 48 + 16 layers + head by weight count."""

    import torch

    from oracle import lane_oracle as O

    torch.set_num_threads(os.cpu_count() or 1)
    cfg = O.Config(hidden=5120, intermediate=17408, layers=4, heads=24, kv_heads=4, head_dim=256, vocab=256, k_heads=16,
                   v_heads=32, dk=128, dv=128, rope_dims=64)
    gen = torch.Generator().manual_seed(0)
    c = cfg
    kd, vd = c.k_heads * c.dk, c.v_heads * c.dv
    x = torch.randn((rows, c.hidden), generator=gen).to(torch.bfloat16)
    norm = torch.ones(c.hidden, dtype=torch.bfloat16)

    def lin(inp, n, k):
        q = O.random_q4(gen, n, k, 64)
        return O.qmm(inp, q.words, q.scales, q.biases, 64)

    def mlp(h):
        act = O.swiglu(lin(h, c.intermediate, c.hidden), lin(h, c.intermediate, c.hidden))
        return lin(act, c.hidden, c.intermediate)

    t0 = time.perf_counter()
    _, h = O.add_rmsnorm(x, None, norm, c.eps)
    qkv, z, b, a = lin(h, 2 * kd + vd, c.hidden), lin(h, vd, c.hidden), lin(h, c.v_heads, c.hidden), lin(h, c.v_heads, c.hidden)
    q, k, v, g, beta = O.gdn_pre(qkv, torch.zeros((3, 2 * kd + vd), dtype=torch.bfloat16), torch.ones((2 * kd + vd, 4), dtype=torch.bfloat16),
                                 a, b, torch.zeros(c.v_heads), torch.zeros(c.v_heads), kh=c.k_heads, vh=c.v_heads, dk=128, dv=128)
    per_seq = args.width
    ys = []
    for s0 in range(0, rows, per_seq):
        y, _ = O.gdn_recurrence(q[s0:s0 + per_seq], k[s0:s0 + per_seq], v[s0:s0 + per_seq], g[s0:s0 + per_seq], beta[s0:s0 + per_seq],
                                torch.zeros((c.v_heads, 128, 128)))
        ys.append(y)
    out = O.gated_norm(torch.cat(ys), z.reshape(rows, c.v_heads, 128), torch.ones(128, dtype=torch.bfloat16), c.eps)
    x1 = (x.float() + lin(out, c.hidden, vd).float()).to(torch.bfloat16)
    _, h = O.add_rmsnorm(x1, None, norm, c.eps)
    x1 = (x1.float() + mlp(h).float()).to(torch.bfloat16)
    t_gdn = time.perf_counter() - t0

    t0 = time.perf_counter()
    _, h = O.add_rmsnorm(x1, None, norm, c.eps)
    qg, kk, vv = lin(h, c.heads * 2 * c.head_dim, c.hidden), lin(h, c.kv_heads * c.head_dim, c.hidden), lin(h, c.kv_heads * c.head_dim, c.hidden)
    pos = torch.arange(rows) % per_seq + 256
    qh, kh_ = O.attn_prep(qg, kk, torch.ones(c.head_dim, dtype=torch.bfloat16), torch.ones(c.head_dim, dtype=torch.bfloat16), pos,
                          cfg.inv_freq(), c.eps, heads=c.heads, kv_heads=c.kv_heads, head_dim=c.head_dim)
    ctx = 256                                                   # a short context: the sample is bounded by the projections
    kc = torch.randn((ctx + per_seq, c.kv_heads, c.head_dim), generator=gen).to(torch.bfloat16)
    os_ = []
    for s0 in range(0, rows, per_seq):
        os_.append(O.attention(qh[s0:s0 + per_seq], kc, kc, torch.arange(per_seq) + ctx + 1, c.head_dim ** -0.5))
    o = O.gate_mul(torch.cat(os_), qg, heads=c.heads, head_dim=c.head_dim)
    x2 = (x1.float() + lin(o, c.hidden, c.heads * c.head_dim).float()).to(torch.bfloat16)
    _, h = O.add_rmsnorm(x2, None, norm, c.eps)
    x2 = (x2.float() + mlp(h).float()).to(torch.bfloat16)
    t_att = time.perf_counter() - t0
    layer_params = 3 * c.intermediate * c.hidden + (2 * kd + 2 * vd + 2 * c.v_heads + vd) * c.hidden
    t_head = t_gdn * (248320 * c.hidden) / layer_params
    total = 48 * t_gdn + 16 * t_att + t_head
    return {"value": rows / total, "unit": "rows/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"1 GDN layer ({t_gdn:.1f} s) + 1 attention layer at 256 keys ({t_att:.1f} s) of the 27B-class shapes over "
                      f"{rows} rows, scaled to 48 + 16 layers + head by weight count"}


def reference_gpu(args, rows: int):
    """The reference's own CUDA lane path (its Triton kernels and JIT-built GDN kernel, copied unmodified into
    ``oracle/_ref`` by ``oracle/make_ref.py``) timed on this GPU: the tiled lane matmul at the headline shape, and one
    verify window of the 64-layer 27B-class model through its ``forward.tree_forward`` as its engine calls it (eager).
    Random weights in its stored layout, regrouped by its own ``qmm_fast.prepare``; context set directly (random
    K/V rows, zero recurrent state). Returns {"unavailable": why} where that path cannot run."""

    ref_dir = ROOT / "oracle" / "_ref"
    if not (ref_dir / "tensorfold").is_dir():
        return {"unavailable": "oracle/_ref is absent (made by oracle/make_ref.py where the reference checkout exists)"}
    try:
        import torch

        if not torch.cuda.is_available():
            return {"unavailable": "no CUDA device"}
        sys.path.insert(0, str(ref_dir))
        from tensorfold.families.qwen3_5.cuda import forward as RF, qmm_fast
        from tensorfold.families.qwen3_5.cuda.weights import Attention, Config, GDN, Layer, QLinear, Weights
    except Exception as exc:
        return {"unavailable": f"the reference's CUDA path does not import here: {type(exc).__name__}: {exc}"}
    try:
        dev = torch.device("cuda", 0)
        gen = torch.Generator(device=dev).manual_seed(1)
        bf = torch.bfloat16

        def ql(n, k):
            words = torch.randint(-2 ** 31, 2 ** 31 - 1, (n, k // 8), generator=gen, dtype=torch.int64, device=dev).to(torch.int32)
            sc = ((torch.rand((n, k // 64), generator=gen, device=dev) / 8 + 1 / 64) * (4.0 / k ** 0.5)).to(bf)
            return QLinear(words, sc, (-7.5 * sc.float()).to(bf))

        def time_us(fn, n):
            for _ in range(3):
                fn(0)
            torch.cuda.synchronize(dev)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for i in range(n):
                fn(i)
            e1.record()
            torch.cuda.synchronize(dev)
            return 1000.0 * e0.elapsed_time(e1) / n

        out = {"kind": "the reference's Triton lane kernels on this GPU, called through its own Python API"}
        # the headline matmul: four weight copies rotated through so every launch streams from HBM
        n, k = 17408, 5120
        x = torch.randn((rows, k), device=dev, generator=gen).to(bf)
        copies = [qmm_fast.tile(ql(n, k)) for _ in range(4)]
        eager = time_us(lambda i: qmm_fast.matmul(x, copies[i % 4]), 40)
        out["qmm_17408x5120"] = {"rows": rows, "eager_us_per_launch": eager}
        try:
            side, graph = torch.cuda.Stream(dev), torch.cuda.CUDAGraph()
            with torch.cuda.stream(side):
                qmm_fast.matmul(x, copies[0])
                side.synchronize()
                with torch.cuda.graph(graph, stream=side):
                    for q in copies:
                        qmm_fast.matmul(x, q)
            torch.cuda.synchronize(dev)
            out["qmm_17408x5120"]["graph_us_per_launch"] = time_us(lambda i: graph.replay(), 10) / 4
        except Exception as exc:
            out["qmm_17408x5120"]["graph_us_per_launch"] = None
            out["qmm_17408x5120"]["graph_note"] = f"not capturable: {type(exc).__name__}"
            torch.cuda.synchronize(dev)
        alg = n * k // 2 + n * (k // 64) * 4 + rows * k * 2 + rows * n * 2
        best = out["qmm_17408x5120"].get("graph_us_per_launch") or eager
        out["qmm_17408x5120"]["achieved_gbs"] = alg / best / 1e3
        del copies
        # the whole verify window
        c = dict(hidden=5120, intermediate=17408, layers=args.layers, heads=24, kv_heads=4, head_dim=256, vocab=248320, k_heads=16,
                 v_heads=32, dk=128, dv=128)
        cfg = Config(**c, conv_kernel=4, interval=4, eps=1e-6, rope_dims=64, rope_theta=1e7, eos=(0,))
        kd, vd, h = 16 * 128, 32 * 128, 5120

        def norm(m):
            return (1 + 0.05 * torch.randn(m, generator=gen, device=dev)).to(bf)
        layers = []
        for i in range(cfg.layers):
            if cfg.is_linear(i):
                gdn = GDN(ql(2 * kd + vd, h), ql(vd, h), ql(32, h), ql(32, h), ql(h, vd),
                          (0.3 * torch.randn((2 * kd + vd, 4), generator=gen, device=dev)).to(bf),
                          0.5 * torch.randn(32, generator=gen, device=dev), 0.5 * torch.randn(32, generator=gen, device=dev), norm(128))
                layers.append(Layer(True, norm(h), norm(h), gdn, None, ql(17408, h), ql(17408, h), ql(h, 17408)))
            else:
                att = Attention(ql(24 * 512, h), ql(4 * 256, h), ql(4 * 256, h), ql(h, 24 * 256), norm(256), norm(256))
                layers.append(Layer(False, norm(h), norm(h), None, att, ql(17408, h), ql(17408, h), ql(h, 17408)))
        half = 32
        inv_freq = (1e7 ** (-torch.arange(0, half, dtype=torch.float64) / half)).to(torch.float32).to(dev)
        w = Weights(cfg, ql(cfg.vocab, h), layers, norm(h), ql(cfg.vocab, h), inv_freq)
        qmm_fast.prepare(w)
        st = RF.State(w)
        st.pos = args.ctx
        for i, layer in enumerate(w.layers):
            if not layer.linear:
                st.kv[i] = tuple(torch.randn((args.ctx + 64, 4, 256), device=dev, generator=gen).to(bf) for _ in range(2))
        width = args.width
        tokens = torch.randint(0, cfg.vocab, (width,), generator=gen, device=dev, dtype=torch.int32)
        parents = [-1] + list(range(width - 1))
        ms = time_us(lambda i: RF.tree_forward(w, tokens, parents, st), max(args.steps, 5)) / 1000.0
        out["forward"] = {"ms_per_window": ms, "rows_per_s": width / ms * 1000.0, "rows": width, "context": args.ctx, "layers": cfg.layers,
                          "note": "one sequence; eager launches, as the reference's engine issues them; synthetic context"}
        return out
    except Exception as exc:
        return {"unavailable": f"the reference's CUDA path failed here: {type(exc).__name__}: {str(exc)[:200]}"}
    finally:
        if str(ref_dir) in sys.path:
            sys.path.remove(str(ref_dir))


def only_qmm(args, dev):
    """The lane matmul alone: --copies weights of --shape rotated through so that every launch streams
    from HBM; CUDA-event time per launch, algorithmic bytes, fraction of the measured copy bandwidth."""

    import torch

    from tensorfold_b200 import _lib, lane_qmm, prefill_qmm, synthetic

    n, k = (int(v) for v in args.shape.split("x"))
    group, rows = 64, args.rows
    gen = torch.Generator(device=dev).manual_seed(3)
    xr = torch.randn((rows, k), device=dev, generator=gen).to(torch.bfloat16)
    if args.only == "prefill":
        def weight():
            words = torch.randint(-2 ** 31, 2 ** 31 - 1, (n, k // 8), generator=gen, dtype=torch.int64, device=dev).to(torch.int32)
            sc = ((torch.rand((n, k // group), generator=gen, device=dev) / 8 + 1 / 64) * (4.0 / k ** 0.5)).to(torch.bfloat16)
            return prefill_qmm.tile_weight(words, sc, (-7.5 * sc.float()).to(torch.bfloat16), group)
        ws = [weight() for _ in range(args.copies)]

        def run(q):
            return prefill_qmm.prefill_matmul(xr, q)        # packs the rows, then the tcgen05 matmul
    else:
        ws = [synthetic.random_q4(gen, n, k, group, dev) for _ in range(args.copies)]
        x = lane_qmm.pack_rows(xr, group)
        out = torch.empty((rows, n), dtype=torch.bfloat16, device=dev)

        def run(q):
            return lane_qmm.lane_matmul(x, q, out=out)
    for q in ws:
        run(q)
    torch.cuda.synchronize(dev)
    # eager: launches back to back from the host (includes launch gaps)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches = max(args.steps, 1) * args.copies
    e0.record()
    for i in range(launches):
        run(ws[i % args.copies])
    e1.record()
    torch.cuda.synchronize(dev)
    eager_us = 1000.0 * e0.elapsed_time(e1) / launches
    # graph: the same rotation captured once and replayed, as the forward issues it
    side = torch.cuda.Stream(dev)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        run(ws[0])
        side.synchronize()
        with torch.cuda.graph(graph, stream=side):
            for q in ws:
                run(q)
    torch.cuda.synchronize(dev)
    graph.replay()
    torch.cuda.synchronize(dev)
    reps = max(args.steps, 1)
    e0.record()
    for _ in range(reps):
        graph.replay()
    e1.record()
    torch.cuda.synchronize(dev)
    _lib.status(dev).raise_if_set()
    us = 1000.0 * e0.elapsed_time(e1) / (reps * args.copies)
    kg = k // group
    alg = n * k // 2 + n * kg * 4 + rows * k * 2 + rows * kg * 4 + rows * n * 2
    peak, kind = peaks()
    flops = 2.0 * rows * n * k
    print(json.dumps({"only": args.only, "tflops": flops / us / 1e6, "shape": [n, k], "rows": rows, "launches": reps * args.copies,
                      "us_per_launch": us, "eager_us_per_launch": eager_us,
                      "note": f"{args.copies} weight copies rotated through, captured in a CUDA graph and replayed; eager figure beside it",
                      "algorithmic_bytes": alg, "achieved_gbs": alg / us / 1e3, "frac": alg / us / 1e3 / peak, "peak_kind": kind}))


def only_timeline(args, dev):
    """Where a verify step's time goes around its matmuls: one captured step of --layers layers (1 sequence x
    --width rows, context set directly) with the lane matmul's timeline hook on (`tf_qmm_set_trace`: globaltimer
    stamps per CTA and launch). Per kind of projection, medians over the layers after the first: the time from the
    predecessor's memory being visible to the first stage in shared memory, the main loop, the K-segment finish and
    output (tail), and the gap until the next matmul may start (the glue kernels between them)."""

    import numpy as np
    import torch

    from tensorfold_b200 import _lib, forward as F, runner, synthetic

    cfg = F.Config(**dict(synthetic.DENSE_27B, layers=args.layers))
    w = synthetic.random_weights(cfg, seed=2, device=dev)
    st = F.State(w, 1, args.ctx + 2 * args.width, dev)
    run = runner.LaneRunner(w, st, [args.width], max_context=args.ctx + args.width)
    run.capture()
    st.lens = [args.ctx]
    run.refresh()
    run.tokens.copy_(torch.randint(0, cfg.vocab, (args.width,), device=dev, dtype=torch.int32))
    for _ in range(10):
        run.step_device()
    torch.cuda.synchronize(dev)
    slots, launches, workers = 16, 512, 148
    tr = torch.zeros(workers + launches * workers * slots, dtype=torch.int64, device=dev)
    lib = _lib.load()
    _lib.check(lib.tf_qmm_set_trace(tr.data_ptr()), "set_trace")
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    run.step_device()
    e1.record()
    torch.cuda.synchronize(dev)
    lib.tf_qmm_set_trace(None)
    n = 4 * args.layers + 1
    t = tr.cpu().numpy()[workers:].reshape(launches, workers, slots).astype(np.float64)

    def stat(launch, slot, f=np.median):
        col = t[launch, :, slot]
        col = col[col > 0]
        return float(f(col)) if len(col) else float("nan")
    kinds = ["in_proj", "out_proj", "gate_up", "down"]
    rows = {k: [] for k in kinds}
    for i in range(4, n - 1):                       # skip the first layer (cold) and the head
        wait, first, loop = stat(i, 2), stat(i, 3), stat(i, 4)
        ends = [v for v in (stat(i, 9, np.max), stat(i, 6, np.max)) if v == v]
        end = max(ends)
        rows[kinds[i % 4]].append((first - wait, loop - first, end - loop, stat(i + 1, 2) - end))
    out = {"only": "timeline", "layers": args.layers, "step_us_with_tracing": 1000.0 * e0.elapsed_time(e1), "unit": "us (medians)"}
    busy = gaps = 0.0
    for k in kinds:
        a = np.median(np.array(rows[k]), axis=0) / 1000.0
        out[k] = {"fill": round(a[0], 2), "main_loop": round(a[1], 2), "tail": round(a[2], 2), "gap_to_next_matmul": round(a[3], 2)}
        busy += a[0] + a[1] + a[2]
        gaps += a[3]
    out["per_layer"] = {"matmul_busy": round(busy, 2), "between_matmuls": round(gaps, 2)}
    print(json.dumps(out))


def only_gdn(args, dev):
    """The gated-DeltaNet lane step alone (conv1d + gates + recurrence + gated norm, one fused kernel per layer):
    --seqs sequences x --width rows, 16 QK heads, 32 V heads, head dim 128, fp32 state N(0, 0.1) per layer;
    --layers layers with their own state rotated through (32 sequences: 67 MB of state a layer), graph-replayed."""

    import torch

    from tensorfold_b200 import _lib, lane_gdn, lane_qmm

    seqs, w, nk, nv, layers = args.seqs, args.width, 16, 32, min(args.layers, 12)
    c = (2 * 16 + 32) * 128
    per = max(1, 128 // w)                       # sequences a launch: a packed buffer holds 128 rows
    groups = [(s0, min(per, seqs - s0)) for s0 in range(0, seqs, per)]
    gen = torch.Generator(device=dev).manual_seed(5)
    conv_w = (0.3 * torch.randn((c, 4), device=dev, generator=gen)).to(torch.bfloat16)
    a_log, dt = 0.5 * torch.randn(nv, device=dev, generator=gen), 0.5 * torch.randn(nv, device=dev, generator=gen)
    nw = torch.ones(128, device=dev, dtype=torch.bfloat16)
    conv_state = torch.randn((layers, seqs, 3, c), device=dev, generator=gen).to(torch.bfloat16)
    state = 0.1 * torch.randn((layers, seqs, nv, 128, 128), device=dev, generator=gen)
    parts = []
    for s0, n in groups:
        r = n * w
        proj = torch.randn((r, c + nv * 128 + 2 * nv), device=dev, generator=gen).to(torch.bfloat16)
        rec = (torch.empty((r, nk, 128), device=dev, dtype=torch.bfloat16), torch.empty((r, nv, 128), device=dev, dtype=torch.bfloat16),
               torch.empty((r, nv), device=dev), torch.empty((r, nv), device=dev))
        parts.append((s0, n, proj, rec, torch.arange(0, r + 1, w, dtype=torch.int32, device=dev), lane_qmm.new_packed(r, nv * 128, 64, dev)))

    def layer(i):
        for s0, n, proj, rec, starts, out in parts:
            qkv, z = proj[:, :c], proj[:, c:c + nv * 128]
            bb, aa = proj[:, c + nv * 128:c + nv * 128 + nv], proj[:, c + nv * 128 + nv:]
            lane_gdn.gdn_mixer(qkv, z, aa, bb, conv_state[i, s0:s0 + n], conv_w, a_log, dt, nw, state[i, s0:s0 + n], starts, nk=nk, nv=nv,
                               eps=1e-6, group=64, record=rec, out=out)
    for i in range(layers):
        layer(i)
    torch.cuda.synchronize(dev)
    side, graph = torch.cuda.Stream(dev), torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        layer(0)
        side.synchronize()
        with torch.cuda.graph(graph, stream=side):
            for i in range(layers):
                layer(i)
    torch.cuda.synchronize(dev)
    for _ in range(max(args.warmup, 3)):
        graph.replay()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = max(args.steps, 1)
    e0.record()
    for _ in range(reps):
        graph.replay()
    e1.record()
    torch.cuda.synchronize(dev)
    _lib.status(dev).raise_if_set()
    us = 1000.0 * e0.elapsed_time(e1) / (reps * layers)
    r = seqs * w
    alg = seqs * nv * 128 * 128 * 4 + r * (c + nv * 128) * 2 + r * nv * 128 * 2      # state read (kept in place), rows in, rows out
    peak, kind = peaks()
    print(json.dumps({"only": "gdn", "seqs": seqs, "width": w, "launches_per_layer": len(groups), "layers_rotated": layers, "us_per_layer": us,
                      "rows_per_s": r / us * 1e6, "algorithmic_bytes": alg, "achieved_gbs": alg / us / 1e3, "frac": alg / us / 1e3 / peak,
                      "peak_kind": kind,
                      "note": "state is read once and not written back by the verify step (the accepted prefix is replayed at commit)"}))


def only_attn(args, dev):
    """Lane GQA attention alone at the 27B-class shape (24 Q heads, 4 KV heads, head dim 256, 16-token pages): --seqs
    sequences x --width rows at context --ctx; 16 layers of KV rotated through, graph-replayed."""

    import torch

    from tensorfold_b200 import _lib, lane_attention as LA

    seqs, w, ctx, h, hk, d = args.seqs, args.width, args.ctx, 24, 4, 256
    layers = 16
    while layers > 1 and layers * seqs * (ctx + w) * 2 * hk * d * 2 > (24 << 30):
        layers //= 2
    pages_per = -(-(ctx + w) // 16)
    kv = LA.PagedKV(layers, seqs, seqs * pages_per, hk, d, pages_per, dev)
    for s_ in range(seqs):
        kv.reserve(s_, ctx + w)
    kv.sync_table()
    kv.k.normal_()
    kv.v.normal_()
    r = seqs * w
    gen = torch.Generator(device=dev).manual_seed(9)
    q = torch.randn((r, h, d), device=dev, generator=gen).to(torch.bfloat16)
    kn = torch.randn((r, hk, d), device=dev, generator=gen).to(torch.bfloat16)
    vn = torch.randn((r, hk, d), device=dev, generator=gen).to(torch.bfloat16)
    lens = torch.full((seqs,), ctx, dtype=torch.int32, device=dev)
    starts = torch.arange(0, r + 1, w, dtype=torch.int32, device=dev)
    nkeys = torch.tensor([ctx + t + 1 for _ in range(seqs) for t in range(w)], dtype=torch.int32, device=dev)
    ch = LA.chunks_for(ctx + w)
    scratch = torch.empty(LA.scratch_bytes(r, h, d, ch), dtype=torch.uint8, device=dev)
    out = torch.empty_like(q)

    def layer(i):
        LA.lane_attention(q, kn, vn, kv.k[i], kv.v[i], kv.table, lens, starts, nkeys, scale=d ** -0.5, max_window=w, max_chunks=ch,
                          scratch=scratch, out=out)
    for i in range(layers):
        layer(i)
    torch.cuda.synchronize(dev)
    side, graph = torch.cuda.Stream(dev), torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        layer(0)
        side.synchronize()
        with torch.cuda.graph(graph, stream=side):
            for i in range(layers):
                layer(i)
    torch.cuda.synchronize(dev)
    for _ in range(max(args.warmup, 3)):
        graph.replay()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = max(args.steps, 1)
    e0.record()
    for _ in range(reps):
        graph.replay()
    e1.record()
    torch.cuda.synchronize(dev)
    _lib.status(dev).raise_if_set()
    us = 1000.0 * e0.elapsed_time(e1) / (reps * layers)
    alg = seqs * (ctx + w) * 2 * hk * d * 2 + 2 * r * h * d * 2
    peak, kind = peaks()
    print(json.dumps({"only": "attn", "seqs": seqs, "width": w, "context": ctx, "layers_rotated": layers, "key_chunks": ch,
                      "us_per_layer": us, "algorithmic_bytes": alg, "achieved_gbs": alg / us / 1e3, "frac": alg / us / 1e3 / peak,
                      "peak_kind": kind, "l2": "KV of the rotated layers exceeds L2" if layers * alg > (126 << 20) else "KV fits L2"}))


def bench_moe(args, dev, rank=0, world=1):
    """The 30B-A3B-class workload: 48-layer MoE hybrid, 32 sequences with draft widths uniform in 1..8 (redrawn until
    they fit the 128-row forward) and contexts uniform in 1k..16k. The context is set synthetically (zero
    KV pages and recurrent state: same kernels, same traffic). With N ranks the experts are spread over
    the ranks (expert parallelism); attention, GDN and routing are replicated."""

    import random

    import torch

    from tensorfold_b200 import _lib, forward as F, lane_moe, runner, synthetic

    cfg = F.Config(**dict(synthetic.MOE_30B, layers=min(args.layers, 48)))
    ep = None
    if world > 1:
        ep = lane_moe.ExpertGroup(cfg.experts, cfg.top_k, cfg.shared_expert, cfg.hidden, dev)
    w = synthetic.random_weights(cfg, seed=2, device=dev, expert_ids=ep.local_experts(cfg.shared_expert) if ep else None)
    rng = random.Random(11)
    seqs = 32
    widths = [rng.randint(1, 8) for _ in range(seqs)]
    while sum(widths) > 128:
        widths = [rng.randint(1, 8) for _ in range(seqs)]
    ctxs = [rng.randint(1024, 16384) for _ in range(seqs)]
    rows = sum(widths)
    st = F.State(w, seqs, max(ctxs) + 16, dev)
    run = runner.LaneRunner(w, st, widths, max_context=max(ctxs) + 8, ep=ep)
    run.capture()
    st.lens = list(ctxs)
    run.refresh()
    gen = torch.Generator(device=dev).manual_seed(7)
    run.tokens.copy_(torch.randint(0, cfg.vocab, (rows,), generator=gen, device=dev, dtype=torch.int32))
    for _ in range(max(args.warmup, 3)):
        run.step_device()
    t_end = time.time() + (0.0 if args.no_spinup else 0.5)
    while time.time() < t_end:
        run.step_device()
        torch.cuda.synchronize(dev)
    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize(dev)

    def max_over_ranks(v):
        if world == 1:
            return v
        t = torch.tensor([v], device=dev, dtype=torch.float64)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        return float(t.item())

    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(dev.index or 0) as clk:
        e0.record()
        for _ in range(args.steps):
            run.step_device()
        e1.record()
        barrier()
    ms = max_over_ranks(e0.elapsed_time(e1))
    host_tokens = torch.randint(0, cfg.vocab, (rows,), dtype=torch.int32, generator=torch.Generator().manual_seed(13))   # every rank feeds the same tokens
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        run.step(host_tokens)
    barrier()
    e2e_s = max_over_ranks(time.perf_counter() - t0)
    _lib.status(dev).raise_if_set()
    if rank != 0:
        leave_group()
        return
    peak, kind = peaks()
    g = cfg.group
    bits = 0.5 + 4.0 / g
    dense = w.nbytes()
    per_expert = (3 * cfg.moe_intermediate * cfg.hidden) * bits
    touched = min(cfg.experts, rows * cfg.top_k) + 1          # upper bound of distinct experts a layer streams
    print(json.dumps({
        "metric": "lane-verify rows/sec", "value": args.steps * rows / (ms / 1000.0), "unit": "rows/s", "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"MoE hybrid 30B-A3B-class 4-bit g32 verify forward: {cfg.layers} layers, hidden 2048, 128 experts top-8 + "
                               f"shared, expert width 768; 32 sequences, draft widths uniform 1..8 ({rows} rows), contexts uniform 1k..16k "
                               "(set synthetically)", "seqs": seqs, "rows": rows,
                   "parallelism": "single GPU" if world == 1 else f"ep{world} (experts over ranks, the rest replicated)",
                   "l2": "weights streamed per forward exceed the 126 MB L2; no flush needed"},
        "clocks": clk.summary(),
        "e2e": {"value": args.steps * rows / e2e_s, "unit": "rows/s", "h2d_bytes_per_step": rows * 4, "d2h_bytes_per_step": rows * 4},
        "gpu_launches": run.launches * args.steps,
        "forward": {"dense_weight_bytes_per_step": dense,
                    "expert_weight_bytes_per_step_upper_bound": int(cfg.layers * touched * per_expert),
                    "weight_roofline_ms_upper_bound": (dense + cfg.layers * touched * per_expert) / (peak * 1e6), "peak_kind": kind}}),
          flush=True)
    if world > 1:
        leave_group()


def leave_group():
    """Every rank leaves the process group together; a timer ends the process if the teardown itself
    stalls (the result line is already printed by then)."""

    import torch

    guard = threading.Timer(60.0, lambda: os._exit(0))
    guard.daemon = True
    guard.start()
    torch.distributed.barrier()
    torch.distributed.destroy_process_group()
    guard.cancel()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--seqs", type=int, default=1)
    ap.add_argument("--ctx", type=int, default=4096)
    ap.add_argument("--width", type=int, default=8)
    ap.add_argument("--layers", type=int, default=64)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-batch16", action="store_true", help="skip the extra 16-sequence step (the 'batch16' key)")
    ap.add_argument("--synthetic-context", action="store_true",
                    help="skip the prefill: set the context length directly (KV pages and recurrent state stay zero); for profiler runs")
    ap.add_argument("--no-spinup", action="store_true", help="skip the half second of untimed steps that brings the clocks up")
    ap.add_argument("--exchange", default="peer", help="tensor-parallel exchange: 'peer' (own kernel over NVLink peer memory), 'peer-fused' (the same packets stored by "
                    "the row-parallel matmul's epilogue and awaited by the next norm kernel; slower as measured) or 'nccl' (all-gather)")
    ap.add_argument("--model", default="dense27b", help="'dense27b' (the headline workload) or 'moe30b': the 30B-A3B-class "
                    "mixture-of-experts hybrid (group 32, 128 experts top-8 + shared) on a ragged batch of 32 sequences")
    ap.add_argument("--only", default="", help="'qmm': time the lane matmul alone on --shape with --rows rows and exit; "
                    "'prefill': the same for the tcgen05 prefill-width matmul; 'gdn': the gated-DeltaNet lane step alone on --seqs x --width rows; "
                    "'attn': lane attention alone on --seqs x --width rows at --ctx; 'timeline': per-role breakdown of the matmuls of a step")
    ap.add_argument("--shape", default="17408x5120")
    ap.add_argument("--rows", type=int, default=8)
    ap.add_argument("--copies", type=int, default=4, help="--only qmm: weight copies rotated through (4 x 50 MB > L2)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rows = args.seqs * args.width
    workload = (f"dense hybrid 27B-class 4-bit g64 verify forward: {args.layers} layers (3 gated-DeltaNet : 1 GQA), hidden 5120, "
                f"MLP 17408, vocab 248320; {args.seqs} sequences x W={args.width} rows, context {args.ctx}")
    config = {"workload": workload, "seqs": args.seqs, "width": args.width, "context": args.ctx, "parallelism": f"tp{world}" + (f" ({args.exchange} exchange)" if world > 1 else ""),
              "l2": "weights (13.6 GB per forward) exceed the 126 MB L2; no flush needed"}

    if args.impl == "reference":
        if rank != 0:
            return
        base = cpu_reference(args, rows)
        gpu_leg = reference_gpu(args, rows)
        print(json.dumps({"reference_gpu": gpu_leg, "metric": "lane-verify rows/sec", "value": base["value"], "unit": "rows/s", "n_gpus": args.gpus,
                          "steps": 1, "warmup": 0, "ms_per_step": 1000.0 * rows / base["value"], "higher_is_better": True,
                          "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "reference",
                          "config": config, "cpu_baseline": base,
                          "e2e": {"value": base["value"], "unit": "rows/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))
        return

    import torch

    from tensorfold_b200 import _lib, build, forward as F, lane_qmm, runner, synthetic

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the lane kernels have no CPU path")
    build.build()
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    tp = None
    if world > 1:
        import torch.distributed as dist

        from tensorfold_b200 import distributed

        dist.init_process_group("nccl", device_id=dev)
        if args.model != "moe30b":
            try:
                tp = distributed.RankGroup(exchange="peer" if args.exchange == "peer-fused" else args.exchange,
                                           hidden=synthetic.DENSE_27B["hidden"], device=dev, fused=args.exchange == "peer-fused")
            except Exception as exc:      # no symmetric memory between these GPUs: the library collective still works
                if not args.exchange.startswith("peer"):
                    raise
                print(f"bench: peer exchange unavailable ({type(exc).__name__}: {exc}); using the NCCL all-gather", file=sys.stderr)
                args.exchange = "nccl"
                tp = distributed.RankGroup(exchange="nccl")
            config["parallelism"] = f"tp{world} ({args.exchange} exchange)"
    if args.gpus != world:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE is {world}: launch with torchrun --nproc-per-node {args.gpus}")

    if args.only in ("qmm", "prefill"):
        return only_qmm(args, dev)
    if args.only == "timeline":
        return only_timeline(args, dev)
    if args.only == "gdn":
        return only_gdn(args, dev)
    if args.only == "attn":
        return only_attn(args, dev)

    if args.model == "moe30b":
        return bench_moe(args, dev, rank, world)

    spec = dict(synthetic.DENSE_27B, layers=args.layers)
    cfg = F.Config(**spec)
    w = synthetic.random_weights(cfg, seed=2, device=dev, rank=rank, world=world)
    st = F.State(w, args.seqs, args.ctx + 2 * args.width, dev)
    run = runner.LaneRunner(w, st, [args.width] * args.seqs, max_context=args.ctx + args.width, tp=tp)
    run.capture()

    # ---- context: real prefill, W rows per sequence per replay, through the captured step ----
    gen = torch.Generator(device=dev).manual_seed(7)
    full = [args.width] * args.seqs
    if args.synthetic_context:
        st.lens = [args.ctx] * args.seqs
        run.refresh()
    while st.lens[0] + args.width <= args.ctx:
        run.tokens.copy_(torch.randint(0, cfg.vocab, (rows,), generator=gen, device=dev, dtype=torch.int32))
        run.step_device()
        run.commit(full)
    if st.lens[0] < args.ctx:                       # context not a multiple of W: a last partial commit
        run.tokens.copy_(torch.randint(0, cfg.vocab, (rows,), generator=gen, device=dev, dtype=torch.int32))
        run.step_device()
        run.commit([args.ctx - st.lens[0]] * args.seqs)
    torch.cuda.synchronize(dev)
    _lib.status(dev).raise_if_set()

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize(dev)

    run.tokens.copy_(torch.randint(0, cfg.vocab, (rows,), generator=gen, device=dev, dtype=torch.int32))
    for _ in range(max(args.warmup, 3)):
        run.step_device()
    # spin the clocks up: short bursts right after idle run at low clocks
    t_end = time.time() + (0.0 if args.no_spinup else 0.5)
    while time.time() < t_end:
        run.step_device()
        torch.cuda.synchronize(dev)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local) as clk:
        e0.record()
        for _ in range(args.steps):
            run.step_device()
        e1.record()
        barrier()
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device=dev)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        ms = float(t.item())
    value = args.steps * rows / (ms / 1000.0)

    # ---- end to end through the public call: host tokens in, chosen tokens out, every step ----
    host_tokens = torch.randint(0, cfg.vocab, (rows,), dtype=torch.int32, generator=torch.Generator().manual_seed(13))   # every rank feeds the same tokens
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        run.step(host_tokens)
    barrier()
    e2e_s = time.perf_counter() - t0
    if world > 1:
        t = torch.tensor([e2e_s], device=dev)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        e2e_s = float(t.item())

    # ---- extra: the same forward over 16 concurrent sequences x W rows (context set directly) ----
    batch16 = None
    if not args.no_batch16 and world == 1 and args.seqs == 1 and 16 * args.width <= 128:
        F.enable_wide(w)                 # 128 rows a step: the tcgen05 wide-row kernel for every matmul of this state
        st16 = F.State(w, 16, args.ctx + 2 * args.width, dev, wide=True)
        run16 = runner.LaneRunner(w, st16, [args.width] * 16, max_context=args.ctx + args.width, tp=tp)
        run16.capture()
        st16.lens = [args.ctx] * 16
        run16.refresh()
        run16.tokens.copy_(torch.randint(0, cfg.vocab, (16 * args.width,), generator=gen, device=dev, dtype=torch.int32))
        for _ in range(3):
            run16.step_device()
        barrier()
        b0, b1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        b0.record()
        for _ in range(args.steps):
            run16.step_device()
        b1.record()
        barrier()
        ms16 = b0.elapsed_time(b1)
        if world > 1:
            t = torch.tensor([ms16], device=dev)
            torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
            ms16 = float(t.item())
        batch16 = {"seqs": 16, "rows": 16 * args.width, "ms_per_step": ms16 / args.steps, "matmul": "tcgen05 wide-row kernel (bf16 x bf16 -> fp32 in tensor memory)",
                   "rows_per_s": args.steps * 16 * args.width / (ms16 / 1000.0), "context": f"{args.ctx} (set directly: zero KV pages and state)"}
        del run16, st16

    # ---- dominant kernel: the lane matmul, every launch of one forward replayed alone ----
    mats = []
    for layer in w.layers:
        mats += [layer.in_proj, layer.out_proj, layer.gate_up, layer.down]
    mats.append(w.head)
    packs = {}
    for q in mats:
        if q.k not in packs:
            packs[q.k] = lane_qmm.pack_rows(torch.randn((rows, q.k), device=dev).to(torch.bfloat16), cfg.group)
    outs = {q.n: torch.empty((rows, q.n), dtype=torch.bfloat16, device=dev) for q in mats}
    side = torch.cuda.Stream(dev)
    with torch.cuda.stream(side):
        for q in mats[:5]:
            lane_qmm.lane_matmul(packs[q.k], q, out=outs[q.n])
        side.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            for q in mats:
                lane_qmm.lane_matmul(packs[q.k], q, out=outs[q.n])
    torch.cuda.synchronize(dev)
    g.replay()
    torch.cuda.synchronize(dev)
    q0, q1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = 5
    q0.record()
    for _ in range(reps):
        g.replay()
    q1.record()
    torch.cuda.synchronize(dev)
    qmm_ms = q0.elapsed_time(q1) / reps

    def alg_bytes(q):
        kg = q.k // q.group
        return q.n * q.k // 2 + q.n * kg * 4 + rows * q.k * 2 + rows * kg * 4 + rows * q.n * 2
    total_bytes = sum(alg_bytes(q) for q in mats)
    peak, peak_kind = peaks()
    achieved = total_bytes / (qmm_ms / 1000.0) / 1e9
    weight_bytes = sum(q.n * q.k // 2 + q.n * (q.k // q.group) * 4 for q in mats)
    _lib.status(dev).raise_if_set()
    if rank != 0:
        leave_group()       # a rank that exits alone leaves the others waiting
        return
    line = {
        "metric": "lane-verify rows/sec", "value": value, "unit": "rows/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": config,
        "clocks": clk.summary(),
        "e2e": {"value": args.steps * rows / e2e_s, "unit": "rows/s", "h2d_bytes_per_step": rows * 4, "d2h_bytes_per_step": rows * 4},
        "gpu_launches": run.launches * args.steps,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "peak_kind": f"of {peak_kind}", "frac_of_8000": achieved / 8000.0,
                     "kernel": "qmm_kernel (4-bit lane matmul)", "launches_per_step": len(mats),
                     "avg_launch_us": 1000.0 * qmm_ms / len(mats), "algorithmic_bytes_per_launch": total_bytes / len(mats),
                     "traffic": 0.996 * total_bytes / len(mats),
                     "traffic_note": "dram bytes of one ncu capture (17408x5120, 8 rows: 50.28 MB read + 0.03 MB written for 50.50 MB algorithmic), scaled by units"},
        "forward": {"weight_bytes_per_step": weight_bytes, "weight_roofline_ms": weight_bytes / (peak * 1e6),
                    "frac_of_weight_roofline": (weight_bytes / (peak * 1e6)) / (ms / args.steps),
                    "qmm_ms_per_step": qmm_ms, "qmm_share": qmm_ms / (ms / args.steps)},
    }
    if batch16 is not None:
        batch16["frac_of_weight_roofline"] = (weight_bytes / (peak * 1e6)) / batch16["ms_per_step"]
        line["batch16"] = batch16
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_reference(args, rows)
    print(json.dumps(line), flush=True)
    if world > 1:
        leave_group()


if __name__ == "__main__":
    main()
