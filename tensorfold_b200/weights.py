"""Reading a 4-bit MLX checkpoint (safetensors + config.json) into the lane forward's weights.

Mirror of the reference's ``families/qwen3_5/cuda/weights.py:38-198`` (``Config.read``, ``load``): the
same ``config.json`` keys and tensor names (``model.layers.N.linear_attn.in_proj_qkv.weight/.scales/
.biases`` and so on, optionally under ``language_model.``); vision and MTP tensors are skipped, any other
unused tensor is an error. Stored arrays are MLX affine 4-bit: uint32 words [N, K/8] with scales and
biases [N, K/group]. ``load`` returns the stored-layout dict that ``forward.load_weights`` (one GPU) or
``distributed.split_model`` (a tensor-parallel rank) take; nothing is repacked on the way.
"""

from __future__ import annotations

import json
from pathlib import Path
from types import SimpleNamespace

import torch

from .forward import Config


def read_config(model_dir: str | Path, group: int = 64) -> Config:
    raw = json.loads((Path(model_dir) / "config.json").read_text())
    t = raw.get("text_config", raw)
    rope = t.get("rope_parameters") or {}
    head_dim = int(t.get("head_dim") or t["hidden_size"] // t["num_attention_heads"])
    q = raw.get("quantization") or t.get("quantization") or {}
    return Config(hidden=int(t["hidden_size"]), intermediate=int(t["intermediate_size"]), layers=int(t["num_hidden_layers"]),
                  heads=int(t["num_attention_heads"]), kv_heads=int(t["num_key_value_heads"]), head_dim=head_dim,
                  vocab=int(t["vocab_size"]), k_heads=int(t["linear_num_key_heads"]), v_heads=int(t["linear_num_value_heads"]),
                  dk=int(t["linear_key_head_dim"]), dv=int(t["linear_value_head_dim"]),
                  conv_kernel=int(t["linear_conv_kernel_dim"]), interval=int(t.get("full_attention_interval", 4)),
                  eps=float(t.get("rms_norm_eps", 1e-6)),
                  rope_dims=int(head_dim * float(rope.get("partial_rotary_factor", t.get("partial_rotary_factor", 0.25)))),
                  rope_theta=float(rope.get("rope_theta", t.get("rope_theta") or 10000000.0)),
                  group=int(q.get("group_size", group)))


def _tensors(model_dir: Path) -> dict:
    from safetensors import safe_open

    out = {}
    for path in sorted(model_dir.glob("*.safetensors")):
        with safe_open(str(path), framework="pt", device="cpu") as f:
            for name in f.keys():
                if name.startswith("vision_tower") or ".mtp." in name or name.startswith("mtp."):
                    continue
                out[name] = f.get_tensor(name)
    return out


def load(model_dir: str | Path) -> dict:
    """The checkpoint as the stored-layout model dict (host tensors)."""

    model_dir = Path(model_dir)
    cfg = read_config(model_dir)
    t = _tensors(model_dir)
    prefix = "language_model." if any(k.startswith("language_model.") for k in t) else ""

    def get(name):
        return t.pop(prefix + name)

    def q4(name):
        w = get(name + ".weight")
        w = w.view(torch.int32) if w.dtype != torch.int32 else w
        return SimpleNamespace(words=w.contiguous(), scales=get(name + ".scales").contiguous(), biases=get(name + ".biases").contiguous())

    layers = []
    for i in range(cfg.layers):
        p = f"model.layers.{i}."
        layer = {"linear": cfg.is_linear(i), "input_norm": get(p + "input_layernorm.weight"),
                 "post_norm": get(p + "post_attention_layernorm.weight"), "gate": q4(p + "mlp.gate_proj"),
                 "up": q4(p + "mlp.up_proj"), "down": q4(p + "mlp.down_proj")}
        if layer["linear"]:
            a = p + "linear_attn."
            layer.update(qkv=q4(a + "in_proj_qkv"), z=q4(a + "in_proj_z"), b=q4(a + "in_proj_b"), a=q4(a + "in_proj_a"),
                         out=q4(a + "out_proj"), conv=get(a + "conv1d.weight").reshape(-1, cfg.conv_kernel).contiguous(),
                         A_log=get(a + "A_log").float(), dt_bias=get(a + "dt_bias").float(), norm=get(a + "norm.weight"))
        else:
            a = p + "self_attn."
            layer.update(q=q4(a + "q_proj"), k=q4(a + "k_proj"), v=q4(a + "v_proj"), o=q4(a + "o_proj"),
                         q_norm=get(a + "q_norm.weight"), k_norm=get(a + "k_norm.weight"))
        layers.append(layer)
    model = {"config": cfg, "layers": layers, "embed": q4("model.embed_tokens"), "norm": get("model.norm.weight"),
             "head": q4("lm_head")}
    left = [k for k in t if not k.startswith("vision")]
    if left:
        raise ValueError(f"unused checkpoint tensors: {left[:5]} ...")
    return model


def save(model: dict, model_dir: str | Path) -> None:
    """Write a stored-layout model dict as ``config.json`` + ``model.safetensors`` under the names ``load``
    reads (for tests and for exporting synthetic models)."""

    from safetensors.torch import save_file

    model_dir = Path(model_dir)
    model_dir.mkdir(parents=True, exist_ok=True)
    c = model["config"]
    out = {}

    def put(name, q):
        out[name + ".weight"] = q.words.contiguous()
        out[name + ".scales"] = q.scales.contiguous()
        out[name + ".biases"] = q.biases.contiguous()

    for i, layer in enumerate(model["layers"]):
        p = f"model.layers.{i}."
        out[p + "input_layernorm.weight"] = layer["input_norm"]
        out[p + "post_attention_layernorm.weight"] = layer["post_norm"]
        for name in ("gate", "up", "down"):
            put(p + f"mlp.{name}_proj", layer[name])
        if layer["linear"]:
            a = p + "linear_attn."
            for name in ("qkv", "z", "b", "a"):
                put(a + "in_proj_" + name, layer[name])
            put(a + "out_proj", layer["out"])
            out[a + "conv1d.weight"] = layer["conv"].reshape(layer["conv"].shape[0], 1, -1).contiguous()
            out[a + "A_log"] = layer["A_log"]
            out[a + "dt_bias"] = layer["dt_bias"]
            out[a + "norm.weight"] = layer["norm"]
        else:
            a = p + "self_attn."
            for name in ("q", "k", "v", "o"):
                put(a + name + "_proj", layer[name])
            out[a + "q_norm.weight"] = layer["q_norm"]
            out[a + "k_norm.weight"] = layer["k_norm"]
    put("model.embed_tokens", model["embed"])
    put("lm_head", model["head"])
    out["model.norm.weight"] = model["norm"]
    save_file({k: v.contiguous() for k, v in out.items()}, str(model_dir / "model.safetensors"))
    cfg = {"hidden_size": c.hidden, "intermediate_size": c.intermediate, "num_hidden_layers": c.layers,
           "num_attention_heads": c.heads, "num_key_value_heads": c.kv_heads, "head_dim": c.head_dim, "vocab_size": c.vocab,
           "linear_num_key_heads": c.k_heads, "linear_num_value_heads": c.v_heads, "linear_key_head_dim": c.dk,
           "linear_value_head_dim": c.dv, "linear_conv_kernel_dim": c.conv_kernel, "full_attention_interval": c.interval,
           "rms_norm_eps": c.eps, "partial_rotary_factor": c.rope_dims / c.head_dim, "rope_theta": c.rope_theta,
           "quantization": {"group_size": c.group, "bits": 4}, "eos_token_id": 0}
    (model_dir / "config.json").write_text(json.dumps(cfg))


__all__ = ["load", "read_config", "save"]
