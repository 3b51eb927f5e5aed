"""Plan of the Gebasun design: token embedding; parallel blocks in which the mixer and the
feed-forward each read an RMS norm of their own of the same stream, x + mixer(norm1(x)) +
ff(norm2(x)); three kinds of mixer, chosen layer by layer — window attention whose values are
the projected keys, with unit-norm queries and keys, a learned bias by (bucketed) distance, a
learned sink and an output bias; window attention that also keeps a request's first tokens,
with rotary positions on part of a head, unit-norm queries and keys, a learned sink and a
gate on every output value; a selective state-space recurrence — and a routed feed-forward
(the largest logits chosen, a softmax over the chosen ones, experts without a gate whose
activation is the square of relu, an expert every token runs) or none; a final RMS norm and
an output head of its own.

Every layer's parts are made from that layer's entry of the configuration, so the order of
the layers and all sizes are the file's.
"""
from __future__ import annotations

from ..config.gebasun_config import (BiasAttentionConfig, GebasunConfig, RotaryAttentionConfig,
                                     StateSpaceConfig, fill_from_tensor_shapes)
from ..config.registry import register_architecture
from ..parts import ModelPlan, OutputHead, TokenEmbedding, part_class

_MIXER_NAMES = ("q", "k", "v", "o", "g", "q.norm", "k.norm")


def build_gebasun_plan(cfg: GebasunConfig) -> ModelPlan:
    norm_cls = part_class("norm", "rmsnorm")
    block_cls = part_class("block", "parallel")
    attention_cls = part_class("mixer", "sink_gqa_attention")
    state_cls = part_class("mixer", "selective_state")
    ffn_cls = part_class("feed_forward", "routed_experts")
    rotary_cls = part_class("position_encoding", "rotary")
    encodings = {}          # one encoding per distinct (dims, base): layers that agree share its tables

    def norm():
        return norm_cls(cfg.width, cfg.norm_eps, tensor_name="")

    layers, prefixes = [], []
    for i, layer in enumerate(cfg.layers):
        mx = layer.mixer
        if isinstance(mx, BiasAttentionConfig):
            mixer = attention_cls(cfg.width, mx.heads, mx.kv_heads, mx.dim, mx.scale, value_dim=mx.vdim,
                                  qk_norm="plain", eps=cfg.norm_eps, sink="learned", head_gate=False,
                                  window=mx.window, names=_MIXER_NAMES, values="keys",
                                  distance_table=(_rows_of(mx, i), mx.bias_max), qk_bias=True, out_bias=True)
        elif isinstance(mx, RotaryAttentionConfig):
            key = (mx.rot_dims, mx.rot_base)
            if key not in encodings:
                encodings[key] = rotary_cls(mx.rot_dims, mx.rot_base)
            mixer = attention_cls(cfg.width, mx.heads, mx.kv_heads, mx.dim, mx.scale, value_dim=mx.vdim,
                                  qk_norm="plain", eps=cfg.norm_eps, sink="learned", head_gate="wide",
                                  window=mx.window, names=_MIXER_NAMES, values="keys",
                                  position=encodings[key], rotary_dim=mx.rot_dims, keep_first=mx.keep_first,
                                  qk_bias=True, out_bias=False)
        elif isinstance(mx, StateSpaceConfig):
            mixer = state_cls(cfg.width, mx.heads, mx.vdim, mx.state, mx.groups, mx.conv, mx.norm_groups,
                              cfg.norm_eps)
        else:
            raise ValueError(f"layer {i}: no mixer for {type(mx).__name__}")
        ml = layer.mlp
        ffn = None
        if ml is not None:
            ffn = ffn_cls(cfg.width, ml.ff, ml.experts, ml.top, router="top_softmax", router_bias=True,
                          weight_on="output", activation="relu2", shared_inner=ml.shared_ff)
        layers.append(block_cls(norm(), mixer, ffn, mult=1.0, layer_scale=False,
                                ffn_norm=norm() if ffn is not None else None))
        prefixes.append(f"l{i}.")
    return ModelPlan(
        config=cfg,
        embedding=TokenEmbedding(cfg.vocab_size, cfg.width, tensor_name=""),
        position=None,
        layers=layers,
        layer_prefixes=prefixes,
        final_norm=norm(),
        head=OutputHead(cfg.vocab_size, cfg.width, tensor_name=""),
        embedding_prefix="embed",
        final_norm_prefix="final.norm",
        head_prefix="head",
        benign_suffixes=(),
    )


def _rows_of(mx: BiasAttentionConfig, layer: int) -> int:
    rows = mx.bias_rows
    if rows is None:
        raise ValueError(f"layer {layer}: the number of rows of the distance-bias table is read off the "
                         "checkpoint ('rel'), and no checkpoint was given")
    return rows


def _toy_config(sizes):
    """config.json of a small model of the design from the sizes ``make-toy-model`` takes: the
    three kinds of mixer in turn; every layer but the last has a routed feed-forward."""
    width = sizes["hidden_size"]
    heads = sizes["heads"]
    hd = sizes.get("head_dim") or max(8, (width // heads) // 2 * 2)
    inner = sizes.get("intermediate_size") or 2 * width
    n = sizes["layers"]
    layers = []
    for i in range(n):
        kind = ("attention", "attention_2", "mamba2")[i % 3]
        if kind == "attention":
            mixer = {"heads": heads, "kv_heads": sizes["kv_heads"], "dim": hd, "vdim": hd, "scale": hd ** -0.5,
                     "bias_max": 96, "bias_rows": 16, "mask": {"size": 48}}
        elif kind == "attention_2":
            mixer = {"heads": heads, "kv_heads": sizes["kv_heads"], "dim": hd, "vdim": hd, "scale": hd ** -0.5,
                     "mask": {"size": 32, "keep_first": 4}, "rot": {"dims": hd // 2 // 2 * 2, "base": 10000.0}}
        else:
            mixer = {"heads": heads, "vdim": hd, "state": 16, "groups": sizes["kv_heads"], "conv": 4,
                     "norm_groups": 1}
        mlp = None if (i == n - 1 and n > 1) else \
            {"kind": "moe", "expert": {"ff": max(8, inner // 4)}, "router": {"experts": 4, "top": 2},
             "shared": {"ff": max(8, inner // 2)}}
        layers.append({"type": kind, "mixer": mixer, "mlp": mlp})
    return {"architecture": "Gebasun", "vocab": sizes["vocab_size"], "width": width,
            "norm": {"eps": sizes["rms_eps"]}, "layers": layers}


register_architecture("Gebasun", GebasunConfig.from_json, build_gebasun_plan, toy_config=_toy_config,
                      sizes_from_tensors=fill_from_tensor_shapes, replace=True)
