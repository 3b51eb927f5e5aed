"""Plan of the Fobanex design: a token embedding times a constant; parallel blocks with ONE
RMS norm whose output both sublayers read, x + mixer(norm(x)) + ff(norm(x)); three kinds of
mixer, chosen layer by layer — grouped-query attention with an RMS norm over the whole query
and key projections ahead of rotary positions on neighbouring pairs of part of a head;
attention whose values are the keys as projected, with the same rotation and a gate on every
output value; attention over a low-rank latent whose queries pass a latent of their own, with
rotary positions on halves of a shared key part, a gate on every output value, and, for a
layer that says so, the latent rows another layer keeps instead of rows of its own — and a
feed-forward that is dense (silu gate, biases), routed (softmax router, the choice limited to
the best groups of neighbouring experts, the chosen scores normalised and scaled, clamped-swish
experts weighted on their outputs) or absent; a final RMS norm and an output head of its own.

Every layer's parts are made from that layer's entry of the configuration, so the order of
the layers and all sizes are the file's.  Layers with equal rotary constants share one
encoding (one cos/sin table a step).  A layer that reads another layer's latent rows is
scheduled with that layer's cache and does not write it.
"""
from __future__ import annotations

from ..config.fobanex_config import (DenseFfnConfig, FobanexConfig, GroupedRouterFfnConfig,
                                     KeyValueAttentionConfig, QueryLatentAttentionConfig,
                                     RowNormAttentionConfig, fill_from_tensor_shapes)
from ..config.registry import register_architecture
from ..parts import ModelPlan, OutputHead, TokenEmbedding, part_class
from ..parts.plan import Run
from .zokelix import _encoding

_MIXER_NAMES = ("q", "k", "v", "o", "g", "q.norm", "k.norm")


def build_fobanex_plan(cfg: FobanexConfig) -> ModelPlan:
    norm_cls = part_class("norm", "rmsnorm")
    block_cls = part_class("block", "parallel")
    attention_cls = part_class("mixer", "sink_gqa_attention")
    latent_cls = part_class("mixer", "latent_attention")
    encodings = {}          # one encoding per distinct set of rotary constants

    def norm():
        return norm_cls(cfg.width, cfg.norm_eps, tensor_name="")

    layers, prefixes, schedule = [], [], []
    for i, layer in enumerate(cfg.layers):
        mx = layer.mixer
        run = Run(i)
        if isinstance(mx, RowNormAttentionConfig):
            mixer = attention_cls(cfg.width, mx.heads, mx.kv_heads, mx.dim, mx.scale, value_dim=mx.vdim,
                                  qk_norm="row", eps=cfg.norm_eps, sink=False, head_gate=False,
                                  names=_MIXER_NAMES, position=_encoding(mx.rot, encodings),
                                  rotary_dim=mx.rot.dims, rotary_pairing="neighbours")
        elif isinstance(mx, KeyValueAttentionConfig):
            mixer = attention_cls(cfg.width, mx.heads, mx.kv_heads, mx.dim, mx.scale, value_dim=mx.vdim,
                                  qk_norm=False, eps=cfg.norm_eps, sink=False, head_gate="wide",
                                  names=_MIXER_NAMES, values="keys", position=_encoding(mx.rot, encodings),
                                  rotary_dim=mx.rot.dims, rotary_pairing="neighbours")
        elif isinstance(mx, QueryLatentAttentionConfig):
            if mx.q_rank is None:
                raise ValueError(f"layer {i}: the rank of the query latent is neither in config.json "
                                 "('q_rank') nor read off a checkpoint")
            mixer = latent_cls(cfg.width, mx.heads, mx.dim, mx.rot_dim, mx.vdim, mx.kv_rank, mx.scale,
                               cfg.norm_eps, _encoding(mx.rot, encodings), q_rank=mx.q_rank,
                               pairing="halves", gate=True, own_rows=mx.kv_from is None)
            if mx.kv_from is not None:
                run = Run(i, cache=mx.kv_from, writes_cache=False)      # one run a layer: entry = layer
        else:
            raise ValueError(f"layer {i}: no mixer for {type(mx).__name__}")
        ml = layer.mlp
        if ml is None:
            ffn = None
        elif isinstance(ml, DenseFfnConfig):
            ffn = part_class("feed_forward", "gated_mlp")(
                cfg.width, ml.ff, activation="silu", bias=True, names=("gate", "up", "down"))
        elif isinstance(ml, GroupedRouterFfnConfig):
            ffn = part_class("feed_forward", "routed_experts")(
                cfg.width, ml.ff, ml.experts, ml.top, ml.limit, router="softmax", weight_on="output",
                activation="clamped_swish", groups=(ml.group_count, ml.group_keep), normalize=True,
                weight_scale=ml.scale)
        else:
            raise ValueError(f"layer {i}: no feed-forward for {type(ml).__name__}")
        layers.append(block_cls(norm(), mixer, ffn, mult=1.0, layer_scale=False))
        prefixes.append(f"l{i}.")
        schedule.append(run)
    return ModelPlan(
        config=cfg,
        embedding=TokenEmbedding(cfg.vocab_size, cfg.width, tensor_name="", scale=cfg.embedding_scale),
        position=None,
        layers=layers,
        layer_prefixes=prefixes,
        final_norm=norm(),
        head=OutputHead(cfg.vocab_size, cfg.width, tensor_name=""),
        schedule=schedule,
        embedding_prefix="embed",
        final_norm_prefix="final.norm",
        head_prefix="head",
        benign_suffixes=(),
    )


def _toy_config(sizes):
    """config.json of a small model of the design from the sizes ``make-toy-model`` takes: the
    kinds of mixer in turn (attention, latent attention, latent attention on the rows of the
    layer before, attention whose values are its keys); the first feed-forward is dense, the
    others routed, the last layer has none."""
    width = sizes["hidden_size"]
    heads = sizes["heads"]
    hd = sizes.get("head_dim") or max(8, (width // heads) // 2 * 2)
    inner = sizes.get("intermediate_size") or 2 * width
    n = sizes["layers"]
    rot = {"base": sizes["rope_theta"], "dims": max(2, hd // 2 // 2 * 2)}
    if sizes.get("rope_scaling"):
        f, lo, hi, orig = sizes["rope_scaling"]
        rot["scaling"] = {"factor": f, "fast": hi, "slow": lo, "original": int(orig)}
    layers = []
    for i in range(n):
        kind = ("attention", "latent_attention", "latent_attention", "attention_2")[i % 4]
        if kind == "latent_attention":
            mixer = {"heads": heads, "dim": hd, "rot_dim": rot["dims"], "vdim": hd, "kv_rank": 2 * hd,
                     "q_rank": max(8, width // 4), "scale": (hd + rot["dims"]) ** -0.5,
                     "rot": {"base": sizes["rope_theta"], "dims": rot["dims"]}}
            if i % 4 == 2:
                mixer["kv_from"] = i - 1
        else:
            mixer = {"heads": heads, "kv_heads": sizes["kv_heads"], "dim": hd, "vdim": hd, "scale": hd ** -0.5,
                     "rot": rot}
        if i == n - 1 and n > 1:
            mlp = None
        elif i == 0:
            mlp = {"kind": "dense", "ff": inner}
        else:
            mlp = {"kind": "moe", "expert": {"ff": max(8, inner // 4), "limit": 7.0},
                   "router": {"experts": 4, "top": 2, "scale": 1.0, "groups": {"count": 2, "keep": 1}}}
        layers.append({"type": kind, "mixer": mixer, "mlp": mlp})
    return {"architecture": "Fobanex", "vocab": sizes["vocab_size"], "width": width,
            "embedding": {"scale": float(width) ** 0.5}, "norm": {"eps": sizes["rms_eps"]}, "layers": layers}


register_architecture("Fobanex", FobanexConfig.from_json, build_fobanex_plan, toy_config=_toy_config,
                      sizes_from_tensors=fill_from_tensor_shapes, replace=True)
