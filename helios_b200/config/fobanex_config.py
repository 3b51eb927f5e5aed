"""Typed configuration of the Fobanex design, read from ``config.json``.

The file lists the layers one by one; every entry names its mixer by ``type`` (``attention``:
grouped-query attention with an RMS norm over the whole query and key projections and rotary
positions on neighbouring pairs; ``attention_2``: the same rotation, the values are the keys as
projected, a gate on every output value; ``latent_attention``: attention over a low-rank latent
with queries through a latent of their own, a gate on every output value, and optionally the
latent rows of ANOTHER layer, ``kv_from``) with the mixer's sizes, and its feed-forward (dense,
routed, or null for none).  Two models of the design may differ in every size, in the order of
the layers and in every constant; nothing here has a default that stands for a value of some
particular model.  What the file leaves out of an optional piece (a rotary scaling, the groups
of a router, the embedding's scale, a layer's feed-forward) is absent.  Sizes that the file
does not give are read off the checkpoint's tensor shapes.
"""
from __future__ import annotations

from dataclasses import dataclass, replace
from typing import Any, Dict, Optional, Tuple, Union

from .model_config import ConfigError
from .zokelix_config import RotaryConfig, YarnScaling, _need


@dataclass(frozen=True)
class RowNormAttentionConfig:
    """``attention``."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot: RotaryConfig


@dataclass(frozen=True)
class KeyValueAttentionConfig:
    """``attention_2``: the values are the keys as projected."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot: RotaryConfig


@dataclass(frozen=True)
class QueryLatentAttentionConfig:
    """``latent_attention``."""
    heads: int
    dim: int                  # unrotated query/key values per head
    rot_dim: int              # rotated query/key values per head (the key part is shared)
    vdim: int
    kv_rank: int
    q_rank: Optional[int]     # None until read off the checkpoint's 'dq'
    scale: float
    rot: RotaryConfig
    kv_from: Optional[int]    # the layer whose latent rows this one reads; None: its own


@dataclass(frozen=True)
class DenseFfnConfig:
    ff: int


@dataclass(frozen=True)
class GroupedRouterFfnConfig:
    ff: int
    limit: float
    experts: int
    top: int
    scale: float              # factor on the chosen experts' normalised weights
    group_count: int          # 1: every expert is eligible
    group_keep: int


MixerConfig = Union[RowNormAttentionConfig, KeyValueAttentionConfig, QueryLatentAttentionConfig]


@dataclass(frozen=True)
class FobanexLayer:
    type: str
    mixer: MixerConfig
    mlp: Union[DenseFfnConfig, GroupedRouterFfnConfig, None]


@dataclass(frozen=True)
class FobanexConfig:
    architecture: str
    vocab_size: int
    width: int
    norm_eps: float
    embedding_scale: float
    layers: Tuple[FobanexLayer, ...]
    eos_token_ids: Tuple[int, ...] = ()

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    @property
    def max_position_embeddings(self) -> int:
        """No part of the design bounds a request's length."""
        return 1 << 30

    @classmethod
    def from_json(cls, cfg: Dict[str, Any]) -> "FobanexConfig":
        vocab = _need(cfg, "vocab", "the file")
        width = _need(cfg, "width", "the file")
        eps = _need(cfg.get("norm"), "eps", "norm", float)
        emb = cfg.get("embedding")
        scale = _need(emb, "scale", "embedding", float) if isinstance(emb, dict) and "scale" in emb else 1.0
        layers = cfg.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        out = []
        for i, layer in enumerate(layers):
            where = f"layers[{i}]"
            kind = layer.get("type") if isinstance(layer, dict) else None
            reader = _MIXERS.get(kind)
            if reader is None:
                raise ConfigError(f"config.json: {where}.type {kind!r} is not supported "
                                  f"({', '.join(sorted(_MIXERS))})")
            out.append(FobanexLayer(kind, reader(layer.get("mixer"), where + ".mixer"),
                                    _mlp(layer.get("mlp"), where + ".mlp")))
        for i, layer in enumerate(out):
            _check_source(out, i)
        eos = cfg.get("eos_token_id")
        eos_ids = () if eos is None else tuple(int(e) for e in (eos if isinstance(eos, (list, tuple)) else [eos]))
        return cls(architecture=str(cfg.get("architecture", "Fobanex")), vocab_size=vocab, width=width,
                   norm_eps=eps, embedding_scale=scale, layers=tuple(out), eos_token_ids=eos_ids)


def _check_source(layers, i: int) -> None:
    """A layer that reads another layer's latent rows: that layer comes earlier, keeps rows
    of its own, and rows of the same sizes and rotation."""
    mx = layers[i].mixer
    if not isinstance(mx, QueryLatentAttentionConfig) or mx.kv_from is None:
        return
    where = f"config.json: layers[{i}].mixer.kv_from {mx.kv_from}"
    if not 0 <= mx.kv_from < i:
        raise ConfigError(f"{where} must name an earlier layer")
    src = layers[mx.kv_from].mixer
    if not isinstance(src, QueryLatentAttentionConfig) or src.kv_from is not None:
        raise ConfigError(f"{where} must name a latent_attention layer that keeps rows of its own")
    if (src.kv_rank, src.rot_dim, src.rot) != (mx.kv_rank, mx.rot_dim, mx.rot):
        raise ConfigError(f"{where}: that layer's kv_rank, rot_dim or rotation differ from this layer's")


def _rotary(rot, where, most: int) -> RotaryConfig:
    dims = _need(rot, "dims", where)
    if dims % 2 or dims > most:
        raise ConfigError(f"config.json: {where}.dims {dims} must be even and at most {most}")
    sc = rot.get("scaling")
    scaling = None
    if sc:
        scaling = YarnScaling(_need(sc, "factor", where + ".scaling", float),
                              _need(sc, "original", where + ".scaling", float),
                              _need(sc, "fast", where + ".scaling", float),
                              _need(sc, "slow", where + ".scaling", float))
    return RotaryConfig(_need(rot, "base", where, float), dims, scaling)


def _heads(mx, where):
    heads, kv_heads = _need(mx, "heads", where), _need(mx, "kv_heads", where)
    if heads % kv_heads:
        raise ConfigError(f"config.json: {where}.kv_heads {kv_heads} must divide heads {heads}")
    return heads, kv_heads, _need(mx, "dim", where), _need(mx, "vdim", where)


def _attention(mx, where) -> RowNormAttentionConfig:
    heads, kv_heads, dim, vdim = _heads(mx, where)
    return RowNormAttentionConfig(heads, kv_heads, dim, vdim, _need(mx, "scale", where, float),
                                  _rotary(mx.get("rot"), where + ".rot", dim))


def _attention_2(mx, where) -> KeyValueAttentionConfig:
    heads, kv_heads, dim, vdim = _heads(mx, where)
    if vdim != dim:
        raise ConfigError(f"config.json: {where}.vdim {vdim} differs from dim {dim}, but the values are "
                          "the projected keys")
    return KeyValueAttentionConfig(heads, kv_heads, dim, vdim, _need(mx, "scale", where, float),
                                   _rotary(mx.get("rot"), where + ".rot", dim))


def _optional(mx, key, where):
    return _need(mx, key, where) if isinstance(mx, dict) and mx.get(key) is not None else None


def _latent(mx, where) -> QueryLatentAttentionConfig:
    rot_dim = _need(mx, "rot_dim", where)
    rot = _rotary(mx.get("rot"), where + ".rot", rot_dim)
    src = mx.get("kv_from")
    if src is not None and (not isinstance(src, int) or isinstance(src, bool) or src < 0):
        raise ConfigError(f"config.json: {where}.kv_from must be a layer's index, got {src!r}")
    return QueryLatentAttentionConfig(
        heads=_need(mx, "heads", where), dim=_need(mx, "dim", where), rot_dim=rot_dim,
        vdim=_need(mx, "vdim", where), kv_rank=_need(mx, "kv_rank", where),
        q_rank=_optional(mx, "q_rank", where), scale=_need(mx, "scale", where, float), rot=rot, kv_from=src)


_MIXERS = {"attention": _attention, "attention_2": _attention_2, "latent_attention": _latent}


def _mlp(ml, where):
    if ml is None:
        return None
    kind = ml.get("kind") if isinstance(ml, dict) else None
    if kind == "dense":
        return DenseFfnConfig(_need(ml, "ff", where))
    if kind != "moe":
        raise ConfigError(f"config.json: {where}.kind {kind!r} is not supported (dense, moe)")
    ex, ro = ml.get("expert"), ml.get("router")
    experts, top = _need(ro, "experts", where + ".router"), _need(ro, "top", where + ".router")
    count, keep = 1, 1
    groups = ro.get("groups")
    if groups:
        count, keep = _need(groups, "count", where + ".router.groups"), _need(groups, "keep", where + ".router.groups")
        if experts % count or keep > count:
            raise ConfigError(f"config.json: {where}.router.groups: {count} groups must divide the {experts} "
                              f"experts and keep {keep} of them at most")
    if top > keep * (experts // count):
        raise ConfigError(f"config.json: {where}.router.top {top} exceeds the {keep * (experts // count)} "
                          "experts that can be chosen")
    return GroupedRouterFfnConfig(
        ff=_need(ex, "ff", where + ".expert"), limit=_need(ex, "limit", where + ".expert", float),
        experts=experts, top=top,
        scale=_need(ro, "scale", where + ".router", float) if ro.get("scale") is not None else 1.0,
        group_count=count, group_keep=keep)


def fill_from_tensor_shapes(cfg: FobanexConfig, shapes: Dict[str, Tuple[int, ...]]) -> FobanexConfig:
    """Sizes the file leaves to the checkpoint's tensor shapes: the rank of a layer's query
    latent (``l<i>.mix.dq`` is [q_rank, width])."""
    layers = list(cfg.layers)
    for i, layer in enumerate(layers):
        mx = layer.mixer
        if isinstance(mx, QueryLatentAttentionConfig) and mx.q_rank is None:
            dq = shapes.get(f"l{i}.mix.dq")
            if dq is None or len(dq) != 2:
                raise ConfigError(f"config.json: layers[{i}].mixer has no 'q_rank' and the checkpoint no "
                                  f"matrix 'l{i}.mix.dq'")
            layers[i] = replace(layer, mixer=replace(mx, q_rank=int(dq[0])))
    return replace(cfg, layers=tuple(layers))
