"""Typed configuration of the Gebasun design, read from ``config.json``.

The file lists the layers one by one; every entry names its mixer by ``type`` (``attention``:
window attention with a learned bias by distance; ``attention_2``: window attention that also
keeps a request's first tokens, with rotary positions and a gate on every output value;
``mamba2``: a state-space recurrence) with the mixer's sizes, and its feed-forward (routed
experts, or null for none).  Two models of the design may differ in every size, in the order
of the layers and in every constant; nothing here has a default that stands for a value of
some particular model.  What the file leaves out of an optional piece (kept first tokens, the
shared expert, a layer's feed-forward) is absent.
"""
from __future__ import annotations

from dataclasses import dataclass, replace
from typing import Any, Dict, Optional, Tuple, Union

from .model_config import ConfigError
from .zokelix_config import _need


@dataclass(frozen=True)
class BiasAttentionConfig:
    """``attention``: the values are the projected keys; a bias table by distance."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int
    bias_max: float           # the distance from which the last row of the bias table serves
    bias_rows: Optional[int]  # rows of the bias table; None until read off the checkpoint's 'rel'


@dataclass(frozen=True)
class RotaryAttentionConfig:
    """``attention_2``: rotary positions on the first ``rot_dims`` values of a head."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int
    keep_first: int
    rot_dims: int
    rot_base: float


@dataclass(frozen=True)
class StateSpaceConfig:
    """``mamba2``."""
    heads: int
    vdim: int
    state: int
    groups: int
    conv: int
    norm_groups: int


@dataclass(frozen=True)
class RoutedFfnConfig:
    ff: int
    experts: int
    top: int
    shared_ff: Optional[int]


MixerConfig = Union[BiasAttentionConfig, RotaryAttentionConfig, StateSpaceConfig]


@dataclass(frozen=True)
class GebasunLayer:
    type: str
    mixer: MixerConfig
    mlp: Optional[RoutedFfnConfig]


@dataclass(frozen=True)
class GebasunConfig:
    architecture: str
    vocab_size: int
    width: int
    norm_eps: float
    layers: Tuple[GebasunLayer, ...]
    eos_token_ids: Tuple[int, ...] = ()

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    @property
    def max_position_embeddings(self) -> int:
        """No part of the design bounds a request's length."""
        return 1 << 30

    @classmethod
    def from_json(cls, cfg: Dict[str, Any]) -> "GebasunConfig":
        vocab = _need(cfg, "vocab", "the file")
        width = _need(cfg, "width", "the file")
        eps = _need(cfg.get("norm"), "eps", "norm", float)
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
            out.append(GebasunLayer(kind, reader(layer.get("mixer"), where + ".mixer"),
                                    _mlp(layer.get("mlp"), where + ".mlp")))
        eos = cfg.get("eos_token_id")
        eos_ids = () if eos is None else tuple(int(e) for e in (eos if isinstance(eos, (list, tuple)) else [eos]))
        return cls(architecture=str(cfg.get("architecture", "Gebasun")), vocab_size=vocab, width=width,
                   norm_eps=eps, layers=tuple(out), eos_token_ids=eos_ids)


def _heads(mx, where):
    heads, kv_heads = _need(mx, "heads", where), _need(mx, "kv_heads", where)
    if heads % kv_heads:
        raise ConfigError(f"config.json: {where}.kv_heads {kv_heads} must divide heads {heads}")
    dim, vdim = _need(mx, "dim", where), _need(mx, "vdim", where)
    if vdim != dim:
        raise ConfigError(f"config.json: {where}.vdim {vdim} differs from dim {dim}, but the values are "
                          "the projected keys")
    return heads, kv_heads, dim, vdim


def _count(d, key, where) -> int:
    """A count that may be 0 or absent."""
    v = d.get(key, 0) if isinstance(d, dict) else 0
    if v is None:
        return 0
    if not isinstance(v, int) or isinstance(v, bool) or v < 0:
        raise ConfigError(f"config.json: {where}.{key} must be a count, got {v!r}")
    return v


def _bias_attention(mx, where) -> BiasAttentionConfig:
    heads, kv_heads, dim, vdim = _heads(mx, where)
    return BiasAttentionConfig(heads, kv_heads, dim, vdim, _need(mx, "scale", where, float),
                               _need(mx.get("mask"), "size", where + ".mask"),
                               _need(mx, "bias_max", where, float),
                               _need(mx, "bias_rows", where) if mx.get("bias_rows") is not None else None)


def _rotary_attention(mx, where) -> RotaryAttentionConfig:
    heads, kv_heads, dim, vdim = _heads(mx, where)
    rot = mx.get("rot")
    dims = _need(rot, "dims", where + ".rot")
    if dims % 2 or dims > dim:
        raise ConfigError(f"config.json: {where}.rot.dims {dims} must be even and at most dim {dim}")
    mask = mx.get("mask")
    return RotaryAttentionConfig(heads, kv_heads, dim, vdim, _need(mx, "scale", where, float),
                                 _need(mask, "size", where + ".mask"),
                                 _count(mask, "keep_first", where + ".mask"), dims,
                                 _need(rot, "base", where + ".rot", float))


def _state_space(mx, where) -> StateSpaceConfig:
    heads, groups = _need(mx, "heads", where), _need(mx, "groups", where)
    if heads % groups:
        raise ConfigError(f"config.json: {where}.groups {groups} must divide heads {heads}")
    vdim, parts = _need(mx, "vdim", where), _need(mx, "norm_groups", where)
    if (heads * vdim) % parts:
        raise ConfigError(f"config.json: {where}.norm_groups {parts} must divide heads * vdim {heads * vdim}")
    return StateSpaceConfig(heads, vdim, _need(mx, "state", where), groups, _need(mx, "conv", where), parts)


_MIXERS = {"attention": _bias_attention, "attention_2": _rotary_attention, "mamba2": _state_space}


def _mlp(ml, where) -> Optional[RoutedFfnConfig]:
    if ml is None:
        return None
    kind = ml.get("kind") if isinstance(ml, dict) else None
    if kind != "moe":
        raise ConfigError(f"config.json: {where}.kind {kind!r} is not supported (moe)")
    ro = ml.get("router")
    experts, top = _need(ro, "experts", where + ".router"), _need(ro, "top", where + ".router")
    if top > experts:
        raise ConfigError(f"config.json: {where}.router.top {top} exceeds the {experts} experts")
    shared = ml.get("shared")
    return RoutedFfnConfig(ff=_need(ml.get("expert"), "ff", where + ".expert"), experts=experts, top=top,
                           shared_ff=_need(shared, "ff", where + ".shared") if shared else None)


def fill_from_tensor_shapes(cfg: GebasunConfig, shapes: Dict[str, Tuple[int, ...]]) -> GebasunConfig:
    """Sizes the file leaves to the checkpoint's tensor shapes: the rows of every distance-bias
    table (``l<i>.mix.rel`` is [rows, heads])."""
    layers = list(cfg.layers)
    for i, layer in enumerate(layers):
        mx = layer.mixer
        if isinstance(mx, BiasAttentionConfig) and mx.bias_rows is None:
            rel = shapes.get(f"l{i}.mix.rel")
            if rel is None or len(rel) != 2:
                raise ConfigError(f"config.json: layers[{i}].mixer has no 'bias_rows' and the checkpoint no "
                                  f"table 'l{i}.mix.rel'")
            layers[i] = replace(layer, mixer=replace(mx, bias_rows=int(rel[0])))
    return replace(cfg, layers=tuple(layers))
