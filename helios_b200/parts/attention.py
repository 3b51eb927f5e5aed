"""Grouped-query attention over the paged cache
(python/helios/exec/model.py:156-251; math of python/helios/exec/paged_attn.py:264-408).

One fused projection gives q, k and v (+ bias where the configuration has one);
one kernel rotates q and k and writes k and v into the request's pages before
attending, so a portion of a prompt sees itself (model.py:203-206); attention
runs over the cache for every token of the batch, whatever mix of prompt
portions and single decoded tokens it is; then the output projection.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..csrc import ops
from .base import DeferredNorm, LayerCache, Mixer, PagedCacheSpec, WeightSpec, register_part
from .norm import RMSNorm


class GQAAttention(Mixer):
    def __init__(self, width: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 scale: float, qkv_bias: bool, window: Optional[int] = None,
                 rotary: bool = True, position=None) -> None:
        """``position``: the encoding whose cos/sin tables rotate q and k (its
        ``tables(ctx)``); None takes the tables the plan's own encoding left on the step
        context.  ``rotary=False``: no rotation at all."""
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} query heads are not a multiple of {num_kv_heads} KV heads")
        if head_dim % 2 or head_dim > 256:
            raise ValueError(f"head_dim {head_dim} is not supported (even, at most 256)")
        self.width = width
        self.num_heads = num_heads
        self.num_kv_heads = num_kv_heads
        self.head_dim = head_dim
        self.scale = float(scale)
        self.qkv_bias = qkv_bias
        self.window = window
        self.rotary = rotary
        self.position = position
        self.w_qkv = self.b_qkv = self.w_o = None

    # ---------------------------------------------------------------- what it keeps
    def cache_spec(self) -> PagedCacheSpec:
        return PagedCacheSpec(self.num_kv_heads, self.head_dim, self.window)

    def kernel_libraries(self, dtype):
        return (ops.linear_libraries(dtype, self.width)
                + ops.attention_libraries(dtype, self.num_heads, self.num_kv_heads, self.head_dim))

    # ---------------------------------------------------------------- tensors
    def weight_specs(self) -> Dict[str, WeightSpec]:
        q, kv = self.num_heads * self.head_dim, self.num_kv_heads * self.head_dim
        specs = {
            "q_proj.weight": WeightSpec((q, self.width)),
            "k_proj.weight": WeightSpec((kv, self.width)),
            "v_proj.weight": WeightSpec((kv, self.width)),
            "o_proj.weight": WeightSpec((self.width, q)),
        }
        if self.qkv_bias:
            specs["q_proj.bias"] = WeightSpec((q,), kind="vector", init="normal")
            specs["k_proj.bias"] = WeightSpec((kv,), kind="vector", init="normal")
            specs["v_proj.bias"] = WeightSpec((kv,), kind="vector", init="normal")
        return specs

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.w_qkv = torch.cat([tensors["q_proj.weight"], tensors["k_proj.weight"],
                                tensors["v_proj.weight"]], dim=0).contiguous()
        self.w_o = tensors["o_proj.weight"].contiguous()
        if self.qkv_bias:
            self.b_qkv = torch.cat([tensors["q_proj.bias"], tensors["k_proj.bias"],
                                    tensors["v_proj.bias"]], dim=0).contiguous()

    # ---------------------------------------------------------------- forward
    def _rotary_tables(self, ctx):
        if not self.rotary:
            return None, None
        if self.position is not None:
            return self.position.tables(ctx)
        return ctx.rotary_cos, ctx.rotary_sin

    def forward_from_residual(self, ctx, residual: torch.Tensor, norm, cache: LayerCache, state=None,
                              pre=None, then=None):
        """Steps of few tokens run without norm launches: q|k|v takes the 1 / rms of ``pre``
        as a factor on its accumulators (the norm kernel runs where nothing was handed over),
        and the output projection adds into the residual and leaves ``then`` all but done."""
        if ctx.act_dtype != torch.bfloat16 or type(norm) is not RMSNorm or cache is None \
                or not ops.deferred_norm_fits(ctx.num_tokens, self.w_qkv, self.w_o):
            return False
        if pre is not None:
            qkv = ops.linear_bf16(pre.scaled, self.w_qkv, self.b_qkv, sumsq=pre.sumsq, eps=norm.eps)
        else:
            qkv = ops.linear_bf16(norm.add_forward(residual, None, ctx.act_dtype), self.w_qkv, self.b_qkv)
        attn = self._attend(ctx, qkv, cache)
        if type(then) is RMSNorm:
            scaled, sumsq = ops.linear_bf16(attn, self.w_o, residual=residual, norm_weight=then.weight)
            return DeferredNorm(then, scaled, sumsq)
        ops.linear_bf16(attn, self.w_o, residual=residual)
        return True

    def _attend(self, ctx, qkv: torch.Tensor, cache: LayerCache) -> torch.Tensor:
        table = ctx.block_tables[cache.group]
        cos, sin = self._rotary_tables(ctx)
        return ops.attention(ctx, qkv, cache.k_pages, cache.v_pages, table, self.num_heads,
                             self.num_kv_heads, self.head_dim, cache.page_size, self.window,
                             self.scale, fresh=(cos, sin, cache.write))

    def forward(self, ctx, x: torch.Tensor, cache: LayerCache, state=None) -> torch.Tensor:
        return ops.linear(self._attend(ctx, ops.linear(x, self.w_qkv, self.b_qkv), cache), self.w_o)


register_part("mixer", "gqa_attention", GQAAttention)


def distance_slopes(num_heads: int, exponent: float = 8.0):
    """Slope of head h = 2 ^ (-exponent * (h + 1) / heads): the geometric sequence a linear
    distance bias on the scores usually takes."""
    return [2.0 ** (-exponent * (h + 1) / num_heads) for h in range(num_heads)]


class SinkGQAAttention(Mixer):
    """Grouped-query attention whose score may carry the position, with a sink in the softmax:

        q = norm_q(W_q h) * temp(p),   k = norm_k(W_k h),   v = W_v h
        s_ij = q_i . k_j * scale - slope_h * (i - j)              (j <= i)
        p_ij = exp(s_ij) / (1 + sum_j exp(s_ij))                  (``sink``: a key of score 0 without a value)
        out  = W_o concat_h(sigmoid(W_g h)_h * sum_j p_ij v_j)    (``head_gate``: one number a head)

    norm_q / norm_k: RMS norm over a head's ``head_dim`` values with one weight shared by all
    heads (``qk_norm``); temp(p) = 1 + coef * ln(floor((p + 1) / every) + 1)
    (``q_temperature`` = (coef, every) or None); slope_h from ``slopes`` (a list, one a head, or
    None).  Values may have another size than keys (``value_dim``).  Every option can be left
    out; the constants are the caller's.  One fused projection gives q | k | v | gate; q and
    k are normed and k and v written into the request's pages by one launch before attention,
    or, in steps of single tokens, inside the decode kernel; the gate is applied where
    attention writes its output.

    Further options, each off by default:

    ``values="keys"``     there is no W_v: v_j = W_k h_j (+ bias) as projected, before any
                          rotation or norm of the key
    ``qk_norm="plain"``   q and k are divided by their root mean square without a weight
    ``qk_norm="row"``     the RMS norm runs over the WHOLE query projection and the whole key
                          projection (all heads at once, weights of those sizes), and BEFORE the
                          rotation
    ``position``, ``rotary_dim``  q and k are rotated BEFORE their norm by the tables of this
                          encoding, on the first ``rotary_dim`` values of a head, value i paired
                          with value i + rotary_dim / 2 (``rotary_pairing="halves"``) or value 2i
                          with value 2i + 1 ("neighbours")
    ``distance_table``    (rows, far): a learned bias ``rel`` [rows, heads] by the distance i - j,
                          looked up through ``ops.distance_bias_rows``
    ``sink="learned"``    the sink's score is a learned number a head (tensor ``sink``) instead of 0
    ``keep_first``        with ``window``: the request's first ``keep_first`` tokens stay visible
    ``head_gate="wide"``  W_g has a row per output VALUE, and every value its own gate
    ``qk_bias``, ``out_bias``  biases of the q and k projections (and v, where it exists) and of
                          the output projection (``<name>.b``)
    """

    def __init__(self, width: int, num_heads: int, num_kv_heads: int, head_dim: int, scale: float,
                 value_dim: Optional[int] = None, qk_norm=True, eps: float = 1e-6,
                 q_temperature=None, slopes=None, sink=True, head_gate=True,
                 window: Optional[int] = None,
                 names=("q", "k", "v", "o", "g", "q.norm", "k.norm"), values: str = "projected",
                 position=None, rotary_dim: int = 0, distance_table=None, keep_first: int = 0,
                 qk_bias: bool = False, out_bias: bool = False, rel_name: str = "rel",
                 sink_name: str = "sink", bias_suffix: str = ".b", rotary_pairing: str = "halves") -> None:
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} query heads are not a multiple of {num_kv_heads} KV heads")
        value_dim = value_dim or head_dim
        if not 0 < head_dim <= 256 or not 0 < value_dim <= 256:
            raise ValueError(f"heads of {head_dim} / {value_dim} values are not supported (at most 256)")
        if slopes is not None and len(slopes) != num_heads:
            raise ValueError(f"{len(slopes)} slopes for {num_heads} heads")
        if values not in ("projected", "keys") or qk_norm not in (True, False, "plain", "row") \
                or sink not in (True, False, "learned") or head_gate not in (True, False, "wide") \
                or rotary_pairing not in ops.ROTARY_PAIRINGS:
            raise ValueError(f"values {values!r} / qk_norm {qk_norm!r} / sink {sink!r} / head_gate {head_gate!r} "
                             f"/ rotary_pairing {rotary_pairing!r}")
        if values == "keys" and value_dim != head_dim:
            raise ValueError("values that are the keys have the keys' size")
        if (position is None) != (not rotary_dim) or rotary_dim % 2 or rotary_dim > head_dim:
            raise ValueError(f"a rotation needs an encoding and an even rotary_dim of at most {head_dim}")
        if keep_first and not window:
            raise ValueError("first tokens are kept beside a window only")
        self.width, self.num_heads, self.num_kv_heads = width, num_heads, num_kv_heads
        self.head_dim, self.value_dim = head_dim, value_dim
        self.scale, self.eps = float(scale), float(eps)
        self.qk_norm, self.sink, self.head_gate = qk_norm, sink, head_gate
        self.q_temperature = None if not q_temperature else (float(q_temperature[0]), int(q_temperature[1]))
        self.slope_values = None if slopes is None else [float(x) for x in slopes]
        self.window = window
        self.names = tuple(names)
        self.values, self.position, self.rotary_dim = values, position, int(rotary_dim)
        self.rotary_pairing = rotary_pairing
        self.distance_table = None if distance_table is None else (int(distance_table[0]), float(distance_table[1]))
        self.keep_first = int(keep_first or 0)
        self.qk_bias, self.out_bias = bool(qk_bias), bool(out_bias)
        self.rel_name, self.sink_name, self.bias_suffix = rel_name, sink_name, bias_suffix
        self.w_in = self.b_in = self.w_o = self.b_o = self.q_weight = self.k_weight = self.slopes = None
        self.bias_rows = self.bias_rows_t = self.sink_values = None
        q, kv = num_heads * head_dim, num_kv_heads * head_dim
        self._value_col = q + kv if values == "projected" else None
        self._gate_col = q + kv + (num_kv_heads * value_dim if values == "projected" else 0)
        # the launch that readies q, k and v: the one with weights and temperature, or the one
        # that also rotates, norms without weights and may take the values from the keys
        self._rotate_prepare = values == "keys" or position is not None or qk_norm in ("plain", "row")
        if self._rotate_prepare and self.q_temperature is not None:
            raise ValueError("a query temperature goes with weighted q/k norms and projected values only")
        self._tiled_options = value_dim == head_dim

    # ---------------------------------------------------------------- what it keeps
    def cache_spec(self) -> PagedCacheSpec:
        vd = None if self.value_dim == self.head_dim else self.value_dim
        return PagedCacheSpec(self.num_kv_heads, self.head_dim, self.window, value_dim=vd,
                              keep_first=self.keep_first)

    def kernel_libraries(self, dtype):
        return ops.linear_libraries(dtype, self.width) + ops.option_attention_libraries(
            dtype, self.num_heads, self.num_kv_heads, self.head_dim, self.value_dim,
            tiled=self._tiled_options)

    # ---------------------------------------------------------------- tensors
    def weight_specs(self) -> Dict[str, WeightSpec]:
        nq, nk, nv, no, ng, nqn, nkn = self.names
        q, kv = self.num_heads * self.head_dim, self.num_kv_heads * self.head_dim
        specs = {nq: WeightSpec((q, self.width)), nk: WeightSpec((kv, self.width)),
                 no: WeightSpec((self.width, self.num_heads * self.value_dim))}
        if self.values == "projected":
            specs[nv] = WeightSpec((self.num_kv_heads * self.value_dim, self.width))
        if self.head_gate:
            rows = self.num_heads * (self.value_dim if self.head_gate == "wide" else 1)
            specs[ng] = WeightSpec((rows, self.width))
        if self.qk_norm is True:
            specs[nqn] = WeightSpec((self.head_dim,), kind="vector", init="ones_jitter")
            specs[nkn] = WeightSpec((self.head_dim,), kind="vector", init="ones_jitter")
        elif self.qk_norm == "row":
            specs[nqn] = WeightSpec((q,), kind="vector", init="ones_jitter")
            specs[nkn] = WeightSpec((kv,), kind="vector", init="ones_jitter")
        if self.qk_bias:
            for n in (nq, nk) + ((nv,) if self.values == "projected" else ()):
                specs[n + self.bias_suffix] = WeightSpec((specs[n].shape[0],), kind="vector", init="normal")
        if self.out_bias:
            specs[no + self.bias_suffix] = WeightSpec((self.width,), kind="vector", init="normal")
        if self.distance_table is not None:
            specs[self.rel_name] = WeightSpec((self.distance_table[0], self.num_heads), kind="vector",
                                              init="normal", std=0.5)
        if self.sink == "learned":
            specs[self.sink_name] = WeightSpec((self.num_heads,), kind="vector", init="normal", std=0.5)
        return specs

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        nq, nk, nv, no, ng, nqn, nkn = self.names
        order = [nq, nk] + ([nv] if self.values == "projected" else [])
        mats = [tensors[n] for n in order]
        if self.head_gate:
            mats.append(tensors[ng])
        rows = sum(m.shape[0] for m in mats)
        pad = -rows % 8            # rows of the fused projection's output stay 16-byte aligned
        if pad:
            mats.append(torch.zeros((pad, self.width), dtype=mats[0].dtype, device=mats[0].device))
        self.w_in = torch.cat(mats, dim=0).contiguous()
        self.w_o = tensors[no].contiguous()
        if self.qk_bias:
            biases = [tensors[n + self.bias_suffix].float() for n in order]
            rest = self.w_in.shape[0] - sum(b.numel() for b in biases)
            biases.append(torch.zeros((rest,), dtype=torch.float32, device=self.w_in.device))
            self.b_in = torch.cat(biases).contiguous()
        if self.out_bias:
            self.b_o = tensors[no + self.bias_suffix].contiguous()
        if self.qk_norm in (True, "row"):
            self.q_weight, self.k_weight = tensors[nqn].contiguous(), tensors[nkn].contiguous()
        if self.slope_values is not None:
            self.slopes = torch.tensor(self.slope_values, dtype=torch.float32, device=self.w_o.device)
        if self.distance_table is not None:
            self.bias_rows = ops.distance_bias_rows(tensors[self.rel_name], self.distance_table[1], self.window)
            self.bias_rows_t = self.bias_rows.t().contiguous()      # what the tcgen05 kernel reads
        if self.sink == "learned":
            self.sink_values = tensors[self.sink_name].contiguous()

    # ---------------------------------------------------------------- forward
    def _options(self, gate) -> "ops.AttentionOptions":
        return ops.AttentionOptions(slopes=self.slopes, sink=bool(self.sink), gate=gate,
                                    value_dim=None if self.value_dim == self.head_dim else self.value_dim,
                                    bias_table=self.bias_rows, sink_values=self.sink_values,
                                    keep_first=self.keep_first, gate_wide=self.head_gate == "wide",
                                    bias_table_t=self.bias_rows_t)

    def forward(self, ctx, x: torch.Tensor, cache: LayerCache, state=None) -> torch.Tensor:
        rows = ops.linear(x, self.w_in, self.b_in)
        table = ctx.block_tables[cache.group]
        gate = None
        if self.head_gate:
            n = self.num_heads * (self.value_dim if self.head_gate == "wide" else 1)
            gate = rows[:, self._gate_col:self._gate_col + n]
        if self._rotate_prepare:
            cos, sin = self.position.tables(ctx) if self.position is not None else (None, None)
            prepare = ops.RotateNormPrepare(cos, sin, "row" if self.qk_norm == "row" else bool(self.qk_norm),
                                            self.q_weight, self.k_weight, self.eps, self._value_col,
                                            cache.write, pairing=self.rotary_pairing)
        else:
            coef, every = self.q_temperature or (0.0, 0)
            prepare = (self.q_weight, self.k_weight, self.eps, coef, every, cache.write)
        attn = ops.attention(ctx, rows, cache.k_pages, cache.v_pages, table, self.num_heads,
                             self.num_kv_heads, self.head_dim, cache.page_size, self.window, self.scale,
                             options=self._options(gate), prepare=prepare)
        return ops.linear(attn, self.w_o, self.b_o)


register_part("mixer", "sink_gqa_attention", SinkGQAAttention)
