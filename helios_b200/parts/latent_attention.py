"""Attention over a low-rank latent cache.

Per token the mixer keeps ONE row: the latent c (``rank`` values, RMS-normed) and a rotated
key part r (``rot`` values) that all heads share.  Head h's key is [W_uk[h] c | r] and its
value W_uv[h] c; a query is [q_nope (``nope`` values) | q_rot (``rot`` values, rotated)] and

    score = (q_nope . W_uk[h] c + q_rot . r) * scale,     softmax over the positions <= own.

The up-projections are folded into the query and the output, so that the cache is never
expanded: q_lat = W_uk[h]^T q_nope attends the latents themselves, and the head's output is
W_uv[h] (sum_j p_j c_j).  Rotary pairs dimension 2i with 2i + 1 over the first
``position.rotary_dim`` of the ``rot`` values.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..csrc import ops
from .base import LayerCache, Mixer, PagedCacheSpec, WeightSpec, register_part


class LatentAttention(Mixer):
    """Options, each off by default:

    ``q_rank``      the queries go through a latent of their own: c_q = RMSnorm(W_dq h) (weight
                    ``dq.norm``, the mixer's eps), q = W_uq c_q; there is no direct query matrix
    ``pairing``     "neighbours": value 2i of a rotated part is paired with value 2i + 1;
                    "halves": value i with value i + rotary_dim / 2
    ``gate``        the concatenated heads are multiplied by sigmoid(W_g h), value by value,
                    before the output projection
    ``own_rows``    False: the mixer has no W_dkv and keeps nothing; it attends the rows that
                    ANOTHER layer keeps (the plan names that layer's cache for this one's run),
                    with up-projections, queries and everything else of its own
    """

    def __init__(self, width: int, heads: int, nope: int, rot: int, vdim: int, rank: int,
                 scale: float, eps: float, position,
                 names=("q", "dkv", "dkv.norm", "uk", "uv", "o"), q_rank: Optional[int] = None,
                 pairing: str = "neighbours", gate: bool = False, own_rows: bool = True,
                 query_names=("dq", "dq.norm", "uq"), gate_name: str = "g") -> None:
        """``position``: the rotary encoding whose tables rotate the ``rot`` parts
        (``position.rotary_dim`` <= rot, even).  ``scale`` multiplies the scores as given.
        ``eps``: of the latents' RMS norms."""
        if position.rotary_dim > rot:
            raise ValueError(f"{position.rotary_dim} rotated dimensions exceed the rotated part of {rot}")
        if pairing not in ops.ROTARY_PAIRINGS:
            raise ValueError(f"pairing {pairing!r} is not one of {sorted(ops.ROTARY_PAIRINGS)}")
        self.width, self.heads, self.nope, self.rot = width, heads, nope, rot
        self.vdim, self.rank = vdim, rank
        self.scale, self.eps = float(scale), float(eps)
        self.position = position
        self.names = tuple(names)
        self.q_rank = int(q_rank) if q_rank else None
        self.pairing, self.gate, self.own_rows = pairing, bool(gate), bool(own_rows)
        self.query_names, self.gate_name = tuple(query_names), gate_name
        self.w_in = self.w_uq = self.w_uk_t = self.w_uv = self.w_o = None
        self.norm_weight = self.query_norm_weight = None
        # columns of the fused first projection: [queries or their latent | latent rows | gate]
        self._n_first = self.q_rank or heads * (nope + rot)
        self._lat_col = self._n_first
        self._gate_col = self._lat_col + (rank + rot if self.own_rows else 0)

    def cache_spec(self) -> PagedCacheSpec:
        return PagedCacheSpec(1, self.rank + self.rot, None, planes=1)

    def kernel_libraries(self, dtype):
        return ops.linear_libraries(dtype, self.width) + ("latent_attention",) \
            + (("elementwise",) if self.gate else ())

    def weight_specs(self) -> Dict[str, WeightSpec]:
        q, dkv, norm, uk, uv, o = self.names
        H = self.heads
        specs = {
            uk: WeightSpec((H * self.nope, self.rank)),
            uv: WeightSpec((H * self.vdim, self.rank)),
            o: WeightSpec((self.width, H * self.vdim)),
        }
        if self.q_rank:
            dq, dq_norm, uq = self.query_names
            specs[dq] = WeightSpec((self.q_rank, self.width))
            specs[dq_norm] = WeightSpec((self.q_rank,), kind="vector", init="ones_jitter")
            specs[uq] = WeightSpec((H * (self.nope + self.rot), self.q_rank))
        else:
            specs[q] = WeightSpec((H * (self.nope + self.rot), self.width))
        if self.own_rows:
            specs[dkv] = WeightSpec((self.rank + self.rot, self.width))
            specs[norm] = WeightSpec((self.rank,), kind="vector", init="ones_jitter")
        if self.gate:
            specs[self.gate_name] = WeightSpec((H * self.vdim, self.width))
        return specs

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        q, dkv, norm, uk, uv, o = self.names
        H = self.heads
        mats = [tensors[self.query_names[0]] if self.q_rank else tensors[q]]
        if self.own_rows:
            mats.append(tensors[dkv])
            self.norm_weight = tensors[norm].contiguous()
        if self.gate:
            mats.append(tensors[self.gate_name])
        if len(mats) > 1:
            pad = -sum(m.shape[0] for m in mats) % 8     # output rows stay 16-byte aligned
            if pad:
                mats.append(torch.zeros((pad, self.width), dtype=mats[0].dtype, device=mats[0].device))
        self.w_in = torch.cat(mats, dim=0).contiguous()
        if self.q_rank:
            self.query_norm_weight = tensors[self.query_names[1]].contiguous()
            self.w_uq = tensors[self.query_names[2]].contiguous()
        # [heads, rank, nope]: the matrix that takes a head's q_nope to the latent space
        self.w_uk_t = tensors[uk].view(H, self.nope, self.rank).transpose(1, 2).contiguous()
        self.w_uv = tensors[uv].view(H, self.vdim, self.rank).contiguous()
        self.w_o = tensors[o].contiguous()

    def forward(self, ctx, x: torch.Tensor, cache: LayerCache, state=None) -> torch.Tensor:
        H, T = self.heads, x.shape[0]
        proj = ops.linear(x, self.w_in)
        cos, sin = self.position.tables(ctx)
        table = ctx.block_tables[cache.group]
        first = proj[:, :self._n_first]
        latent = proj[:, self._lat_col:self._lat_col + self.rank + self.rot] if self.own_rows else None

        def prepare(q, lat, query_latent, out=None):
            ops.latent_prepare_parts(q, lat, query_latent, cache.k_pages, self.norm_weight,
                                     self.query_norm_weight, cos, sin, ctx.positions, ctx.seq_of_token,
                                     table, H, self.nope, self.rot, self.rank, cache.page_size, self.eps,
                                     write_cache=cache.write and self.own_rows, pairing=self.pairing,
                                     query_latent_out=out)

        if self.q_rank:
            # the query latent normed into rows of its own (the product that follows wants
            # contiguous rows), the latent rows stored
            cq = torch.empty((T, self.q_rank), dtype=proj.dtype, device=proj.device)
            prepare(None, latent, first, cq)
            q = ops.linear(cq, self.w_uq)
            prepare(q, None, None)
        else:
            q = first
            prepare(q, latent, None)
        q = q.view(T, H, self.nope + self.rot) if q.is_contiguous() else \
            q.unflatten(1, (H, self.nope + self.rot))
        q_lat = ops.head_gemm(q[:, :, :self.nope], self.w_uk_t)
        o_lat = ops.latent_attention(ctx, q_lat, q[:, :, self.nope:], cache.k_pages, table,
                                     self.rank, self.rot, cache.page_size, self.scale)
        o = ops.head_gemm(o_lat, self.w_uv)
        if self.gate:          # the gate's launch also lays the heads side by side, whatever the product's strides
            o = ops.gate_heads(o, proj[:, self._gate_col:self._gate_col + H * self.vdim])
        else:
            o = o.reshape(T, H * self.vdim)
        return ops.linear(o, self.w_o)


register_part("mixer", "latent_attention", LatentAttention)
