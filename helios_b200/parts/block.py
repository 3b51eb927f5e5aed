"""Pre-norm residual block (python/helios/exec/model.py:340-392):
x + mixer(norm(x)), then x + feed_forward(norm(x)).

The residual stream is float32.  A block receives the stream and the output of
the part before that is still to be added; the add is fused into the next norm.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch

from .base import (Block, DeferredNorm, FeedForward, LayerCache, Mixer, Norm, Part, PendingSum, WeightSpec,
                   register_part)


class PreNormBlock(Block):
    def __init__(self, mixer_norm: Norm, mixer: Mixer, ffn_norm: Norm, ffn: FeedForward,
                 names: Tuple[str, str, str, str] = ("input_layernorm.", "self_attn.",
                                                     "post_attention_layernorm.", "mlp.")) -> None:
        self.mixer_norm = mixer_norm
        self._mixer = mixer
        self.ffn_norm = ffn_norm
        self.ffn = ffn
        self.names = names

    @property
    def mixer(self) -> Mixer:
        return self._mixer

    def named_parts(self) -> List[Tuple[str, Part]]:
        return list(zip(self.names, (self.mixer_norm, self._mixer, self.ffn_norm, self.ffn)))

    @property
    def graph_safe(self) -> bool:
        return all(p.graph_safe for _, p in self.named_parts())

    @property
    def first_norm(self) -> Norm:
        return self.mixer_norm

    def forward(self, ctx, residual: torch.Tensor, delta, cache: Optional[LayerCache],
                state: Optional[torch.Tensor]):
        # A part may take the norm before it and the add after it into its own kernels (steps
        # of few tokens); that needs a residual stream to which nothing is pending.  Such a
        # part may also leave the NEXT norm all but done (a DeferredNorm) for the part after it.
        pre = None
        if isinstance(delta, DeferredNorm):
            pre, delta = (delta if delta.norm is self.mixer_norm else None), None
        done = False
        if delta is None:
            done = self._mixer.forward_from_residual(ctx, residual, self.mixer_norm, cache, state,
                                                     pre=pre, then=self.ffn_norm)
        if done is False:
            x = self.mixer_norm.add_forward(residual, delta, ctx.act_dtype)
            delta = self._mixer.forward(ctx, x, cache, state)
        else:
            delta = None
            done = self.ffn.forward_from_residual(ctx, residual, self.ffn_norm,
                                                  pre=done if isinstance(done, DeferredNorm) else None,
                                                  then=ctx.norm_after_block)
            if done is not False:
                return residual, (done if isinstance(done, DeferredNorm) else None)
        x = self.ffn_norm.add_forward(residual, delta, ctx.act_dtype)
        return residual, self.ffn.forward(ctx, x)


register_part("block", "pre_norm", PreNormBlock)


class PostNormBlock(Block):
    """x + norm(mixer(x)), then x + norm(feed_forward(x)): the norm sits on a sublayer's
    OUTPUT, and the sublayers read the residual stream itself (in the activation dtype).
    The feed-forward, with its norm, may be absent.  The residual sum and the norms are
    float32; each add is one kernel with its norm, which also leaves the new residual in the
    activation dtype for the next sublayer (kept for the next block of this kind under the
    index of the run that made it)."""

    _COPY = "post_norm_block.residual_copy"

    def __init__(self, mixer: Mixer, mixer_norm: Norm, ffn: Optional[FeedForward] = None,
                 ffn_norm: Optional[Norm] = None,
                 names: Tuple[str, str, str, str] = ("mix.", "norm1", "mlp.", "norm2")) -> None:
        if (ffn is None) != (ffn_norm is None):
            raise ValueError("a feed-forward and its norm come together")
        self._mixer = mixer
        self.mixer_norm = mixer_norm
        self.ffn = ffn
        self.ffn_norm = ffn_norm
        self.names = names

    @property
    def mixer(self) -> Mixer:
        return self._mixer

    def named_parts(self) -> List[Tuple[str, Part]]:
        parts = [(self.names[0], self._mixer), (self.names[1], self.mixer_norm)]
        if self.ffn is not None:
            parts += [(self.names[2], self.ffn), (self.names[3], self.ffn_norm)]
        return parts

    @property
    def graph_safe(self) -> bool:
        return all(p.graph_safe for _, p in self.named_parts())

    def forward(self, ctx, residual: torch.Tensor, delta, cache: Optional[LayerCache],
                state: Optional[torch.Tensor]):
        if isinstance(delta, DeferredNorm):
            raise ValueError("a post-norm block takes no deferred norm")
        kept = ctx.step_tables.pop(self._COPY, None)
        if delta is not None:
            residual.add_(delta.float())
            kept = None
        if kept is not None and kept[0] == ctx.run_index - 1:
            h = kept[1]
        else:
            h = self.mixer_norm.add_normed(residual, None, ctx.act_dtype) \
                if ctx.act_dtype != torch.float32 else residual
        h = self.mixer_norm.add_normed(residual, self._mixer.forward(ctx, h, cache, state), ctx.act_dtype)
        if self.ffn is not None:
            h = self.ffn_norm.add_normed(residual, self.ffn.forward(ctx, h), ctx.act_dtype)
        ctx.step_tables[self._COPY] = (ctx.run_index, h)
        return residual, None


register_part("block", "post_norm", PostNormBlock)


class ChannelScale(Part):
    """A learned factor per channel on a sublayer's output (float32 in both modes)."""

    def __init__(self, width: int, tensor_name: str = "") -> None:
        self.width, self.tensor_name = width, tensor_name
        self.scale: Optional[torch.Tensor] = None

    def weight_specs(self):
        return {self.tensor_name: WeightSpec((self.width,), kind="vector", init="ones_jitter")}

    def bind(self, tensors) -> None:
        self.scale = tensors[self.tensor_name].contiguous()


class ParallelBlock(Block):
    """x + mult * (ls1 * mixer(h) + ls2 * feed_forward(h)) with h = norm(x): ONE norm, and both
    sublayers read its output.  ``ls1`` / ``ls2`` are learned per-channel factors
    (``layer_scale``; without it they are 1); the feed-forward may be absent.  The sum is not
    formed here: the block returns its outputs as a ``PendingSum``, and the norm that meets the
    stream next adds them in float32 in its own kernel.

    With ``ffn_norm`` the feed-forward reads a norm of its own of the SAME stream,
    x + mult * (ls1 * mixer(norm(x)) + ls2 * feed_forward(ffn_norm(x))); two RMS norms share the
    row's 1 / rms and run, with the add that was pending, as one kernel (``RMSNorm.add_forward_pair``)."""

    def __init__(self, norm: Norm, mixer: Mixer, ffn: Optional[FeedForward] = None, mult: float = 1.0,
                 layer_scale: bool = True, names: Tuple[str, str, str, str, str] =
                 ("norm1", "mix.", "mlp.", "ls1", "ls2"), ffn_norm: Optional[Norm] = None,
                 ffn_norm_name: str = "norm2") -> None:
        if ffn_norm is not None and ffn is None:
            raise ValueError("a second norm needs a feed-forward to read it")
        self.norm = norm
        self.ffn_norm, self.ffn_norm_name = ffn_norm, ffn_norm_name
        self._mixer = mixer
        self.ffn = ffn
        self.mult = float(mult)
        self.names = names
        width = getattr(norm, "width")
        self.mixer_scale = ChannelScale(width) if layer_scale else None
        self.ffn_scale = ChannelScale(width) if layer_scale and ffn is not None else None

    @property
    def mixer(self) -> Mixer:
        return self._mixer

    def named_parts(self) -> List[Tuple[str, Part]]:
        n_norm, n_mix, n_ffn, n_ls1, n_ls2 = self.names
        parts = [(n_norm, self.norm), (n_mix, self._mixer)]
        if self.ffn is not None:
            parts.append((n_ffn, self.ffn))
        if self.ffn_norm is not None:
            parts.append((self.ffn_norm_name, self.ffn_norm))
        if self.mixer_scale is not None:
            parts.append((n_ls1, self.mixer_scale))
        if self.ffn_scale is not None:
            parts.append((n_ls2, self.ffn_scale))
        return parts

    @property
    def graph_safe(self) -> bool:
        return all(p.graph_safe for _, p in self.named_parts())

    def forward(self, ctx, residual: torch.Tensor, delta, cache: Optional[LayerCache],
                state: Optional[torch.Tensor]):
        if isinstance(delta, DeferredNorm):
            raise ValueError("a parallel block takes no deferred norm")
        if self.ffn_norm is None:
            h = h2 = self.norm.add_forward(residual, delta, ctx.act_dtype)
        elif hasattr(self.norm, "add_forward_pair"):
            h, h2 = self.norm.add_forward_pair(residual, delta, self.ffn_norm, ctx.act_dtype)
        else:
            h = self.norm.add_forward(residual, delta, ctx.act_dtype)
            h2 = self.ffn_norm.add_forward(residual, None, ctx.act_dtype)
        terms = [(self._mixer.forward(ctx, h, cache, state),
                  self.mixer_scale.scale if self.mixer_scale is not None else None)]
        if self.ffn is not None:
            terms.append((self.ffn.forward(ctx, h2),
                          self.ffn_scale.scale if self.ffn_scale is not None else None))
        return residual, PendingSum(terms, self.mult)


register_part("block", "parallel", ParallelBlock)
