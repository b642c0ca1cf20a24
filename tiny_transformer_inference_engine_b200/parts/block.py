"""Arrangement of a layer's parts.

``pre_norm`` is the reference's block (models/transformer_block.py:149-158):
``x = x + mixer(norm1(x))``, ``x = x + ffn(norm2(x))``.  The sums are formed in the
32-bit residual stream by the norm kernels: a sub-layer's output waits in
``stream.delta`` and the next norm adds it while normalising.  A layer without a
feed-forward (``ffn`` None) has only the first sub-layer.
"""
from __future__ import annotations

from typing import Optional

import torch

from .base import Block, ParamSpec, PartSpec, FixedStateNeed, ResidualStream, StepContext, mixer_cache_argument
from ..registry import register_part, build_part


@register_part("block", "pre_norm")
class PreNormBlock(Block):
    def __init__(self, prefix: str, mixer_norm: PartSpec, mixer: PartSpec, ffn_norm: PartSpec = None, ffn: PartSpec = None):
        super().__init__(prefix)
        self.mixer_norm = build_part("norm", mixer_norm)
        self.mixer = build_part("mixer", mixer)
        self.ffn_norm = build_part("norm", ffn_norm) if ffn is not None else None
        self.ffn = build_part("ffn", ffn) if ffn is not None else None

    def children(self):
        return [p for p in (self.mixer_norm, self.mixer, self.ffn_norm, self.ffn) if p is not None]

    def cache_needs(self):
        return self.mixer.cache_needs()                            # the feed-forward parts here keep nothing between steps

    def forward(self, stream: ResidualStream, ctx: StepContext, caches) -> None:
        h = self.mixer_norm.add_norm(stream.resid, stream.delta)
        a = self.mixer.forward(h, ctx, mixer_cache_argument(self.mixer, caches))
        if self.ffn is None:
            stream.delta = a
            return
        h = self.ffn_norm.add_norm(stream.resid, a)
        stream.delta = self.ffn.forward(h, ctx)


@register_part("block", "post_norm")
class PostNormBlock(Block):
    """Post-norm: ``x = LN_a(alpha * x + mixer(x))`` followed by ``x = LN_b(alpha * x + ffn(x))``; each sub-layer's input is
    the (already normalised) stream, not a normed copy of it.  The stream holds ``x`` in 32-bit; each norm kernel forms the scaled sum, normalises, rewrites the
    stream and hands the next sub-layer a copy in the compute dtype.  A layer without a feed-forward (``ffn`` None) ends
    after the first norm."""

    def __init__(self, prefix: str, mixer: PartSpec, mixer_norm: PartSpec, ffn, ffn_norm, alpha: float = 1.0):
        super().__init__(prefix)
        self.alpha = float(alpha)
        self.mixer = build_part("mixer", mixer)
        self.mixer_norm = build_part("norm", mixer_norm)
        self.ffn = build_part("ffn", ffn) if ffn is not None else None
        self.ffn_norm = build_part("norm", ffn_norm) if ffn is not None else None

    def children(self):
        return [p for p in (self.mixer, self.mixer_norm, self.ffn, self.ffn_norm) if p is not None]

    def cache_needs(self):
        return self.mixer.cache_needs()

    def forward(self, stream: ResidualStream, ctx: StepContext, caches) -> None:
        if stream.delta is not None:
            raise ValueError("a post-norm block cannot follow a block that leaves a sum unformed")
        x = stream.x
        if x is None:                                               # the first layer: the embedding's rows
            x = stream.resid if self.dtype == stream.resid.dtype else self.ops.cast_rows(stream.resid, self.dtype)
        a = self.mixer.forward(x, ctx, mixer_cache_argument(self.mixer, caches))
        x = self.mixer_norm.scale_add_norm(stream.resid, a, self.alpha)
        if self.ffn is not None:
            f = self.ffn.forward(x, ctx)
            x = self.ffn_norm.scale_add_norm(stream.resid, f, self.alpha)
        stream.x = x


@register_part("block", "sublayer_norm")
class SublayerNormBlock(Block):
    """The norm sits on each sub-layer's OUTPUT: ``x = x + norm_a(mixer(x))`` followed by ``x = x + norm_b(ffn(x))``; the
    sub-layers read the stream itself (a copy in the compute dtype that the norm kernel writes beside the 32-bit sum).  The
    norm parts carry a layer scale if the design has one (``LayerNorm(scale=)``).  A layer without a feed-forward (``ffn``
    None) ends after the first sum.

    ``input_conv`` (``name``, ``taps``; None: none): what the mixer reads is ``x + conv(x)``, a causal convolution over time on
    every channel, ``conv(x)_t = sum_j w[:, j] * x_(t - taps + 1 + j)`` with zeros before the sequence's start (tensor ``name``
    [dim, taps]; tap ``taps - 1`` multiplies the current token).  The ``x`` itself is one more on the last tap, added in 32-bit
    when the tensor is loaded; the kernel reads the 32-bit stream, and the last ``taps - 1`` stream rows of a request are kept
    in a state row of this block (the first of its cache needs), advanced by the convolution kernel itself in steps of one token
    per request and by a second kernel otherwise."""

    def __init__(self, prefix: str, dim: int, mixer: PartSpec, mixer_norm: PartSpec, ffn: PartSpec = None, ffn_norm: PartSpec = None,
                 input_conv: Optional[dict] = None):
        super().__init__(prefix)
        self.dim = int(dim)
        self.mixer = build_part("mixer", mixer)
        self.mixer_norm = build_part("norm", mixer_norm)
        self.ffn = build_part("ffn", ffn) if ffn is not None else None
        self.ffn_norm = build_part("norm", ffn_norm) if ffn is not None else None
        self.conv_name, self.taps = None, 0
        if input_conv is not None:
            self.conv_name, self.taps = input_conv["name"], int(input_conv["taps"])
            if self.taps < 1:
                raise ValueError(f"input_conv.taps must be >= 1, got {input_conv['taps']}")
        self.conv_w = None

    def children(self):
        return [p for p in (self.mixer, self.mixer_norm, self.ffn, self.ffn_norm) if p is not None]

    def param_specs(self):
        if self.conv_name is None:
            return {}
        return {self.conv_name: ParamSpec((self.dim, self.taps), storage="vector", init="normal", std=0.3)}

    def load(self, params):
        if self.conv_name is not None:                               # tap-major, 32-bit, the stream's own row on the last tap
            w = params[self.conv_name].float().t().contiguous()
            w[self.taps - 1] += 1.0
            self.conv_w = w

    def cache_needs(self):
        own = [FixedStateNeed((self.taps - 1, self.dim), "float32")] if self.taps > 1 else []
        return own + list(self.mixer.cache_needs())

    def forward(self, stream: ResidualStream, ctx: StepContext, caches) -> None:
        if stream.delta is not None:
            raise ValueError("a block that norms its sub-layers' outputs cannot follow a block that leaves a sum unformed")
        ops, resid = self.ops, stream.resid
        caches = list(caches)
        if self.conv_name is not None:
            tail = caches.pop(0) if self.taps > 1 else None
            state = None if tail is None else tail.state
            decode = ctx.max_q_len == 1 and tail is not None and tail.writable      # one token per request: the same kernel advances the state rows
            h = ops.stream_conv(resid, self.conv_w, self.taps, state, ctx.token_seq, ctx.query_start_loc, ctx.slot_ids, self.dtype,
                                update_tail=decode)
            if tail is not None and tail.writable and not decode:
                ops.conv_tail_update(resid, self.dim, self.taps, state, ctx.query_start_loc, ctx.slot_ids, ctx.num_seqs)
        else:
            h = stream.x
            if h is None:                                            # the first layer: the embedding's rows
                h = resid if self.dtype == resid.dtype else ops.cast_rows(resid, self.dtype)
        a = self.mixer.forward(h, ctx, mixer_cache_argument(self.mixer, caches))
        x = self.mixer_norm.add_normed(resid, a)
        if self.ffn is not None:
            x = self.ffn_norm.add_normed(resid, self.ffn.forward(x, ctx))
        stream.x = x
