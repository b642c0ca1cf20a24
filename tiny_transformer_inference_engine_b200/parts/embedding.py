"""Token embedding and output head.

Embedding (models/embedding.py:9-15): a row gather, no position term; the gathered row
(times ``scale``, a parameter; the reference has none) starts the 32-bit residual sum.  ``norm``
(a norm part's spec; the reference has none): the rows are normed in place before the first layer.  Head (models/transformer_block.py:170,181):
``logits = x @ W.T`` without bias, untied from the embedding; logits leave in 32-bit.
"""
from __future__ import annotations

import torch

from .base import Embedding, Head, ParamSpec, PartSpec, StepContext
from ..registry import register_part, build_part


@register_part("embedding", "token")
class TokenEmbedding(Embedding):
    def __init__(self, prefix: str, vocab_size: int, dim: int, name: str = "weight", scale: float = 1.0, norm: PartSpec = None):
        super().__init__(prefix)
        self.vocab_size, self.dim, self.name, self.scale = int(vocab_size), int(dim), name, float(scale)
        self.norm = build_part("norm", norm) if norm is not None else None
        self.table = None

    def children(self):
        return [self.norm] if self.norm is not None else []

    def param_specs(self):
        return {self.name: ParamSpec((self.vocab_size, self.dim))}

    def load(self, params):
        self.table = params[self.name].contiguous()

    def forward(self, ctx: StepContext) -> torch.Tensor:
        resid = torch.empty((ctx.num_tokens, self.dim), dtype=torch.float32, device=ctx.device)
        self.ops.embed(ctx.token_ids, self.table, resid, self.scale)
        if self.norm is not None:
            self.norm.norm_in_place(resid)
        return resid


@register_part("head", "linear")
class LinearHead(Head):
    """``logits = W x``; with ``softcap`` c the logits leave as ``c * tanh(logits / c)``.  ``name``: the matrix's relative name."""

    def __init__(self, prefix: str, dim: int, vocab_size: int, name: str = "weight", softcap=None):
        super().__init__(prefix)
        self.dim, self.vocab_size, self.name = int(dim), int(vocab_size), name
        self.softcap = None if softcap is None else float(softcap)
        if self.softcap is not None and not self.softcap > 0:
            raise ValueError(f"softcap must be positive or None, got {softcap}")
        self.weight = None

    def param_specs(self):
        return {self.name: ParamSpec((self.vocab_size, self.dim))}

    def load(self, params):
        self.weight = params[self.name].contiguous()

    def product_weights(self):
        return [self.weight]

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        logits = self.ops.linear(x, self.weight, None, out_dtype=torch.float32)
        if self.softcap is not None:
            self.ops.activation(logits, "softcap", c=self.softcap, inplace=True)
        return logits


@register_part("head", "tied")
class TiedHead(Head):
    """``logits = E x`` with the embedding table E itself: it owns no tensor; the model hands it the embedding's table once
    the weights are loaded."""
    tied_to_embedding = True

    def __init__(self, prefix: str, dim: int, vocab_size: int):
        super().__init__(prefix)
        self.dim, self.vocab_size = int(dim), int(vocab_size)
        self.weight = None

    def tie(self, embedding) -> None:
        self.weight = embedding.table

    def product_weights(self):
        return [self.weight]

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.ops.linear(x, self.weight, None, out_dtype=torch.float32)
