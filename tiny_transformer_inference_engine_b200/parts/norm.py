"""RMSNorm with the residual add fused in.

Formula of the reference (models/rmsnorm.py:12-18): ``x32 = float(x)``,
``y = x32 * rsqrt(mean(x32**2) + eps)``, ``out = (y * float(w)).to(dtype)`` -
eps inside the square root, weight multiplied in 32-bit before the cast.  The
reference fixes eps in code (models/rmsnorm.py:7) and never passes
``ModelConfig.rms_norm_eps``; here eps is this part's parameter.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .base import Norm, ParamSpec
from ..registry import register_part


@register_part("norm", "rmsnorm")
class RMSNorm(Norm):
    def __init__(self, prefix: str, dim: int, eps: float, name: str = "weight"):
        super().__init__(prefix)
        self.dim = int(dim)
        self.eps = float(eps)
        self.name = name                   # relative name of the weight tensor
        self.weight = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {self.name: ParamSpec((self.dim,), storage="vector", init="ones")}

    def load(self, params):
        self.weight = params[self.name]

    def validate(self, ops, dtype, page_size):
        check = getattr(ops, "check_norm", None)
        if check is not None:
            check(dtype, self.dim)

    def add_norm(self, resid: torch.Tensor, delta: Optional[torch.Tensor]) -> torch.Tensor:
        out = torch.empty(resid.shape, dtype=self.dtype, device=resid.device)
        self.ops.add_rmsnorm(resid, delta, self.weight, self.eps, out)
        return out

    def norm_rows(self, resid, delta, rows, num_rows) -> torch.Tensor:
        out = torch.empty((num_rows, self.dim), dtype=self.dtype, device=resid.device)
        if num_rows:
            self.ops.rmsnorm_rows(resid, delta, rows, num_rows, self.weight, self.eps, out)
        return out


@register_part("norm", "layernorm")
class LayerNorm(Norm):
    """LayerNorm with weight and bias over the 32-bit stream: ``(x - mean) / sqrt(var + eps) * w + b`` with the variance the
    mean of the squared deviations.  For post-norm blocks the scaled residual add is fused in:
    ``x <- LN(alpha * x + delta)``; the stream keeps the normalised value in 32-bit and the next sub-layer gets a copy in the
    compute dtype.  For blocks that norm a sub-layer's output, ``add_normed``: ``x <- x + LN(delta)``.  ``names``: relative
    tensor names of the weight and the bias.  ``bias=False``: a weight only.  ``scale`` (a relative tensor name): a layer
    scale, one factor per channel on the norm's result; it is multiplied into the weight (and the bias) in 32-bit when the
    tensors are loaded."""

    def __init__(self, prefix: str, dim: int, eps: float, names: Optional[Dict[str, str]] = None, bias: bool = True,
                 scale: Optional[str] = None):
        super().__init__(prefix)
        self.dim, self.eps, self.has_bias = int(dim), float(eps), bool(bias)
        self.names = {"weight": "weight", "bias": "bias"}
        if names:
            self.names.update(names)
        self.scale_name = scale
        self.weight = self.bias = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        specs = {self.names["weight"]: ParamSpec((self.dim,), storage="vector", init="ones")}
        if self.has_bias:
            specs[self.names["bias"]] = ParamSpec((self.dim,), storage="vector", init="zeros")
        if self.scale_name is not None:
            specs[self.scale_name] = ParamSpec((self.dim,), storage="vector", init="ones")
        return specs

    def load(self, params):
        self.weight = params[self.names["weight"]]
        self.bias = params[self.names["bias"]] if self.has_bias else None
        if self.scale_name is not None:
            ls = params[self.scale_name].float()
            self.weight = (self.weight.float() * ls).contiguous()
            if self.bias is not None:
                self.bias = (self.bias.float() * ls).contiguous()
        if self.bias is not None and self.bias.dtype != self.weight.dtype:
            self.bias = self.bias.to(self.weight.dtype)

    def validate(self, ops, dtype, page_size):
        check = getattr(ops, "check_norm", None)
        if check is not None:
            check(dtype, self.dim)

    def scale_add_norm(self, resid: torch.Tensor, delta: Optional[torch.Tensor], alpha: float) -> torch.Tensor:
        """``resid <- LN(alpha * resid + delta)`` in place; returns the normalised rows in the compute dtype (the stream
        itself in a 32-bit run)."""
        if self.dtype == torch.float32:
            self.ops.scale_add_layernorm(resid, delta, alpha, self.weight, self.bias, self.eps, None)
            return resid
        out = torch.empty(resid.shape, dtype=self.dtype, device=resid.device)
        self.ops.scale_add_layernorm(resid, delta, alpha, self.weight, self.bias, self.eps, out)
        return out

    def add_normed(self, resid: torch.Tensor, delta: torch.Tensor) -> torch.Tensor:
        """``resid <- resid + LN(delta)`` in place (moments of ``delta`` alone); returns the new rows in the compute dtype (the
        stream itself in a 32-bit run)."""
        if self.dtype == torch.float32:
            self.ops.scale_add_layernorm(resid, delta, 1.0, self.weight, self.bias, self.eps, None, add_normed=True)
            return resid
        out = torch.empty(resid.shape, dtype=self.dtype, device=resid.device)
        self.ops.scale_add_layernorm(resid, delta, 1.0, self.weight, self.bias, self.eps, out, add_normed=True)
        return out

    def norm_in_place(self, resid: torch.Tensor) -> None:
        """``resid <- LN(resid)`` over the 32-bit stream (a norm directly behind the embedding); no copy is made."""
        self.ops.scale_add_layernorm(resid, None, 1.0, self.weight, self.bias, self.eps, None)

    def norm_rows(self, resid, delta, rows, num_rows) -> torch.Tensor:
        out = torch.empty((num_rows, self.dim), dtype=self.dtype, device=resid.device)
        if num_rows:
            self.ops.scale_add_layernorm(resid, delta, 1.0, self.weight, self.bias, self.eps, out, rows=rows, num_rows=num_rows)
        return out
