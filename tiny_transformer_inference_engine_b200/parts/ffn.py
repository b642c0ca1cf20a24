"""Dense SwiGLU feed-forward.

Reference (models/mlp.py:17-32): ``down(silu(gate(x)) * up(x))`` with
``silu(g) = g * sigmoid(g)`` evaluated in 32-bit (kernels/fused_swiglu/kernel.py:20-25),
three linears with bias iff ``bias``.  ``gate`` and ``up`` are fused at load into one
matrix ``[2F, d]`` (gate rows first) so one product feeds the activation kernel.
The width ``F`` is this part's parameter.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .base import FeedForward, ParamSpec, StepContext
from ..registry import register_part


@register_part("ffn", "swiglu")
class SwiGLU(FeedForward):
    def __init__(self, prefix: str, d_model: int, hidden: int, bias: bool = False):
        super().__init__(prefix)
        self.d_model, self.hidden, self.bias = int(d_model), int(hidden), bool(bias)
        self.w_gu = self.b_gu = self.w_down = self.b_down = None

    def param_specs(self):
        d, F = self.d_model, self.hidden
        specs = {"gate_proj.weight": ParamSpec((F, d)), "up_proj.weight": ParamSpec((F, d)),
                 "down_proj.weight": ParamSpec((d, F))}
        if self.bias:
            specs.update({"gate_proj.bias": ParamSpec((F,)), "up_proj.bias": ParamSpec((F,)),
                          "down_proj.bias": ParamSpec((d,))})
        return specs

    def load(self, params):
        self.w_gu = torch.cat([params["gate_proj.weight"], params["up_proj.weight"]], dim=0).contiguous()
        self.w_down = params["down_proj.weight"].contiguous()
        if self.bias:
            self.b_gu = torch.cat([params["gate_proj.bias"], params["up_proj.bias"]], dim=0).contiguous()
            self.b_down = params["down_proj.bias"].contiguous()

    def product_weights(self):
        return [self.w_down]                     # (gate/up beyond 8 rows is the library's product plus the activation kernel)

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        act = self.ops.linear_swiglu(x, self.w_gu, self.b_gu, self.hidden)        # [T, F]
        return self.ops.linear(act, self.w_down, self.b_down, partial_ok=True)


@register_part("ffn", "glu")
class GLU(FeedForward):
    """A gated linear unit with its constants as parameters:
    ``down(g' * sigmoid(alpha * g') * (u' + shift))`` with ``g = gate(x)``, ``u = up(x)``, ``g' = min(g, limit)`` and
    ``u' = clamp(u, -limit, limit)`` (``limit`` None: no clamps).  ``alpha = 1, shift = 0, limit = None`` is SwiGLU;
    ``alpha = 1.702, shift = 1`` with a limit is the clamped form some models use.  No biases.  ``names``: relative tensor
    names of the three matrices."""

    def __init__(self, prefix: str, d_model: int, hidden: int, alpha: float = 1.0, limit: Optional[float] = None,
                 shift: float = 0.0, names: Optional[Dict[str, str]] = None):
        super().__init__(prefix)
        self.d_model, self.hidden = int(d_model), int(hidden)
        self.alpha, self.limit, self.shift = float(alpha), (None if limit is None else float(limit)), float(shift)
        if self.limit is not None and self.limit <= 0:
            raise ValueError(f"limit must be positive or None, got {limit}")
        self.names = {"gate": "gate", "up": "up", "down": "down"}
        if names:
            self.names.update(names)
        self.w_gu = self.w_down = None

    def param_specs(self):
        n, d, F = self.names, self.d_model, self.hidden
        return {n["gate"]: ParamSpec((F, d)), n["up"]: ParamSpec((F, d)), n["down"]: ParamSpec((d, F))}

    def load(self, params):
        n = self.names
        self.w_gu = torch.cat([params[n["gate"]], params[n["up"]]], dim=0).contiguous()
        self.w_down = params[n["down"]].contiguous()

    def product_weights(self):
        return [self.w_gu, self.w_down]

    def forward(self, x: torch.Tensor, ctx: StepContext, partial_ok: bool = True) -> torch.Tensor:
        act = self.ops.linear_glu(x, self.w_gu, self.hidden, self.alpha, self.limit or 0.0, self.shift)
        return self.ops.linear(act, self.w_down, None, partial_ok=partial_ok)


@register_part("ffn", "mlp")
class MLP(FeedForward):
    """A two-matrix feed-forward ``down(act(up(x)))`` without biases.  ``act``: ``"relu2"``, the square of relu.
    ``names``: relative tensor names of the two matrices."""
    ACTIVATIONS = ("relu2",)

    def __init__(self, prefix: str, d_model: int, hidden: int, act: str = "relu2", names: Optional[Dict[str, str]] = None):
        super().__init__(prefix)
        if act not in self.ACTIVATIONS:
            raise ValueError(f"unknown activation {act!r}; known: {self.ACTIVATIONS}")
        self.d_model, self.hidden, self.act = int(d_model), int(hidden), act
        self.names = {"up": "up", "down": "down"}
        if names:
            self.names.update(names)
        self.w_up = self.w_down = None

    def param_specs(self):
        n, d, F = self.names, self.d_model, self.hidden
        return {n["up"]: ParamSpec((F, d)), n["down"]: ParamSpec((d, F))}

    def load(self, params):
        self.w_up = params[self.names["up"]].contiguous()
        self.w_down = params[self.names["down"]].contiguous()

    def product_weights(self):
        return [self.w_up, self.w_down]

    def forward(self, x: torch.Tensor, ctx: StepContext, partial_ok: bool = True) -> torch.Tensor:
        act = self.ops.linear_act(x, self.w_up, self.act)             # [T, F]
        return self.ops.linear(act, self.w_down, None, partial_ok=partial_ok)
