"""A routed mixture of gated-linear-unit experts with grouped top-k selection and an optional shared expert.

Router: ``z = W_r h`` in 32-bit (``h`` in the compute dtype), scores ``s = sigmoid(z)`` or (``score="softmax"``) the softmax
of ``z`` over all experts.  The choice is made by ``c = s + correction`` where the router has a correction tensor (one number
per expert, ``correction=True``), else by ``s`` itself; the weights always use ``s``.  Expert ``e`` belongs to group
``e // (experts / groups)``.  Each group is rated by adding up its ``group_top`` highest ``c``; the ``keep`` best-rated groups
stay eligible and the experts of all other groups are masked out.  Among the eligible experts the ``top`` highest ``c`` are
taken, each weighted ``s * scale`` (``renorm``: divided by the sum of the taken scores first).  The output is the weighted sum of the chosen experts' outputs plus, if there is one, a shared
expert that every token runs.  An expert is ``down(act(gate h) * up h)`` with the activation's constants as parameters.
``identity``: the router has that many more outputs behind the ``experts`` real ones; they stand for identity experts, which
own no tensors and return their input ``h`` (times the weight).  ``expert="mlp"``: an expert is ``down(act(up h))`` without a
gate (``act``: "relu2", the square of relu).  ``weight_on="input"``: the routing weight multiplies the chosen expert's INPUT,
``sum_e expert_e(w_e h)``, not its output (``"output"``, the default); since the first product is linear the weight is applied to
its 32-bit sums, ahead of the activation.  ``shared_gate`` (a relative tensor name, [1, d]): the shared expert's output is
multiplied by ``sigmoid(w_sg . h)``, one number per token; the row rides in the router's product.

On the device, with nothing read on the host (so a step can be captured in a graph): route -> counting sort of the
(token, choice) pairs by expert -> grouped product gate/up over the sorted rows (rows gathered from the tokens) ->
activation -> grouped product down -> weighted sum per token in the order of the choices (32-bit).  The expert matrices are
stacked at load: ``[E, 2F, d]`` and ``[E, d, F]``.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .base import FeedForward, ParamSpec, PartSpec, StepContext
from ..registry import register_part, build_part


@register_part("ffn", "grouped_moe")
class GroupedMoE(FeedForward):
    def __init__(self, prefix: str, d_model: int, hidden: int, experts: int, top: int, groups: int = 1, keep: int = 1,
                 group_top: int = 2, scale: float = 1.0, renorm: bool = False, alpha: float = 1.0,
                 limit: Optional[float] = None, shift: float = 0.0, shared: Optional[PartSpec] = None,
                 names: Optional[Dict[str, str]] = None, score: str = "sigmoid", correction: bool = False, identity: int = 0,
                 expert: str = "glu", act: str = "relu2", weight_on: str = "output", shared_gate: Optional[str] = None):
        super().__init__(prefix)
        if identity < 0 or experts < 0 or experts + identity < 1:
            raise ValueError(f"{experts} experts and {identity} identity experts")
        routed = int(experts) + int(identity)                        # the router's outputs
        if routed % groups:
            raise ValueError(f"{routed} experts do not form {groups} equal groups")
        if not 1 <= keep <= groups:
            raise ValueError(f"keep={keep} of {groups} groups")
        if not 1 <= top <= keep * (routed // groups):
            raise ValueError(f"top={top} experts cannot be chosen from {keep} groups of {routed // groups}")
        if score not in ("sigmoid", "softmax"):
            raise ValueError(f"unknown router score {score!r}; known: sigmoid, softmax")
        if expert not in ("glu", "mlp"):
            raise ValueError(f"unknown kind of expert {expert!r}; known: glu, mlp")
        if act != "relu2":
            raise ValueError(f"unknown expert activation {act!r}; known: relu2")
        if weight_on not in ("output", "input"):
            raise ValueError(f"weight_on must be 'output' or 'input', got {weight_on!r}")
        if weight_on == "input" and (expert != "mlp" or identity):
            raise ValueError("a routing weight on the expert's input is built for ungated experts without identity experts")
        if shared_gate is not None and shared is None:
            raise ValueError("a gate on the shared expert needs a shared expert")
        self.expert_kind, self.act, self.weight_on_input, self.shared_gate = expert, act, weight_on == "input", shared_gate
        self.score, self.has_correction, self.identity, self.routed = score, bool(correction), int(identity), routed
        self.d_model, self.hidden, self.experts, self.top = int(d_model), int(hidden), int(experts), int(top)
        self.groups, self.keep, self.group_top = int(groups), int(keep), int(group_top)
        self.scale, self.renorm = float(scale), bool(renorm)
        self.alpha, self.limit, self.shift = float(alpha), limit, float(shift)
        self.shared = build_part("ffn", shared) if shared is not None else None
        self.names = {"router": "router", "correction": "correction", "expert": "e{}", "gate": "gate", "up": "up", "down": "down"}
        self.correction = None
        if names:
            self.names.update(names)

    def children(self):
        return [self.shared] if self.shared is not None else []

    def _expert_name(self, e: int, which: str) -> str:
        return f"{self.names['expert'].format(e)}.{self.names[which]}"

    def param_specs(self):
        d, F = self.d_model, self.hidden
        specs = {self.names["router"]: ParamSpec((self.routed, d), std=0.5)}
        if self.has_correction:
            specs[self.names["correction"]] = ParamSpec((self.routed,), storage="vector", init="normal", std=0.1)
        if self.shared_gate is not None:
            specs[self.shared_gate] = ParamSpec((1, d), std=0.5)
        for e in range(self.experts):
            if self.expert_kind == "glu":
                specs[self._expert_name(e, "gate")] = ParamSpec((F, d))
            specs[self._expert_name(e, "up")] = ParamSpec((F, d))
            specs[self._expert_name(e, "down")] = ParamSpec((d, F))
        return specs

    def load(self, params):
        E = self.experts
        self.w_router = params[self.names["router"]].contiguous()
        if self.shared_gate is not None:                                 # the shared expert's gate: one more row of the router's product
            self.w_router = torch.cat([self.w_router, params[self.shared_gate].reshape(1, -1)], dim=0).contiguous()
        if self.w_router.shape[0] % 8:                                   # rows of zeros up to a multiple of 8: the library's product
            pad = self.w_router.new_zeros((-self.w_router.shape[0] % 8, self.w_router.shape[1]))     # of many rows wants 32-byte rows of logits
            self.w_router = torch.cat([self.w_router, pad], dim=0).contiguous()
        if self.has_correction:
            self.correction = params[self.names["correction"]].float().contiguous()
        if E == 0:                                                       # (identity experts only: nothing to multiply)
            self.w_gu = self.w_down = None
            return
        if self.expert_kind == "mlp":
            self.w_gu = torch.stack([params[self._expert_name(e, "up")] for e in range(E)]).contiguous()      # [E, F, d]
        else:
            self.w_gu = torch.stack([torch.cat([params[self._expert_name(e, "gate")], params[self._expert_name(e, "up")]], dim=0)
                                     for e in range(E)]).contiguous()                    # [E, 2F, d]
        self.w_down = torch.stack([params[self._expert_name(e, "down")] for e in range(E)]).contiguous()   # [E, d, F]

    def validate(self, ops, dtype, page_size):
        limit = getattr(getattr(ops, "lib", None), "ttie_moe_max_experts", None)
        if limit is not None and self.routed > int(limit()):
            raise ValueError(f"{self.routed} experts exceed the routing kernels' limit of {int(limit())}")

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        ops, T = self.ops, x.shape[0]
        all_logits = ops.linear(x, self.w_router, None, out_dtype=torch.float32)
        logits = all_logits[:, :self.routed]
        idx, wts = ops.moe_route(logits, self.groups, self.keep, self.group_top, self.top, self.scale, self.renorm,
                                 score=self.score, correction=self.correction)
        plan = ops.moe_plan(idx, self.routed, identity=self.identity)
        if self.experts and self.expert_kind == "mlp":
            act = ops.grouped_act(x, self.w_gu, plan, self.top, self.act, row_scale=wts if self.weight_on_input else None)
            y = ops.grouped_linear(act, self.w_down, plan, out_dtype=torch.float32)
        elif self.experts:
            act = ops.grouped_glu(x, self.w_gu, plan, self.top, self.hidden, self.alpha, self.limit or 0.0, self.shift)   # [P, F], rows sorted by expert
            y = ops.grouped_linear(act, self.w_down, plan, out_dtype=torch.float32)      # [P, d] float32 (rows of identity experts: never read)
        else:
            y = x
        shared = self.shared.forward(x, ctx, partial_ok=False) if self.shared is not None else None
        gate = all_logits[:, self.routed:self.routed + 1] if self.shared_gate is not None else None
        return ops.moe_combine(y, plan, None if self.weight_on_input else wts, shared, T, self.d_model,
                               x=x if self.identity else None, shared_gate=gate)         # float32 [T, d]
