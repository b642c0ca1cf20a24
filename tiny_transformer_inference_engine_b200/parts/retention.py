"""Retention: linear attention with one fixed decay per head, no softmax and no denominator (a matrix state per head).

With ``h`` the mixer's input: ``q = W_q h`` and ``k = W_k h`` (heads x dim), ``v = W_v h`` (heads x vdim), no biases.  q and k
pass the position encoding (a rotation of the first values of every head); k is then multiplied by ``dim^(-1/2)``.  Per head,
with the state S [dim x vdim] starting at zero,

    S_t = decay_h S_(t-1) + k_t v_t^T          o_t = S_t^T q_t

Each head's ``o`` is divided by its root mean square (``x / sqrt(mean(x^2) + eps)``, no weight), the heads are concatenated,
multiplied by ``silu(W_g h)`` and projected by ``W_o``.

Per request one state row, 32-bit: S as ``[heads, vdim, padded dim]`` (value column major, the layout of the other
matrix-state scans), so a sequence may be cut into steps anywhere.  What enters the recurrence besides the projections is
32-bit in every run: the rotated and scaled q and k are written as 32-bit rows (``rotate_heads``), the decay, the state and
the read-out stay 32-bit.  q, k, v and the gate are one product.
"""
from __future__ import annotations

from typing import Dict, Optional, Sequence

import torch

from .base import Mixer, ParamSpec, PartSpec, FixedStateNeed, StepContext
from .wkv import padded_keys, MAX_KEYS
from ..registry import register_part, build_part


@register_part("mixer", "retention")
class Retention(Mixer):
    def __init__(self, prefix: str, d_model: int, num_heads: int, dim: int, vdim: int, decay: Sequence[float], eps: float,
                 position: Optional[PartSpec] = None, gate_act: str = "silu", names: Optional[Dict[str, str]] = None):
        super().__init__(prefix)
        self.d_model, self.num_heads, self.dim, self.vdim, self.eps = int(d_model), int(num_heads), int(dim), int(vdim), float(eps)
        self.decay = tuple(float(x) for x in decay)
        if len(self.decay) != self.num_heads:
            raise ValueError(f"retention: {len(self.decay)} decays for {self.num_heads} heads")
        if self.dim > MAX_KEYS:
            raise ValueError(f"retention: {dim} key channels per head (at most {MAX_KEYS})")
        if gate_act not in ("silu", "sigmoid"):
            raise ValueError(f"retention: unknown gate activation {gate_act!r}")
        self.gate_act = gate_act
        self.position = build_part("position", position if position is not None else PartSpec("none", "", {}))
        self.rot_dim = int(getattr(self.position, "dim", 0) or 0)
        if self.rot_dim > self.dim:
            raise ValueError(f"retention: the position encoding rotates {self.rot_dim} values of a head of {self.dim}")
        self.names = {"q": "q", "k": "k", "v": "v", "g": "g", "o": "o"}
        if names:
            self.names.update(names)
        self.w_in = self.w_out = self.decay_t = None

    def children(self):
        return [self.position]

    def param_specs(self):
        n, d, H, D, Dv = self.names, self.d_model, self.num_heads, self.dim, self.vdim
        return {n["q"]: ParamSpec((H * D, d)), n["k"]: ParamSpec((H * D, d)), n["v"]: ParamSpec((H * Dv, d)),
                n["g"]: ParamSpec((H * Dv, d)), n["o"]: ParamSpec((d, H * Dv))}

    def load(self, params):
        n = self.names
        self.w_in = torch.cat([params[n[s]] for s in ("q", "k", "v", "g")], dim=0).contiguous()       # [2*H*dim + 2*H*vdim, d]
        self.w_out = params[n["o"]].contiguous()
        self.decay_t = torch.tensor(self.decay, dtype=torch.float32, device=self.w_in.device)

    def product_weights(self):
        return [self.w_in, self.w_out]

    def cache_needs(self):
        return [FixedStateNeed((self.num_heads, self.vdim, padded_keys(self.dim)), "float32")]

    def forward(self, x: torch.Tensor, ctx: StepContext, cache) -> torch.Tensor:
        ops, H, D, Dv = self.ops, self.num_heads, self.dim, self.vdim
        S = cache[0]
        proj = ops.linear(x, self.w_in, None)                                                  # [T, q | k | v | g]
        table = self.position.rotary_table()
        inv_freq, style = table if table is not None else (None, 0)
        rot = self.rot_dim if inv_freq is not None else 0
        cs = self.position.step_table(ctx) if rot else None
        qk = ops.rotate_heads(proj, 2 * H, D, cs, rot, style, scale_from=H, scale=D ** -0.5)   # float32 [T, q | k]
        v, g = proj[:, 2 * H * D:2 * H * D + H * Dv], proj[:, 2 * H * D + H * Dv:]
        o = ops.retention_scan(qk[:, :H * D], qk[:, H * D:], v, self.decay_t, S.state, ctx.query_start_loc, ctx.slot_ids,
                               ctx.num_seqs, H, D, Dv)
        y = ops.head_norm_gate(o, g, None, H, Dv, self.eps, self.gate_act)
        return ops.linear(y, self.w_out, None, partial_ok=True)
