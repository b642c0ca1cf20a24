"""Causal attention over a paged key/value cache (multi-query, grouped or multi-head).

Order of the reference's serving path (serving/paged_mqa.py:64-113): project q, k, v;
rotate q and k at the tokens' positions; store rotated k and raw v into the pages
at ``table[pos // page] * page + pos % page``; attend over every key of the request
read back from the pages (new ones included) with scale ``1/sqrt(head_dim)`` and a
bottom-right aligned causal mask (kernels/pagedattn/pagedattn.cu:196-207,256);
project the concatenated heads with ``out``.  Query head ``h`` uses kv head
``h // (heads / kv_heads)`` (kernels/flashattn/flashattn.cu, same rule).

The three projections are fused at load into one matrix ``[(Hq+2*Hkv)*D, d]`` so one
product feeds the rotate-and-store kernel.  ``window`` (keys ``pos-window+1..pos``), ``chunk`` (instead of a
window: a token sees the keys of its own chunk of ``chunk`` positions, chunks counted from position 0 of the sequence)
and ``page_size`` (a page size of this layer's own cache group) are parameters of the part; the reference's
model has none of them.  A run entry that reads
another entry's cache (``shares_kv``) has no k/v projection and stores nothing.

Further options, each with its constants as parameters (any of them selects the general step below):
``v_head_dim`` (a value size other than the key size), ``conv_taps`` (a short causal convolution over time on every
channel of q, k and v, directly behind the projection and before the rotation; weights ``<name><conv_suffix>``
[channels, taps], tap ``taps - 1`` multiplies the current token; the last ``taps - 1`` projected rows of a request are
kept in a state row), a position encoding that rotates only the first ``position.dim`` values of a head, ``softcap``
(a score s becomes ``softcap * tanh(s / softcap)`` before mask and softmax), ``gated`` (``True`` or ``"head"``: head h's
output is scaled by ``sigmoid(W_g x)_h``, one number per head; ``"value"``: the concatenated heads are multiplied value by
value with ``sigmoid(W_g x)``, ``W_g`` as large as ``W_q`` would be at the value size), ``qkv_bias`` (biases on q, k and v
only), ``qk_norm`` (its eps: every query and key head is divided by its root mean square and multiplied by a weight of
``head_dim`` values that all heads share, ``<q><norm_suffix>`` and ``<k><norm_suffix>``, before the rotation), ``v_from_k``
(there is no value projection: a value head is its key head as projected, before norm and rotation), ``q_temp``
(``coef``, ``every``: the query at position p is multiplied by ``1 + coef * ln(floor((p + 1) / every) + 1)``),
``qk_norm_over="projection"`` (with ``qk_norm``: ONE root mean square over all of a token's q and one over all of its k, before
they are cut into heads, and a weight per channel, ``<q><norm_suffix>`` of ``heads * head_dim`` values and ``<k><norm_suffix>`` of
``kv_heads * head_dim``; the default ``"head"`` is the norm per head above), ``weights="sigmoid"`` (no softmax: a visible key
weighs ``sigmoid(score + b_h)`` and the weights are not normalised over the keys; ``head_bias`` names the tensor of one ``b``
per head, None: no bias).  The general step: one product
``[W_q; W_k; W_v; W_g] x``; one kernel convolves, normalises, rotates, writes q and stores k and v - rows padded with zeros to
``padded_dim``, a multiple of 16 that holds both sizes, so every attention kernel of the package applies; a second moves the
convolution's inputs into the state row; attention; the gate kernel drops the padding; ``W_o``.
"""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch

from .base import Mixer, ParamSpec, PartSpec, PagedKVNeed, FixedStateNeed, PagedKVView, StepContext
from ..registry import register_part, build_part


@register_part("mixer", "attention")
class PagedAttention(Mixer):
    def __init__(self, prefix: str, d_model: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 position: PartSpec, bias: bool = False, window: Optional[int] = None,
                 scale: Optional[float] = None, shares_kv: bool = False,
                 names: Optional[Dict[str, str]] = None, page_size: Optional[int] = None,
                 v_head_dim: Optional[int] = None, conv_taps: Optional[int] = None, softcap: Optional[float] = None,
                 gated=False, qkv_bias: bool = False, weight_suffix: str = ".weight", bias_suffix: str = ".bias",
                 conv_suffix: str = ".conv", chunk: Optional[int] = None, qk_norm: Optional[float] = None,
                 norm_suffix: str = ".norm", v_from_k: bool = False, q_temp: Optional[Dict[str, float]] = None,
                 qk_norm_over: str = "head", weights: str = "softmax", head_bias: Optional[str] = None):
        super().__init__(prefix)
        if num_heads % num_kv_heads:
            raise ValueError(f"num_heads={num_heads} is not a multiple of num_kv_heads={num_kv_heads}")
        if window is not None and window < 1:
            raise ValueError(f"window must be >= 1 or None, got {window}")
        if chunk is not None and (chunk < 1 or window is not None):
            raise ValueError(f"chunk must be >= 1 or None and excludes a window, got chunk={chunk} window={window}")
        if gated not in (False, True, "head", "value"):
            raise ValueError(f"gated must be False, True / 'head' or 'value', got {gated!r}")
        self.d_model, self.num_heads, self.num_kv_heads, self.head_dim = d_model, num_heads, num_kv_heads, head_dim
        self.bias, self.window, self.shares_kv = bool(bias), window, bool(shares_kv)
        self.chunk = None if chunk is None else int(chunk)
        self.page_size = None if page_size is None else int(page_size)     # None: the engine's page size
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(head_dim)
        self.position = build_part("position", position)
        self.names = {"q": "q_proj", "k": "k_proj", "v": "v_proj", "o": "out", "g": "gate"}
        if names:
            self.names.update(names)
        self.w_in = self.b_in = self.w_out = self.b_out = None
        self.v_head_dim = int(v_head_dim) if v_head_dim is not None else head_dim
        self.has_conv = conv_taps is not None                         # (one tap is a weight per channel and keeps no state)
        self.conv_taps = int(conv_taps) if self.has_conv else 1
        if self.conv_taps < 1:
            raise ValueError(f"conv_taps must be >= 1 or None, got {conv_taps}")
        self.softcap = float(softcap) if softcap else None
        if self.softcap is not None and self.softcap <= 0:
            raise ValueError(f"softcap must be positive or None, got {softcap}")
        self.gated, self.qkv_bias = bool(gated), bool(qkv_bias)
        self.gate_per_value = gated == "value"
        self.weight_suffix, self.bias_suffix, self.conv_suffix, self.norm_suffix = weight_suffix, bias_suffix, conv_suffix, norm_suffix
        self.qk_norm = None if qk_norm is None else float(qk_norm)
        if qk_norm_over not in ("head", "projection"):
            raise ValueError(f"qk_norm_over must be 'head' or 'projection', got {qk_norm_over!r}")
        self.norm_whole = self.qk_norm is not None and qk_norm_over == "projection"
        if self.norm_whole and conv_taps is not None:
            raise ValueError("a norm over the whole projection and a convolution on it exclude each other")
        if weights not in ("softmax", "sigmoid"):
            raise ValueError(f"weights must be 'softmax' or 'sigmoid', got {weights!r}")
        if head_bias is not None and weights != "sigmoid":
            raise ValueError("a bias per head belongs to sigmoid weights (a softmax does not see it)")
        self.weights, self.head_bias_name, self.head_bias = weights, head_bias, None
        self.v_from_k = bool(v_from_k)
        if self.v_from_k and self.v_head_dim != head_dim:
            raise ValueError(f"values that are the keys have the keys' size {head_dim}, not {self.v_head_dim}")
        self.q_temp = None
        if q_temp is not None:
            self.q_temp = (float(q_temp["coef"]), int(q_temp["every"]))
            if self.q_temp[1] < 1:
                raise ValueError(f"q_temp.every must be >= 1, got {q_temp['every']}")
        self.rot_dim = int(getattr(self.position, "dim", 0) or 0)      # rotated values per head (0: none)
        if self.rot_dim > head_dim:
            raise ValueError(f"the position encoding rotates {self.rot_dim} values of a head of {head_dim}")
        self.general = (self.v_head_dim != head_dim or self.has_conv or self.gated or self.qkv_bias
                        or self.rot_dim not in (0, head_dim) or self.qk_norm is not None or self.v_from_k
                        or self.q_temp is not None or self.weights != "softmax")
        if self.general and (self.shares_kv or self.bias):
            raise ValueError("the general attention step has neither a shared cache nor an output bias")
        self.padded_dim = -(-max(head_dim, self.v_head_dim) // 16) * 16 if self.general else head_dim
        self.channels = (num_heads + num_kv_heads) * head_dim + (0 if self.v_from_k else num_kv_heads * self.v_head_dim)   # of [q | k | v]
        self.conv_w = self.norm_w = None

    def children(self):
        return [self.position]

    # ---------------------------------------------------------------- tensors
    def param_specs(self):
        if self.general:
            return self._general_specs()
        n, d, D = self.names, self.d_model, self.head_dim
        specs = {f"{n['q']}.weight": ParamSpec((self.num_heads * D, d)),
                 f"{n['o']}.weight": ParamSpec((d, self.num_heads * D))}
        if not self.shares_kv:
            specs[f"{n['k']}.weight"] = ParamSpec((self.num_kv_heads * D, d))
            specs[f"{n['v']}.weight"] = ParamSpec((self.num_kv_heads * D, d))
        if self.bias:
            for key in list(specs):
                w = specs[key]
                specs[key.replace(".weight", ".bias")] = ParamSpec((w.shape[0],), storage="matrix", init="normal")
        return specs

    def _general_specs(self):
        n, d, D, Dv, ws = self.names, self.d_model, self.head_dim, self.v_head_dim, self.weight_suffix
        rows = {"q": self.num_heads * D, "k": self.num_kv_heads * D, "v": self.num_kv_heads * Dv}
        if self.v_from_k:
            del rows["v"]
        specs = {f"{n['o']}{ws}": ParamSpec((d, self.num_heads * Dv))}
        for key, r in rows.items():
            specs[f"{n[key]}{ws}"] = ParamSpec((r, d))
            if self.qkv_bias:
                specs[f"{n[key]}{self.bias_suffix}"] = ParamSpec((r,), storage="vector", init="normal")
            if self.has_conv:
                specs[f"{n[key]}{self.conv_suffix}"] = ParamSpec((r, self.conv_taps), storage="vector", init="normal", std=0.5)
        if self.qk_norm is not None:
            for key in ("q", "k"):
                specs[f"{n[key]}{self.norm_suffix}"] = ParamSpec((rows[key] if self.norm_whole else D,), storage="vector", init="ones")
        if self.head_bias_name is not None:
            specs[self.head_bias_name] = ParamSpec((self.num_heads,), storage="vector", init="normal", std=0.5)
        if self.gated:
            specs[f"{n['g']}{ws}"] = ParamSpec((self.num_heads * (Dv if self.gate_per_value else 1), d))
        return specs

    def _general_load(self, params):
        n, ws = self.names, self.weight_suffix
        qkv = ["q", "k"] if self.v_from_k else ["q", "k", "v"]
        keys = qkv + (["g"] if self.gated else [])
        self.w_in = torch.cat([params[f"{n[k]}{ws}"] for k in keys], dim=0).contiguous()
        self.w_out = params[f"{n['o']}{ws}"].contiguous()
        if self.qkv_bias:
            b = [params[f"{n[k]}{self.bias_suffix}"].to(self.w_in.dtype) for k in qkv]
            if self.gated:
                b.append(torch.zeros(self.w_in.shape[0] - self.channels, dtype=self.w_in.dtype, device=self.w_in.device))
            self.b_in = torch.cat(b, dim=0).contiguous()
        if self.has_conv:                                               # tap-major, 32-bit: a tap's weights lie side by side
            w = torch.cat([params[f"{n[k]}{self.conv_suffix}"].float() for k in qkv], dim=0)
            self.conv_w = w.t().contiguous()
        if self.qk_norm is not None:                                    # 32-bit, the query heads' weights then the key heads'
            ws_ = [params[f"{n[k]}{self.norm_suffix}"].float() for k in ("q", "k")]
            self.norm_w = (torch.cat(ws_) if self.norm_whole else torch.stack(ws_)).contiguous()
        if self.head_bias_name is not None:
            self.head_bias = params[self.head_bias_name].float().contiguous()

    def load(self, params):
        if self.general:
            return self._general_load(params)
        n = self.names
        keys = ["q"] if self.shares_kv else ["q", "k", "v"]
        self.w_in = torch.cat([params[f"{n[k]}.weight"] for k in keys], dim=0).contiguous()
        self.w_out = params[f"{n['o']}.weight"].contiguous()
        if self.bias:
            self.b_in = torch.cat([params[f"{n[k]}.bias"] for k in keys], dim=0).contiguous()
            self.b_out = params[f"{n['o']}.bias"].contiguous()

    def product_weights(self):
        return [self.w_in, self.w_out]

    def validate(self, ops, dtype, page_size):
        check = getattr(ops, "check_attention", None)
        if check is not None:
            check(dtype, self.num_heads, self.num_kv_heads, self.padded_dim, self.page_size or page_size)

    # ---------------------------------------------------------------- cache
    def cache_needs(self):
        needs = [PagedKVNeed(self.num_kv_heads, self.padded_dim, self.window, self.page_size, chunk=self.chunk)]
        if self.conv_taps > 1:
            needs.append(FixedStateNeed((self.conv_taps - 1, self.channels), "float32"))
        return needs

    # ---------------------------------------------------------------- step
    def _general_forward(self, x, ctx, cache, tail):
        ops = self.ops
        Hq, Hkv, D, Dv, Dp, C = self.num_heads, self.num_kv_heads, self.head_dim, self.v_head_dim, self.padded_dim, self.channels
        proj = ops.linear(x, self.w_in, self.b_in)                   # [T, channels (+ Hq gate columns)]
        T = proj.shape[0]
        table = self.position.rotary_table()
        inv_freq, style = table if table is not None else (None, 0)
        rot = self.rot_dim if inv_freq is not None else 0
        cs = self.position.step_table(ctx) if rot else None
        state = tail.state if tail is not None else None
        row_inv = ops.proj_row_rms(proj, Hq * D, Hkv * D, self.qk_norm) if self.norm_whole else None
        q = ops.qkv_conv_rope_store(proj, Hq, Hkv, D, Dv, Dp, self.conv_taps, self.conv_w, state, ctx.positions, ctx.token_seq,
                                    ctx.query_start_loc, ctx.slot_ids, cs, rot, style, cache.k_pages, cache.v_pages,
                                    cache.block_table, cache.page_size, cache.writable, norm_w=self.norm_w,
                                    norm_eps=self.qk_norm or 0.0, v_from_k=self.v_from_k, q_temp=self.q_temp, row_inv=row_inv)
        if self.conv_taps > 1 and tail.writable:
            ops.conv_tail_update(proj, C, self.conv_taps, state, ctx.query_start_loc, ctx.slot_ids, ctx.num_seqs)
        out = torch.empty((T, Hq * Dp), dtype=x.dtype, device=x.device)
        self._attend(q, Dp, ctx, cache, out)
        if self.gated or Dp != Dv:
            out = ops.gate_head_rows(out, proj[:, C:] if self.gated else None, Hq, Dv, Dp, per_value=self.gate_per_value)
        return ops.linear(out, self.w_out, None, partial_ok=True)

    def _attend(self, q, D, ctx, cache, out):
        """One attention launch per class of requests (decoded tokens; prompt portions), each planned as if it were alone."""
        ops, Hq, Hkv = self.ops, self.num_heads, self.num_kv_heads
        extra = {} if self.weights == "softmax" else {"weights": self.weights, "head_bias": self.head_bias}
        classes = ctx.classes()
        if len(classes) == 1:
            c = classes[0]
            ops.paged_attention(q, Hq, Hkv, D, cache.k_pages, cache.v_pages, cache.block_table, cache.page_size,
                                c.query_start_loc, ctx.seq_lens, ctx.num_seqs, c.max_q_len, c.max_kv_len,
                                self.scale, self.window or 0, out, softcap=self.softcap or 0.0, chunk=self.chunk or 0, **extra)
            return
        for ci, c in enumerate(classes):
            key = ("attention class views", id(cache.block_table), ci)    # the same for every layer of a cache group
            views = ctx.step_cache.get(key)
            if views is None:
                views = ctx.step_cache[key] = (cache.block_table[c.seq_lo:c.seq_hi], ctx.seq_lens[c.seq_lo:c.seq_hi])
            ops.paged_attention(q[c.tok_lo:c.tok_hi], Hq, Hkv, D, cache.k_pages, cache.v_pages, views[0],
                                cache.page_size, c.query_start_loc, views[1], c.seq_hi - c.seq_lo, c.max_q_len,
                                c.max_kv_len, self.scale, self.window or 0, out[c.tok_lo:c.tok_hi], softcap=self.softcap or 0.0,
                                chunk=self.chunk or 0, **extra)

    def forward(self, x: torch.Tensor, ctx: StepContext, cache) -> torch.Tensor:
        tail = None
        if isinstance(cache, (list, tuple)):                         # the views in the order of cache_needs()
            tail = cache[1] if len(cache) > 1 else None
            cache = cache[0]
        if self.general:
            return self._general_forward(x, ctx, cache, tail)
        ops = self.ops
        Hq, Hkv, D = self.num_heads, self.num_kv_heads, self.head_dim
        write = cache.writable and not self.shares_kv
        kv_heads_in_buf = 0 if self.shares_kv else Hkv
        qkv = ops.linear(x, self.w_in, self.b_in, partial_ok=True)   # [T, (Hq + 2*Hkv) * D], or partial sums of it
        T = qkv.shape[-2]
        table = self.position.rotary_table()
        if table is None:
            if qkv.dim() == 3:
                qkv = qkv.sum(0).to(x.dtype)
            q = qkv[:, :Hq * D].view(T, Hq, D)
            k = None if self.shares_kv else qkv[:, Hq * D:(Hq + Hkv) * D].view(T, Hkv, D)
            self.position.apply(q, k, ctx.positions)
            inv_freq, style = None, 0
            cs_table = None
        else:
            inv_freq, style = table
            cs_table = self.position.step_table(ctx) if inv_freq is not None else None
        q = qkv
        if qkv.dim() == 3:
            q = torch.empty((T, Hq * D), dtype=x.dtype, device=x.device)
        ops.rope_store(qkv, Hq, kv_heads_in_buf, D, ctx.positions, ctx.token_seq, inv_freq, style,
                       cache.k_pages, cache.v_pages, cache.block_table, cache.page_size, write,
                       q_out=q if qkv.dim() == 3 else None, cs_table=cs_table)
        out = torch.empty((T, Hq * D), dtype=x.dtype, device=x.device)
        self._attend(q, D, ctx, cache, out)
        return ops.linear(out, self.w_out, self.b_out, partial_ok=True)
