"""Latent attention over a paged cache of low-rank latents (sliding window, gated heads).

Per token the cache holds one row ``[c | k_rot | zeros]``: the latent ``c = rmsnorm(W_dkv h)[:rank]`` and one rotated
key part ``k_rot`` shared by all heads (the last ``rot_dim`` outputs of ``W_dkv``, rotated at the token's position).  A
head's key is ``[W_uk c | k_rot]`` and its value ``W_uv c``; neither is ever formed.  Since
``q_n . (W_uk c) = (W_uk^T q_n) . c``, the head's query is folded to ``q' = [W_uk^T q_n | rot(q_r) | 0]`` and every head
attends over the same cache rows - multi-query attention with one kv head whose keys AND values are that one array (the
cache group has one plane) - and the value up-projection follows: ``o_h = W_uv (sum_j p_j c_j)``.  So a prompt portion and a
decoded token run the same paged attention kernels as ordinary attention, at head size ``rank + rot_dim`` rounded up to the
kernels' granule.  Softmax scale, window (keys ``pos - window + 1 .. pos``), rotation base and all sizes are parameters.
``sigmoid(W_g h)_h`` scales head ``h``'s output (``gated``).  A layer built with ``shares_kv`` has no ``W_dkv`` and writes
nothing: its run entry reads the cache of the entry that owns one; ``cache_window`` is then the owner's need (the widest
window among the layers that read the cache).

``q_rank`` (optional): the queries go through a latent of their own, ``c_q = rmsnorm(W_dq h) * w`` and ``q = W_uq c_q`` (tensors
``dq``, ``dq.norm``, ``uq`` instead of ``q``).  ``gated="value"``: the gate is as wide as the concatenated heads,
``sigmoid(W_g h)`` value by value (``True`` / ``"head"``: one number per head).

One product ``[W_q (or W_dq); W_g; W_dkv] h`` feeds the step; the folds are batched per-head products.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .base import Mixer, ParamSpec, PartSpec, PagedKVNeed, PagedKVView, StepContext
from ..registry import register_part, build_part

ROW_GRANULE = 16            # cache rows are padded to a multiple of this (the tensor-core attention kernels' head-size step)


@register_part("mixer", "latent_attention")
class LatentAttention(Mixer):
    def __init__(self, prefix: str, d_model: int, num_heads: int, dim: int, rot_dim: int, vdim: int, kv_rank: int,
                 position: PartSpec, scale: float, eps: float, window: Optional[int] = None, gated=True,
                 shares_kv: bool = False, cache_window: Optional[int] = None, page_size: Optional[int] = None,
                 names: Optional[Dict[str, str]] = None, q_rank: Optional[int] = None):
        super().__init__(prefix)
        if rot_dim % 2:
            raise ValueError(f"rotated size {rot_dim} must be even")
        if window is not None and window < 1:
            raise ValueError(f"window must be >= 1 or None, got {window}")
        self.d_model, self.num_heads, self.dim, self.rot_dim = int(d_model), int(num_heads), int(dim), int(rot_dim)
        self.vdim, self.kv_rank, self.scale, self.eps = int(vdim), int(kv_rank), float(scale), float(eps)
        if gated not in (False, True, "head", "value"):
            raise ValueError(f"gated must be False, True / 'head' or 'value', got {gated!r}")
        self.window, self.gated, self.shares_kv = window, bool(gated), bool(shares_kv)
        self.gate_per_value = gated == "value"
        self.q_rank = None if q_rank is None else int(q_rank)
        if self.q_rank is not None and self.q_rank < 1:
            raise ValueError(f"q_rank must be >= 1 or None, got {q_rank}")
        self.cache_window = cache_window if cache_window is not None else window
        self.page_size = None if page_size is None else int(page_size)
        self.row = -(-(self.kv_rank + self.rot_dim) // ROW_GRANULE) * ROW_GRANULE
        self.position = build_part("position", position)
        self.names = {"q": "q", "dq": "dq", "dq_norm": "dq.norm", "uq": "uq", "dkv": "dkv", "dkv_norm": "dkv.norm", "uk": "uk", "uv": "uv",
                      "g": "g", "o": "o"}
        if names:
            self.names.update(names)
        self.w_in = self.w_uk_t = self.w_uv = self.w_out = self.norm_w = self.w_uq = self.q_norm_w = None

    def children(self):
        return [self.position]

    # ---------------------------------------------------------------- tensors
    def param_specs(self):
        n, d, H = self.names, self.d_model, self.num_heads
        specs = {n["uk"]: ParamSpec((H * self.dim, self.kv_rank)),
                 n["uv"]: ParamSpec((H * self.vdim, self.kv_rank)),
                 n["o"]: ParamSpec((d, H * self.vdim))}
        if self.q_rank is None:
            specs[n["q"]] = ParamSpec((H * (self.dim + self.rot_dim), d))
        else:
            specs[n["dq"]] = ParamSpec((self.q_rank, d))
            specs[n["dq_norm"]] = ParamSpec((self.q_rank,), storage="vector", init="ones")
            specs[n["uq"]] = ParamSpec((H * (self.dim + self.rot_dim), self.q_rank))
        if self.gated:
            specs[n["g"]] = ParamSpec((H * self.vdim if self.gate_per_value else H, d))
        if not self.shares_kv:
            specs[n["dkv"]] = ParamSpec((self.kv_rank + self.rot_dim, d))
            specs[n["dkv_norm"]] = ParamSpec((self.kv_rank,), storage="vector", init="ones")
        return specs

    def load(self, params):
        n, H = self.names, self.num_heads
        first = params[n["q"]] if self.q_rank is None else params[n["dq"]]
        mats = [first] + ([params[n["g"]]] if self.gated else []) + ([] if self.shares_kv else [params[n["dkv"]]])
        self.w_in = torch.cat(mats, dim=0).contiguous()
        self.col_g = first.shape[0]
        self.gate_cols = 0 if not self.gated else H * self.vdim if self.gate_per_value else H
        self.col_dkv = self.col_g + self.gate_cols
        if self.q_rank is not None:
            self.w_uq = params[n["uq"]].contiguous()
            self.q_norm_w = params[n["dq_norm"]]
        # W_uk^T per head: [H, rank, dim], so that folded[h] = q_n[h] @ w_uk_t[h].T
        self.w_uk_t = params[n["uk"]].view(H, self.dim, self.kv_rank).transpose(1, 2).contiguous()
        self.w_uv = params[n["uv"]].view(H, self.vdim, self.kv_rank).contiguous()
        self.w_out = params[n["o"]].contiguous()
        self.norm_w = None if self.shares_kv else params[n["dkv_norm"]]

    def product_weights(self):
        return [self.w_in, self.w_out] + ([self.w_uq] if self.w_uq is not None else [])

    def validate(self, ops, dtype, page_size):
        check = getattr(ops, "check_attention", None)
        if check is not None:
            check(dtype, self.num_heads, 1, self.row, self.page_size or page_size)

    # ---------------------------------------------------------------- cache
    def cache_need(self):
        return PagedKVNeed(1, self.row, self.cache_window, self.page_size, planes=1)

    # ---------------------------------------------------------------- step
    def forward(self, x: torch.Tensor, ctx: StepContext, cache: PagedKVView) -> torch.Tensor:
        ops, H, R = self.ops, self.num_heads, self.row
        proj = ops.linear(x, self.w_in, None)                        # [T, H*(dim+rot) | H | rank+rot]
        T = proj.shape[0]
        cs = self.position.step_table(ctx)
        if cache.writable and not self.shares_kv:
            ops.latent_store(proj, self.col_dkv, self.kv_rank, self.rot_dim, self.norm_w, self.eps, cs, ctx.positions,
                             ctx.token_seq, cache.k_pages, cache.block_table, cache.page_size)
        if self.q_rank is None:
            qrows = proj                                             # (its first columns; the kernels take the row stride)
        else:
            qrows = ops.linear(ops.rmsnorm_cols(proj, 0, self.q_rank, self.q_norm_w, self.eps), self.w_uq, None)
        qh = qrows[:, :H * (self.dim + self.rot_dim)].view(T, H, self.dim + self.rot_dim)
        folded = ops.batched_linear(qh[:, :, :self.dim].transpose(0, 1), self.w_uk_t)          # [H, T, rank]
        q = ops.latent_query(qrows, folded, H, self.dim, self.kv_rank, self.rot_dim, R, cs)
        out = torch.empty((T, H * R), dtype=x.dtype, device=x.device)
        classes = ctx.classes()
        if len(classes) == 1:
            c = classes[0]
            ops.paged_attention(q, H, 1, R, cache.k_pages, cache.v_pages, cache.block_table, cache.page_size,
                                c.query_start_loc, ctx.seq_lens, ctx.num_seqs, c.max_q_len, c.max_kv_len,
                                self.scale, self.window or 0, out)
        else:
            for ci, c in enumerate(classes):
                key = ("attention class views", id(cache.block_table), ci)
                views = ctx.step_cache.get(key)
                if views is None:
                    views = ctx.step_cache[key] = (cache.block_table[c.seq_lo:c.seq_hi], ctx.seq_lens[c.seq_lo:c.seq_hi])
                ops.paged_attention(q[c.tok_lo:c.tok_hi], H, 1, R, cache.k_pages, cache.v_pages, views[0], cache.page_size,
                                    c.query_start_loc, views[1], c.seq_hi - c.seq_lo, c.max_q_len, c.max_kv_len,
                                    self.scale, self.window or 0, out[c.tok_lo:c.tok_hi])
        lat = out.view(T, H, R)[:, :, :self.kv_rank].transpose(0, 1)                            # [H, T, rank], a view
        v = ops.batched_linear(lat, self.w_uv)                                                  # [H, T, vdim]
        if self.gated:
            heads = ops.gate_heads(v, proj[:, self.col_g:self.col_g + self.gate_cols], H, self.vdim, per_value=self.gate_per_value)
        else:
            heads = v.transpose(0, 1).reshape(T, H * self.vdim)
        return ops.linear(heads, self.w_out, None, partial_ok=True)
