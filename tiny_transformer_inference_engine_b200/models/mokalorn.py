"""The Mokalorn design as data: a pre-norm decoder that mixes two kinds of softmax attention with retention, and whose
feed-forwards are mixtures of experts with identity experts among them.

Token embedding times ``embedding.scale``; pre-norm layers (``x += mixer(rms_norm(x))`` and, where the layer has one,
``x += ff(rms_norm(x))``); the model's RMS norm; logits from an untied head, soft-capped.  The mixer of a layer is

* ``attention``: grouped-query attention without a value projection (a value head is its key head as projected), RMS norm
  with a shared weight on every query and key head, a rotation of the first ``rot.dims`` values of every head (pairs
  ``(2i, 2i+1)``), a chunked mask (a token sees the earlier tokens of its own chunk of ``mask.size`` positions), one
  sigmoid gate per value of the concatenated heads;
* ``attention_2``: the same with a value projection, no rotation, a causal mask over all keys, and queries scaled by a
  temperature that grows with the logarithm of the position;
* ``retention``: linear attention with a fixed decay per head and a matrix state (``parts/retention.py``).

The feed-forward routes every token to ``top`` of ``experts + identity`` experts by the softmax of the router's logits plus a
correction that only the choice sees; the weights are the chosen softmax values, not renormalised; an identity expert returns
its input.  Tensor names: ``embed``, ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.*``, ``l<i>.mlp.router``, ``.correction``,
``.e<j>.gate`` / ``.up`` / ``.down``, ``final.norm``, ``head``.

Constants the design fixes (not in config.json): the experts' activation ``g sigmoid(1.702 g) (u + 1)``, the pairings of
rotated values (interleaved in attention, half-split in retention), silu as retention's gate, one group of experts.
"""
from __future__ import annotations

from ..config.mokalorn_config import MokalornConfig
from ..parts.base import PartSpec, LayerSpec, RunEntry, ModelSpec
from ..registry import register_model

EXPERT_ALPHA, EXPERT_SHIFT = 1.702, 1.0
ATTENTION_ROTARY_STYLE = "interleaved"
RETENTION_ROTARY_STYLE = "half"
RETENTION_GATE = "silu"


def _norm(prefix: str, name: str, d: int, eps: float) -> PartSpec:
    return PartSpec("rmsnorm", prefix, {"dim": d, "eps": eps, "name": name})


def _position(m: dict, style: str) -> PartSpec:
    rot = m.get("rot")
    if rot is not None and rot["dims"] > 0:
        return PartSpec("rope", "", {"dim": rot["dims"], "base": rot["base"], "style": style})
    return PartSpec("none", "", {})


def _mixer(L: dict, p: str, d: int, eps: float) -> PartSpec:
    m = L["mixer"]
    if L["type"] == "retention":
        return PartSpec("retention", f"{p}.mix", {
            "d_model": d, "num_heads": m["heads"], "dim": m["dim"], "vdim": m["vdim"], "decay": tuple(m["decay"]), "eps": eps,
            "position": _position(m, RETENTION_ROTARY_STYLE), "gate_act": RETENTION_GATE})
    first = L["type"] == "attention"                                  # else "attention_2"
    mask = m.get("mask") if first else None
    return PartSpec("attention", f"{p}.mix", {
        "d_model": d, "num_heads": m["heads"], "num_kv_heads": m.get("kv_heads", m["heads"]), "head_dim": m["dim"],
        "v_head_dim": m.get("vdim", m["dim"]),
        "position": _position(m, ATTENTION_ROTARY_STYLE) if first else PartSpec("none", "", {}),
        "chunk": None if mask is None else mask["size"], "scale": m["scale"], "gated": "value", "qk_norm": eps,
        "v_from_k": first, "q_temp": None if first else m.get("q_temp"),
        "names": {"q": "q", "k": "k", "v": "v", "o": "o", "g": "g"}, "weight_suffix": "", "norm_suffix": ".norm"})


def _ffn(f, p: str, d: int):
    if f is None:
        return None
    r = f["router"]
    return PartSpec("grouped_moe", f"{p}.mlp", {
        "d_model": d, "hidden": f["expert"]["ff"], "experts": r["experts"], "identity": r.get("identity", 0), "top": r["top"],
        "groups": 1, "keep": 1, "group_top": 1, "scale": 1.0, "renorm": False, "score": "softmax", "correction": True,
        "alpha": EXPERT_ALPHA, "limit": f["expert"].get("limit"), "shift": EXPERT_SHIFT})


@register_model("Mokalorn")
def mokalorn(config: MokalornConfig) -> ModelSpec:
    d, eps = config.width, config.norm_eps
    layers, run_order = [], []
    for i, L in enumerate(config.layers):
        p = f"l{i}"
        ffn = _ffn(L.get("mlp"), p, d)
        block = PartSpec("pre_norm", p, {
            "mixer_norm": _norm(p, "norm1", d, eps), "mixer": _mixer(L, p, d, eps),
            "ffn_norm": None if ffn is None else _norm(p, "norm2", d, eps), "ffn": ffn})
        layers.append(LayerSpec(block))
        run_order.append(RunEntry(i))
    return ModelSpec(
        d_model=d, vocab_size=config.vocab, max_seq_len=config.max_seq_len,
        embedding=PartSpec("token", "", {"vocab_size": config.vocab, "dim": d, "name": "embed", "scale": config.embedding_scale}),
        layers=tuple(layers), run_order=tuple(run_order),
        final_norm=_norm("final", "norm", d, eps),
        head=PartSpec("linear", "", {"dim": d, "vocab_size": config.vocab, "name": "head", "softcap": config.logit_softcap}),
        eos_token_id=config.eos_token_id,
    )
