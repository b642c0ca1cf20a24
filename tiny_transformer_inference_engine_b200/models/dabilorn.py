"""The Dabilorn design as data: a decoder whose sub-layers read the residual stream itself and are normed on the way out.

Token embedding, then the model's norm (``embed.norm``).  A layer is ``x += ls1 * LN(mixer(x + conv(x)))`` and, where it has a
feed-forward, ``x += ls2 * LN(ff(x))``: LayerNorm with a weight and no bias on the sub-layer's OUTPUT, a layer scale per
channel behind it, and in front of the mixer a causal convolution over time on every channel (``canon1``, ``canon.taps``
taps, added to its input).  The model's norm (``final.norm``) and logits from the embedding table end it.  The mixer is

* ``latent_attention``: queries through a normed low-rank latent, keys and values from a normed low-rank latent plus one
  rotated key part shared by the heads (only those two are cached), interleaved rotation with YaRN-rescaled frequencies,
  causal softmax, a sigmoid gate per value of the concatenated heads (``parts/latent_attention.py``);
* ``attention``: grouped-query attention with one RMS norm over all of q and one over all of k, a rotation in half-split
  pairs, a chunked mask, and ``sigmoid(score + bias_h)`` as the weight of a visible key instead of a softmax, gated per value
  (``parts/attention.py``);
* ``wkv``: RWKV-style time mixing with a token-dependent decay (``parts/wkv.py``).

The feed-forward routes every token to ``top`` of ``experts`` by the sigmoid of the router's logits; the chosen score multiplies
the expert's INPUT; an expert is ``W_down relu(W_up h)^2``; a shared expert of the same form runs for every token and is scaled
by ``sigmoid(w_sg . h)``.  Tensor names: ``embed``, ``embed.norm``, ``l<i>.norm1`` / ``.norm2``, ``.ls1`` / ``.ls2``,
``.canon1``, ``l<i>.mix.*``, ``l<i>.mlp.router``, ``.e<j>.up`` / ``.down``, ``.shared.up`` / ``.down`` / ``.sg``, ``final.norm``.

Constants the design fixes (not in config.json): the experts' activation, the two pairings of rotated values, sigmoid router
scores that are not renormalised, silu as the time mixing's gate (in its part), YaRN's magnitude ``0.1 ln(factor) + 1`` (in
the rotation part).
"""
from __future__ import annotations

from ..config.dabilorn_config import DabilornConfig
from ..parts.base import PartSpec, LayerSpec, RunEntry, ModelSpec
from ..registry import register_model

EXPERT_ACTIVATION = "relu2"
LATENT_ROTARY_STYLE = "interleaved"
ATTENTION_ROTARY_STYLE = "half"


def _norm(prefix: str, name: str, d: int, eps: float, scale: str = None) -> PartSpec:
    """LayerNorm with a weight and no bias; ``scale``: the layer scale behind it."""
    return PartSpec("layernorm", prefix, {"dim": d, "eps": eps, "names": {"weight": name}, "bias": False, "scale": scale})


def _position(m: dict, style: str) -> PartSpec:
    rot = m.get("rot")
    if rot is None or not rot["dims"]:
        return PartSpec("none", "", {})
    sc = rot.get("scaling")
    scaling = None if sc is None else {"kind": "yarn", "factor": sc["factor"], "original": sc["original"],
                                       "fast": sc["fast"], "slow": sc["slow"]}
    return PartSpec("rope", "", {"dim": rot["dims"], "base": rot["base"], "style": style, "scaling": scaling})


def _mixer(L: dict, p: str, d: int, eps: float) -> PartSpec:
    m = L["mixer"]
    if L["type"] == "wkv":
        return PartSpec("wkv", f"{p}.mix", {"d_model": d, "num_heads": m["heads"], "dim": m["dim"], "eps": eps,
                                            "decay_rank": m.get("decay_rank")})
    if L["type"] == "latent_attention":
        return PartSpec("latent_attention", f"{p}.mix", {
            "d_model": d, "num_heads": m["heads"], "dim": m["dim"], "rot_dim": m["rot_dim"], "vdim": m["vdim"],
            "kv_rank": m["kv_rank"], "q_rank": m["q_rank"], "scale": m["scale"], "eps": eps, "window": None, "gated": "value",
            "position": _position(m, LATENT_ROTARY_STYLE)})
    mask = m.get("mask")
    return PartSpec("attention", f"{p}.mix", {
        "d_model": d, "num_heads": m["heads"], "num_kv_heads": m.get("kv_heads", m["heads"]), "head_dim": m["dim"],
        "v_head_dim": m.get("vdim", m["dim"]), "position": _position(m, ATTENTION_ROTARY_STYLE),
        "chunk": None if mask is None else mask["size"], "scale": m["scale"], "gated": "value", "qk_norm": eps,
        "qk_norm_over": "projection", "weights": "sigmoid", "head_bias": "pb",
        "names": {"q": "q", "k": "k", "v": "v", "o": "o", "g": "g"}, "weight_suffix": "", "norm_suffix": ".norm"})


def _ffn(f, p: str, d: int):
    if f is None:
        return None
    r, shared = f["router"], f.get("shared")
    return PartSpec("grouped_moe", f"{p}.mlp", {
        "d_model": d, "hidden": f["expert"]["ff"], "experts": r["experts"], "top": r["top"], "groups": 1, "keep": 1,
        "group_top": 1, "scale": 1.0, "renorm": False, "score": "sigmoid", "expert": "mlp", "act": EXPERT_ACTIVATION,
        "weight_on": "input",
        "shared": None if shared is None else PartSpec("mlp", f"{p}.mlp.shared", {"d_model": d, "hidden": shared["ff"],
                                                                                  "act": EXPERT_ACTIVATION}),
        "shared_gate": None if shared is None else "shared.sg"})


@register_model("Dabilorn")
def dabilorn(config: DabilornConfig) -> ModelSpec:
    d, eps = config.width, config.norm_eps
    layers, run_order = [], []
    for i, L in enumerate(config.layers):
        p = f"l{i}"
        ffn = _ffn(L.get("mlp"), p, d)
        block = PartSpec("sublayer_norm", p, {
            "dim": d, "mixer": _mixer(L, p, d, eps), "mixer_norm": _norm(p, "norm1", d, eps, scale="ls1"),
            "ffn": ffn, "ffn_norm": None if ffn is None else _norm(p, "norm2", d, eps, scale="ls2"),
            "input_conv": None if config.canon_taps is None else {"name": "canon1", "taps": config.canon_taps}})
        layers.append(LayerSpec(block))
        run_order.append(RunEntry(i))
    return ModelSpec(
        d_model=d, vocab_size=config.vocab, max_seq_len=config.max_seq_len,
        embedding=PartSpec("token", "", {"vocab_size": config.vocab, "dim": d, "name": "embed",
                                         "norm": _norm("embed", "norm", d, eps)}),
        layers=tuple(layers), run_order=tuple(run_order),
        final_norm=_norm("final", "norm", d, eps),
        head=PartSpec("tied", "", {"dim": d, "vocab_size": config.vocab}),
        eos_token_id=config.eos_token_id,
    )
