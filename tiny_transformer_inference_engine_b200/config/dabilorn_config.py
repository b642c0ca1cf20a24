"""Configuration of the Dabilorn design: a decoder whose sub-layers read the residual stream itself and whose outputs are
normed before they are added; its layers are listed one by one.

config.json keys: ``architecture`` ("Dabilorn"), ``vocab``, ``width``, ``norm.eps``, ``canon.taps`` (taps of the causal
convolution over time in front of every mixer; ``canon`` absent or null: none) and ``layers``, a list with one entry per
layer: ``type`` (the mixer: ``latent_attention``, ``attention`` or ``wkv``), ``mixer`` (its sizes and constants) and ``mlp``
(``kind`` ``moe`` with ``expert.ff``, ``router.experts``, ``router.top`` and optionally ``shared.ff``; null or absent: no
feed-forward).  Every size and every constant that can differ between models is read from there; nothing has a default in
code.  The design names no longest sequence; ``max_seq_len`` is this engine's own bound on positions (an optional key, else
``DEFAULT_MAX_SEQ_LEN``).  A ``wkv`` mixer may name ``decay_rank``, the width of its decay's low-rank path; without the key
the weight file decides (random weights can then not be drawn).
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Any, Dict, Optional, Tuple

from .model_config import ConfigError, register_config
from .munevik_config import _need, _pos_int, DEFAULT_MAX_SEQ_LEN
from .mizupel_config import _pos_num

MIXERS = ("latent_attention", "attention", "wkv")
MLPS = ("moe",)
YARN_KEYS = ("factor", "original", "fast", "slow")


def _check_rot(m: dict, where: str, limit: int, scaling: bool):
    rot = m.get("rot")
    if rot is None:
        return
    _need(rot, ("base", "dims"), f"{where}.rot")
    dims = rot["dims"]
    if isinstance(dims, bool) or not isinstance(dims, int) or dims < 0 or dims % 2 or dims > limit:
        raise ConfigError(f"{where}.rot.dims={dims!r} must be even and at most {limit}")
    _pos_num(rot["base"], f"{where}.rot.base")
    sc = rot.get("scaling")
    if sc is not None:
        if not scaling:
            raise ConfigError(f"{where}.rot.scaling: this mixer's rotation has no rescaled frequencies")
        _need(sc, YARN_KEYS, f"{where}.rot.scaling")
        for k in YARN_KEYS:
            _pos_num(sc[k], f"{where}.rot.scaling.{k}")
        if rot["base"] == 1:
            raise ConfigError(f"{where}.rot: rescaled frequencies need a base other than 1")


@register_config("Dabilorn")
@dataclass(frozen=True)
class DabilornConfig:
    vocab: int
    width: int
    layers: Tuple[Dict[str, Any], ...]
    norm_eps: float
    canon_taps: Optional[int] = None
    max_seq_len: int = DEFAULT_MAX_SEQ_LEN
    eos_token_id: Optional[int] = None
    architecture: str = "Dabilorn"
    extra: Dict[str, Any] = field(default_factory=dict, compare=False)

    def __post_init__(self):
        _pos_int(self.vocab, "vocab"); _pos_int(self.width, "width"); _pos_int(self.max_seq_len, "max_seq_len")
        if self.canon_taps is not None:
            _pos_int(self.canon_taps, "canon.taps")
        if not self.layers:
            raise ConfigError("'layers' must list at least one layer")
        for i, L in enumerate(self.layers):
            where = f"layers[{i}]"
            _need(L, ("type", "mixer"), where)
            m, mw = L["mixer"], f"{where}.mixer"
            if L["type"] == "latent_attention":
                _need(m, ("heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank", "scale"), mw)
                for k in ("heads", "dim", "vdim", "kv_rank", "q_rank"):
                    _pos_int(m[k], f"{mw}.{k}")
                r = m["rot_dim"]
                if isinstance(r, bool) or not isinstance(r, int) or r < 0 or r % 2:
                    raise ConfigError(f"{mw}.rot_dim={r!r} must be even and not negative")
                _pos_num(m["scale"], f"{mw}.scale")
                if r:
                    _need(m, ("rot",), mw)
                    _check_rot(m, mw, r, scaling=True)
                    if m["rot"]["dims"] != r:
                        raise ConfigError(f"{mw}: the rotated part has rot_dim={r} values, rot.dims says {m['rot']['dims']}")
            elif L["type"] == "attention":
                _need(m, ("heads", "dim", "scale"), mw)               # (kv_heads absent: one per head; vdim absent: dim)
                for k in ("heads", "kv_heads", "dim", "vdim"):
                    if k in m:
                        _pos_int(m[k], f"{mw}.{k}")
                if m["heads"] % m.get("kv_heads", m["heads"]):
                    raise ConfigError(f"{mw}: {m['heads']} heads are not a multiple of {m['kv_heads']} kv_heads")
                _pos_num(m["scale"], f"{mw}.scale")
                if m.get("mask") is not None:
                    _need(m["mask"], ("size",), f"{mw}.mask")
                    _pos_int(m["mask"]["size"], f"{mw}.mask.size")
                _check_rot(m, mw, m["dim"], scaling=False)
            elif L["type"] == "wkv":
                _need(m, ("heads", "dim"), mw)
                for k in ("heads", "dim"):
                    _pos_int(m[k], f"{mw}.{k}")
                if m.get("decay_rank") is not None:
                    _pos_int(m["decay_rank"], f"{mw}.decay_rank")
            else:
                raise ConfigError(f"{where}.type {L['type']!r} unknown; known: {MIXERS}")
            f = L.get("mlp")
            if f is not None:
                fw = f"{where}.mlp"
                _need(f, ("kind",), fw)
                if f["kind"] != "moe":
                    raise ConfigError(f"{fw}.kind {f['kind']!r} unknown; known: {MLPS}")
                _need(f, ("expert", "router"), fw)
                _need(f["expert"], ("ff",), f"{fw}.expert")
                _pos_int(f["expert"]["ff"], f"{fw}.expert.ff")
                r = f["router"]
                _need(r, ("experts", "top"), f"{fw}.router")
                _pos_int(r["experts"], f"{fw}.router.experts")
                _pos_int(r["top"], f"{fw}.router.top")
                if r["top"] > r["experts"]:
                    raise ConfigError(f"{fw}.router: top={r['top']} of {r['experts']} experts")
                if f.get("shared") is not None:
                    _need(f["shared"], ("ff",), f"{fw}.shared")
                    _pos_int(f["shared"]["ff"], f"{fw}.shared.ff")

    # the names the engine asks every configuration for
    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def d_model(self) -> int:
        return self.width

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "DabilornConfig":
        raw = dict(raw)
        _need(raw, ("vocab", "width", "layers", "norm"), "config.json")
        _need(raw["norm"], ("eps",), "config.json 'norm'")
        raw.pop("architecture", None)
        canon = raw.pop("canon", None)
        if canon is not None:
            _need(canon, ("taps",), "config.json 'canon'")
        kw = dict(vocab=raw.pop("vocab"), width=raw.pop("width"), layers=tuple(raw.pop("layers")),
                  norm_eps=float(raw.pop("norm")["eps"]), canon_taps=None if canon is None else canon["taps"])
        if "max_seq_len" in raw:
            kw["max_seq_len"] = raw.pop("max_seq_len")
        if "eos_token_id" in raw:
            kw["eos_token_id"] = raw.pop("eos_token_id")
        return cls(extra=raw, **kw)

    def to_dict(self) -> Dict[str, Any]:
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "layers": list(self.layers),
             "norm": {"eps": self.norm_eps}}
        if self.canon_taps is not None:
            d["canon"] = {"taps": self.canon_taps}
        if self.max_seq_len != DEFAULT_MAX_SEQ_LEN:
            d["max_seq_len"] = self.max_seq_len
        if self.eos_token_id is not None:
            d["eos_token_id"] = self.eos_token_id
        d.update({k: v for k, v in self.extra.items() if k not in d})
        return d

    def save(self, folder: str) -> str:
        os.makedirs(folder, exist_ok=True)
        path = os.path.join(folder, "config.json")
        with open(path, "w", encoding="utf-8") as f:
            json.dump(self.to_dict(), f, indent=2, sort_keys=True)
        return path
