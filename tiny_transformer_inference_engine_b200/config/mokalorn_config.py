"""Configuration of the Mokalorn design: a pre-norm decoder whose layers are listed one by one.

config.json keys: ``architecture`` ("Mokalorn"), ``vocab``, ``width``, ``norm.eps``, ``embedding.scale``, ``logit_softcap``
(optional or null: none) and ``layers``, a list with one entry per layer: ``type`` (the mixer: ``attention``, ``attention_2``
or ``retention``), ``mixer`` (its sizes and constants) and ``mlp`` (``kind`` ``moe`` with ``expert.ff``, ``expert.limit``,
``router.experts``, ``router.top`` and ``router.identity``; null or absent: no feed-forward).  Every size and every constant
that can differ between models is read from there; nothing has a default in code.  The design names no longest sequence;
``max_seq_len`` is this engine's own bound on positions (an optional key, else ``DEFAULT_MAX_SEQ_LEN``).
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Any, Dict, Optional, Tuple

from .model_config import ConfigError, register_config
from .munevik_config import _need, _pos_int, DEFAULT_MAX_SEQ_LEN
from .mizupel_config import _pos_num

MIXERS = ("attention", "attention_2", "retention")
MLPS = ("moe",)


def _check_rot(m: dict, where: str):
    rot = m.get("rot")
    if rot is None:
        return
    _need(rot, ("base", "dims"), f"{where}.rot")
    dims = rot["dims"]
    if isinstance(dims, bool) or not isinstance(dims, int) or dims < 0 or dims % 2 or dims > m["dim"]:
        raise ConfigError(f"{where}.rot.dims={dims!r} must be even and at most dim={m['dim']}")
    _pos_num(rot["base"], f"{where}.rot.base")


@register_config("Mokalorn")
@dataclass(frozen=True)
class MokalornConfig:
    vocab: int
    width: int
    layers: Tuple[Dict[str, Any], ...]
    norm_eps: float
    embedding_scale: float
    logit_softcap: Optional[float] = None
    max_seq_len: int = DEFAULT_MAX_SEQ_LEN
    eos_token_id: Optional[int] = None
    architecture: str = "Mokalorn"
    extra: Dict[str, Any] = field(default_factory=dict, compare=False)

    def __post_init__(self):
        _pos_int(self.vocab, "vocab"); _pos_int(self.width, "width"); _pos_int(self.max_seq_len, "max_seq_len")
        _pos_num(self.embedding_scale, "embedding.scale")
        if self.logit_softcap is not None:
            _pos_num(self.logit_softcap, "logit_softcap")
        if not self.layers:
            raise ConfigError("'layers' must list at least one layer")
        for i, L in enumerate(self.layers):
            where = f"layers[{i}]"
            _need(L, ("type", "mixer"), where)
            m, mw = L["mixer"], f"{where}.mixer"
            if L["type"] in ("attention", "attention_2"):
                _need(m, ("heads", "dim", "scale"), mw)               # (kv_heads absent: one per head; vdim absent: dim)
                for k in ("heads", "kv_heads", "dim", "vdim"):
                    if k in m:
                        _pos_int(m[k], f"{mw}.{k}")
                if m["heads"] % m.get("kv_heads", m["heads"]):
                    raise ConfigError(f"{mw}: {m['heads']} heads are not a multiple of {m['kv_heads']} kv_heads")
                _pos_num(m["scale"], f"{mw}.scale")
                if L["type"] == "attention":
                    if m.get("vdim", m["dim"]) != m["dim"]:
                        raise ConfigError(f"{mw}: the values are the keys, so vdim={m['vdim']} must equal dim={m['dim']}")
                    if m.get("mask") is not None:
                        _need(m["mask"], ("size",), f"{mw}.mask")
                        _pos_int(m["mask"]["size"], f"{mw}.mask.size")
                    _check_rot(m, mw)
                elif m.get("q_temp") is not None:
                    _need(m["q_temp"], ("coef", "every"), f"{mw}.q_temp")
                    _pos_int(m["q_temp"]["every"], f"{mw}.q_temp.every")
                    c = m["q_temp"]["coef"]
                    if isinstance(c, bool) or not isinstance(c, (int, float)):
                        raise ConfigError(f"{mw}.q_temp.coef must be a number, got {c!r}")
            elif L["type"] == "retention":
                _need(m, ("heads", "dim", "vdim", "decay"), mw)
                for k in ("heads", "dim", "vdim"):
                    _pos_int(m[k], f"{mw}.{k}")
                decay = m["decay"]
                if not isinstance(decay, (list, tuple)) or len(decay) != m["heads"]:
                    raise ConfigError(f"{mw}.decay must list one decay for each of the {m['heads']} heads")
                for x in decay:
                    if isinstance(x, bool) or not isinstance(x, (int, float)) or not 0 <= x <= 1:
                        raise ConfigError(f"{mw}.decay: {x!r} is not a number in [0, 1]")
                _check_rot(m, mw)
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
                if f["expert"].get("limit") is not None:
                    _pos_num(f["expert"]["limit"], f"{fw}.expert.limit")
                r = f["router"]
                _need(r, ("experts", "top"), f"{fw}.router")
                _pos_int(r["top"], f"{fw}.router.top")
                for k in ("experts", "identity"):
                    v = r.get(k, 0)
                    if isinstance(v, bool) or not isinstance(v, int) or v < 0:
                        raise ConfigError(f"{fw}.router.{k} must be a non-negative integer, got {v!r}")
                if r["top"] > r["experts"] + r.get("identity", 0):
                    raise ConfigError(f"{fw}.router: top={r['top']} of {r['experts']} + {r.get('identity', 0)} experts")

    # the names the engine asks every configuration for
    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def d_model(self) -> int:
        return self.width

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "MokalornConfig":
        raw = dict(raw)
        _need(raw, ("vocab", "width", "layers", "norm", "embedding"), "config.json")
        _need(raw["norm"], ("eps",), "config.json 'norm'")
        _need(raw["embedding"], ("scale",), "config.json 'embedding'")
        raw.pop("architecture", None)
        kw = dict(vocab=raw.pop("vocab"), width=raw.pop("width"), layers=tuple(raw.pop("layers")),
                  norm_eps=float(raw.pop("norm")["eps"]), embedding_scale=raw.pop("embedding")["scale"],
                  logit_softcap=raw.pop("logit_softcap", None))
        if "max_seq_len" in raw:
            kw["max_seq_len"] = raw.pop("max_seq_len")
        if "eos_token_id" in raw:
            kw["eos_token_id"] = raw.pop("eos_token_id")
        return cls(extra=raw, **kw)

    def to_dict(self) -> Dict[str, Any]:
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "layers": list(self.layers),
             "norm": {"eps": self.norm_eps}, "embedding": {"scale": self.embedding_scale}, "logit_softcap": self.logit_softcap}
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
