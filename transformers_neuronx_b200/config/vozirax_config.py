"""Typed configuration of the Vozirax decoder, read from the keys of its own config.json.

    {"architecture": "Vozirax", "vocab": V, "width": W, "norm": {"eps": e}, "logit_scale": s,
     "layers": [{"type": ..., "mixer": {...}, "mlp": {...} | null}, ...]}

A layer's `type` names its mixer:
  'mamba2'     heads, vdim, state, groups, norm_groups, conv (taps)
  'attention'  heads, kv_heads, dim, vdim, scale, diff, optionally q_temp {coef, every} and kv_from (an earlier attention
               layer whose keys and values this layer reads instead of projecting its own)
A layer's `mlp` is {"kind": "dense", "ff": F}, or {"kind": "moe", "expert": {"ff": F}, "router": {"experts": E, "top": k,
"scale": s, optionally "groups": {"count": n, "keep": m}}}, or null.  Every layer carries its own sizes, so layers of
one model may differ.  Nothing has a default but `init_std` (the spread of random weights, used only when a folder is
written from a seed) and `max_positions` (the longest request the engine admits; the design itself has no limit); a
mechanism whose key is absent is not there (`logit_scale` and a router's `scale`: 1; `groups` and `norm_groups` of a
state-space layer: 1; `kv_heads`: as many as heads; `q_temp`, a router's `groups`, `kv_from`: none).
"""
from __future__ import annotations

import copy
import json
import os
from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .model_config import ConfigError

LAYER_TYPES = ("mamba2", "attention")


def _pos_int(d, key, where):
    v = d.get(key)
    if not isinstance(v, int) or isinstance(v, bool) or v <= 0:
        raise ConfigError(f"{where}: key {key!r} must be a positive integer, got {v!r}")
    return v


def _number(d, key, where):
    v = d.get(key)
    if not isinstance(v, (int, float)) or isinstance(v, bool):
        raise ConfigError(f"{where}: key {key!r} must be a number, got {v!r}")
    return float(v)


def _check_mlp(mlp, where):
    if mlp is None:
        return
    if not isinstance(mlp, dict) or mlp.get("kind") not in ("dense", "moe"):
        raise ConfigError(f"{where}: kind must be 'dense' or 'moe' (or the layer's mlp null), got {mlp!r}")
    if mlp["kind"] == "dense":
        _pos_int(mlp, "ff", where)
        return
    if not isinstance(mlp.get("expert"), dict) or not isinstance(mlp.get("router"), dict):
        raise ConfigError(f"{where}: a mixture of experts holds 'expert' and 'router'")
    _pos_int(mlp["expert"], "ff", where + ".expert")
    r, rw = mlp["router"], where + ".router"
    E, top = _pos_int(r, "experts", rw), _pos_int(r, "top", rw)
    if top > E:
        raise ConfigError(f"{rw}: {top} of {E} experts is not a choice")
    if r.get("scale") is not None:
        _number(r, "scale", rw)
    g = r.get("groups")
    if g is not None:
        if not isinstance(g, dict):
            raise ConfigError(f"{rw}: key 'groups' must hold 'count' and 'keep'")
        count, keep = _pos_int(g, "count", rw + ".groups"), _pos_int(g, "keep", rw + ".groups")
        if E % count:
            raise ConfigError(f"{rw}: {E} experts do not form {count} equal groups")
        if keep > count:
            raise ConfigError(f"{rw}: {keep} of {count} groups cannot be kept")
        if keep * (E // count) < top:
            raise ConfigError(f"{rw}: the {keep} kept groups hold fewer than {top} experts")


def _check_layer(i: int, layer: Dict[str, Any], layers) -> None:
    where = f"layers[{i}]"
    if not isinstance(layer, dict) or layer.get("type") not in LAYER_TYPES:
        t = layer.get("type") if isinstance(layer, dict) else layer
        raise ConfigError(f"{where}: unknown layer type {t!r}; known: {', '.join(LAYER_TYPES)}")
    m = layer.get("mixer")
    if not isinstance(m, dict):
        raise ConfigError(f"{where}: key 'mixer' must hold the mixer's sizes")
    mw = where + ".mixer"
    if layer["type"] == "mamba2":
        m.setdefault("groups", 1)             # what the file does not mention is not there: one group of B and C,
        m.setdefault("norm_groups", 1)        # a norm over the whole inner width
        for k in ("heads", "vdim", "state", "groups", "norm_groups", "conv"):
            _pos_int(m, k, mw)
        if m["heads"] % m["groups"]:
            raise ConfigError(f"{mw}: {m['heads']} heads cannot share {m['groups']} groups")
        if (m["heads"] * m["vdim"]) % m["norm_groups"]:
            raise ConfigError(f"{mw}: {m['heads'] * m['vdim']} inner channels do not form {m['norm_groups']} equal parts")
    else:
        if isinstance(m.get("heads"), int):
            m.setdefault("kv_heads", m["heads"])
        for k in ("heads", "kv_heads", "dim", "vdim"):
            _pos_int(m, k, mw)
        if m["heads"] % m["kv_heads"]:
            raise ConfigError(f"{mw}: {m['heads']} heads cannot share {m['kv_heads']} key/value heads")
        if _number(m, "scale", mw) <= 0:
            raise ConfigError(f"{mw}: scale must be positive")
        _number(m, "diff", mw)
        qt = m.get("q_temp")
        if qt is not None:
            if not isinstance(qt, dict):
                raise ConfigError(f"{mw}: key 'q_temp' must hold 'coef' and 'every'")
            _number(qt, "coef", mw + ".q_temp")
            _pos_int(qt, "every", mw + ".q_temp")
        src = m.get("kv_from")
        if src is not None:
            if not isinstance(src, int) or isinstance(src, bool) or not (0 <= src < i):
                raise ConfigError(f"{mw}: kv_from must name an earlier layer, got {src!r}")
            other = layers[src]
            if other.get("type") != "attention" or other["mixer"].get("kv_from") is not None:
                raise ConfigError(f"{mw}: kv_from names layer {src}, which has no keys and values of its own")
            for k in ("kv_heads", "dim", "vdim"):
                if other["mixer"].get(k) != m[k]:
                    raise ConfigError(f"{mw}: {k} differs from that of layer {src}, whose keys and values it reads")
    _check_mlp(layer.get("mlp"), where + ".mlp")


@dataclass(frozen=True, eq=False)
class VoziraxConfig:
    vocab: int
    width: int
    layers: Tuple[Dict[str, Any], ...]
    norm_eps: float
    logit_scale: float
    init_std: float = 0.05
    max_positions: int = 1 << 20
    architecture: str = "Vozirax"

    def __post_init__(self):
        for name in ("vocab", "width", "max_positions"):
            v = getattr(self, name)
            if not isinstance(v, int) or isinstance(v, bool) or v <= 0:
                raise ConfigError(f"config key {name!r} must be a positive integer, got {v!r}")
        if not (self.norm_eps > 0):
            raise ConfigError(f"norm.eps must be positive, got {self.norm_eps!r}")
        if not self.layers:
            raise ConfigError("config key 'layers' must list at least one layer")
        for i, layer in enumerate(self.layers):
            _check_layer(i, layer, self.layers)

    def __eq__(self, other):
        return isinstance(other, VoziraxConfig) and self.to_dict() == other.to_dict()

    # what the engine's front door asks of any configuration
    @property
    def vocab_size(self) -> int:
        return self.vocab

    torch_dtype = "bfloat16"                 # the type the design's checkpoints are stored in

    @property
    def max_position_embeddings(self) -> int:
        return self.max_positions

    eos_token_id: Optional[int] = None
    bos_token_id: Optional[int] = None
    pad_token_id: Optional[int] = None

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "VoziraxConfig":
        missing = [k for k in ("vocab", "width", "layers", "norm") if k not in d]
        if missing:
            raise ConfigError("config.json lacks required key(s): " + ", ".join(missing))
        if not isinstance(d["norm"], dict) or "eps" not in d["norm"]:
            raise ConfigError("config key 'norm' must hold 'eps'")
        if not isinstance(d["layers"], list):
            raise ConfigError("config key 'layers' must be a list")
        kw = dict(vocab=d["vocab"], width=d["width"], layers=tuple(copy.deepcopy(l) for l in d["layers"]),
                  norm_eps=float(d["norm"]["eps"]),
                  logit_scale=_number(d, "logit_scale", "config") if d.get("logit_scale") is not None else 1.0)
        for k in ("init_std", "max_positions"):
            if k in d:
                kw[k] = d[k]
        return cls(**kw)

    @classmethod
    def from_json(cls, path: str) -> "VoziraxConfig":
        with open(path) as fp:
            return cls.from_dict(json.load(fp))

    @classmethod
    def from_pretrained(cls, folder: str) -> "VoziraxConfig":
        return cls.from_json(os.path.join(folder, "config.json"))

    def to_dict(self) -> Dict[str, Any]:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "norm": {"eps": self.norm_eps}, "logit_scale": self.logit_scale,
                "layers": [copy.deepcopy(l) for l in self.layers], "init_std": self.init_std,
                "max_positions": self.max_positions}

    def save(self, folder: str) -> None:
        os.makedirs(folder, exist_ok=True)
        with open(os.path.join(folder, "config.json"), "w") as fp:
            json.dump(self.to_dict(), fp, indent=1)
