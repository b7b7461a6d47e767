"""Typed configuration of the Tutelix decoder, read from the keys of its own config.json.

    {"architecture": "Tutelix", "vocab": V, "width": W, "embedding": {"scale": s}, "norm": {"eps": e},
     "loop": {"start": a, "stop": b, "times": n},
     "layers": [{"type": ..., "mixer": {...}, "mlp": {"kind": "dense", "ff": F} | null}, ...]}

A layer's `type` names its mixer:
  'attention'         heads, kv_heads, dim, vdim (= dim: the values are the keys), scale, rot {dims, base}, mask {size}
  'latent_attention'  heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, rot {dims (= rot_dim), base}, mask {size}
  'channel_delta'     heads, kv_heads, dim, vdim, conv (taps); optionally decay_rank and gate_rank, the inner sizes of
                      its two low-rank projections, which are otherwise those of the stored tensors
`mask` absent: every earlier position is read; `rot` absent: no rotation.  `loop` (optional): layers start .. stop - 1
run `times` times in a row with the same weights.  Every layer carries its own sizes, so layers of one model may differ.
Nothing has a default but `init_std` (the spread of random weights, used only when a folder is written from a seed)
and `max_positions` (the longest request the engine admits; the design itself has no limit).
"""
from __future__ import annotations

import copy
import json
import os
from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .model_config import ConfigError

LAYER_TYPES = ("attention", "latent_attention", "channel_delta")


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


def _check_mask(m, where):
    mask = m.get("mask")
    if mask is not None:
        if not isinstance(mask, dict):
            raise ConfigError(f"{where}: key 'mask' must hold 'size'")
        _pos_int(mask, "size", where + ".mask")


def _check_rot(m, where, most):
    r = m.get("rot")
    if r is None:
        return 0
    if not isinstance(r, dict):
        raise ConfigError(f"{where}: key 'rot' must hold 'dims' and 'base'")
    dims = r.get("dims")
    if not isinstance(dims, int) or isinstance(dims, bool) or dims < 0 or dims % 2 or dims > most:
        raise ConfigError(f"{where}: rot.dims must be even and at most {most}, got {dims!r}")
    if _number(r, "base", where + ".rot") <= 1:
        raise ConfigError(f"{where}: rot.base must be larger than 1")
    return dims


def _check_layer(i: int, layer: Dict[str, Any]) -> None:
    where = f"layers[{i}]"
    if not isinstance(layer, dict) or layer.get("type") not in LAYER_TYPES:
        t = layer.get("type") if isinstance(layer, dict) else layer
        raise ConfigError(f"{where}: unknown layer type {t!r}; known: {', '.join(LAYER_TYPES)}")
    m = layer.get("mixer")
    if not isinstance(m, dict):
        raise ConfigError(f"{where}: key 'mixer' must hold the mixer's sizes")
    mw, kind = where + ".mixer", layer["type"]
    for k in ("heads", "dim", "vdim"):
        _pos_int(m, k, mw)
    if kind in ("attention", "channel_delta"):
        _pos_int(m, "kv_heads", mw)
        if m["heads"] % m["kv_heads"]:
            raise ConfigError(f"{mw}: {m['heads']} heads cannot share {m['kv_heads']} key heads")
    if kind in ("attention", "latent_attention"):
        if _number(m, "scale", mw) <= 0:
            raise ConfigError(f"{mw}: scale must be positive")
        _check_mask(m, mw)
    if kind == "attention":
        if m["vdim"] != m["dim"]:
            raise ConfigError(f"{mw}: the values are the keys, so vdim must equal dim ({m['vdim']} and {m['dim']})")
        _check_rot(m, mw, m["dim"])
    elif kind == "latent_attention":
        for k in ("q_rank", "kv_rank"):
            _pos_int(m, k, mw)
        rd = m.get("rot_dim")
        if not isinstance(rd, int) or isinstance(rd, bool) or rd < 0 or rd % 2:
            raise ConfigError(f"{mw}: rot_dim must be an even number of dims (0: none), got {rd!r}")
        if _check_rot(m, mw, max(rd, 0)) != rd:
            raise ConfigError(f"{mw}: rot.dims must equal rot_dim (the rotated part is turned as a whole)")
    else:
        conv = m.get("conv")
        if not isinstance(conv, int) or isinstance(conv, bool) or conv < 1:
            raise ConfigError(f"{mw}: conv must be a number of taps (1: the current token only), got {conv!r}")
        for k in ("decay_rank", "gate_rank"):
            if m.get(k) is not None:
                _pos_int(m, k, mw)
    mlp = layer.get("mlp")
    if mlp is not None:
        fw = where + ".mlp"
        if not isinstance(mlp, dict) or mlp.get("kind") != "dense":
            raise ConfigError(f"{fw}: kind must be 'dense' (or the layer's mlp null), got {mlp!r}")
        _pos_int(mlp, "ff", fw)


@dataclass(frozen=True, eq=False)
class TutelixConfig:
    vocab: int
    width: int
    layers: Tuple[Dict[str, Any], ...]
    norm_eps: float
    embedding_scale: float
    loop: Optional[Dict[str, int]] = None
    init_std: float = 0.05
    max_positions: int = 1 << 20
    architecture: str = "Tutelix"

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
            _check_layer(i, layer)
        if self.loop is not None:
            lp = self.loop
            if not isinstance(lp, dict):
                raise ConfigError("config key 'loop' must hold start, stop and times")
            for k in ("start", "stop", "times"):
                v = lp.get(k)
                if not isinstance(v, int) or isinstance(v, bool) or v < 0:
                    raise ConfigError(f"loop: key {k!r} must be a non-negative integer, got {v!r}")
            if not (lp["start"] <= lp["stop"] <= len(self.layers)):
                raise ConfigError(f"loop: layers {lp['start']} .. {lp['stop']} - 1 are not a run of the model's "
                                  f"{len(self.layers)} layers")
            if lp["times"] < 1:
                raise ConfigError("loop: times must be at least 1")

    def __eq__(self, other):
        return isinstance(other, TutelixConfig) and self.to_dict() == other.to_dict()

    def layer_order(self):
        """The layers' indices in the order they run: the looped run repeated `times` times."""
        n = len(self.layers)
        if self.loop is None:
            return list(range(n))
        a, b, t = self.loop["start"], self.loop["stop"], self.loop["times"]
        return list(range(a)) + list(range(a, b)) * t + list(range(b, n))

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
    def from_dict(cls, d: Dict[str, Any]) -> "TutelixConfig":
        missing = [k for k in ("vocab", "width", "layers", "norm", "embedding") if k not in d]
        if missing:
            raise ConfigError("config.json lacks required key(s): " + ", ".join(missing))
        if not isinstance(d["norm"], dict) or "eps" not in d["norm"]:
            raise ConfigError("config key 'norm' must hold 'eps'")
        if not isinstance(d["embedding"], dict):
            raise ConfigError("config key 'embedding' must hold 'scale'")
        if not isinstance(d["layers"], list):
            raise ConfigError("config key 'layers' must be a list")
        kw = dict(vocab=d["vocab"], width=d["width"], layers=tuple(copy.deepcopy(l) for l in d["layers"]),
                  norm_eps=float(d["norm"]["eps"]), embedding_scale=_number(d["embedding"], "scale", "config.embedding"),
                  loop=copy.deepcopy(d["loop"]) if d.get("loop") is not None else None)
        for k in ("init_std", "max_positions"):
            if k in d:
                kw[k] = d[k]
        return cls(**kw)

    @classmethod
    def from_json(cls, path: str) -> "TutelixConfig":
        with open(path) as fp:
            return cls.from_dict(json.load(fp))

    @classmethod
    def from_pretrained(cls, folder: str) -> "TutelixConfig":
        return cls.from_json(os.path.join(folder, "config.json"))

    def to_dict(self) -> Dict[str, Any]:
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
             "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.norm_eps},
             "layers": [copy.deepcopy(l) for l in self.layers], "init_std": self.init_std,
             "max_positions": self.max_positions}
        if self.loop is not None:
            d["loop"] = copy.deepcopy(self.loop)
        return d

    def save(self, folder: str) -> None:
        os.makedirs(folder, exist_ok=True)
        with open(os.path.join(folder, "config.json"), "w") as fp:
            json.dump(self.to_dict(), fp, indent=1)
