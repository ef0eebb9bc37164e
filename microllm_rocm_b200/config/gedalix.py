"""Typed configuration of the Gedalix decoder, read from its own config.json keys.

  architecture            "Gedalix"
  vocab, width            vocabulary and residual width
  max_positions           rows of the learned position table
  embedding.scale         factor on the embedded token
  norm.eps                eps of every RMS norm of the model
  residual_mult           factor on everything a layer adds to the residual stream
  layers[i]               type (the mixer's kind), mixer (its sizes), mlp (the feed-forward, or null for none)
  loop                    {start, stop, times}: layers start..stop-1 run `times` times in a row, each pass with a
                          cache of its own; absent or null: every layer runs once

Mixer "latent_attention": heads, dim, rot_dim, vdim, kv_rank, scale, rot {base, dims}.
Feed-forward kind "moe": router {experts, top}, expert {ff}, shared {ff} (optional).
Every size and constant comes from here or from a tensor's shape; nothing in the engine carries one.
"""
from __future__ import annotations

import copy
import json
import math
import os
from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .qwen2 import ConfigError

ARCHITECTURE = "Gedalix"
MIXER_KINDS = ("latent_attention",)
FEED_FORWARD_KINDS = ("moe",)


def _positive_int(value, what: str) -> int:
    if not isinstance(value, int) or isinstance(value, bool) or value <= 0:
        raise ConfigError(f"{what} must be a positive integer, got {value!r}")
    return value


def _number(value, what: str, positive: bool = False) -> float:
    if isinstance(value, bool) or not isinstance(value, (int, float)) or not math.isfinite(value) or (positive and value <= 0):
        raise ConfigError(f"{what} must be a finite{' positive' if positive else ''} number, got {value!r}")
    return float(value)


@dataclass(frozen=True)
class GedalixConfig:
    vocab: int
    width: int
    max_positions: int
    embedding_scale: float
    norm_eps: float
    residual_mult: float
    layers: Tuple[Dict[str, Any], ...]
    loop: Optional[Tuple[int, int, int]] = None          # (start, stop, times)
    torch_dtype: str = "bfloat16"

    # ---- what the engine asks of any configuration ------------------------------------
    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def max_position_embeddings(self) -> int:
        return self.max_positions

    eos_token_id = None

    def run_order(self):
        """[(layer, pass number if the run opens a pass, else None)] in execution order."""
        n = len(self.layers)
        if self.loop is None:
            return [(i, None) for i in range(n)]
        start, stop, times = self.loop
        order = [(i, None) for i in range(start)]
        for t in range(times):
            order += [(i, t if i == start else None) for i in range(start, stop)]
        return order + [(i, None) for i in range(stop, n)]

    # ---- validation ----------------------------------------------------------------
    def validate(self) -> None:
        _positive_int(self.vocab, "vocab"); _positive_int(self.width, "width"); _positive_int(self.max_positions, "max_positions")
        _number(self.embedding_scale, "embedding.scale"); _number(self.norm_eps, "norm.eps", positive=True)
        _number(self.residual_mult, "residual_mult")
        if not self.layers:
            raise ConfigError("layers must list at least one layer")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            if layer.get("type") not in MIXER_KINDS:
                raise ConfigError(f"{where}.type {layer.get('type')!r} is not one of {', '.join(MIXER_KINDS)}")
            mixer = layer.get("mixer")
            if not isinstance(mixer, dict):
                raise ConfigError(f"{where}.mixer is missing")
            for key in ("heads", "dim", "vdim", "kv_rank"):
                _positive_int(mixer.get(key), f"{where}.mixer.{key}")
            rot_dim = mixer.get("rot_dim")
            if not isinstance(rot_dim, int) or isinstance(rot_dim, bool) or rot_dim < 0:
                raise ConfigError(f"{where}.mixer.rot_dim must be a non-negative integer")
            _number(mixer.get("scale"), f"{where}.mixer.scale", positive=True)
            rot = mixer.get("rot") or {}
            if rot_dim:
                _number(rot.get("base"), f"{where}.mixer.rot.base", positive=True)
                dims = rot.get("dims", rot_dim)
                if not isinstance(dims, int) or dims <= 0 or dims % 2 or dims > rot_dim:
                    raise ConfigError(f"{where}.mixer.rot.dims must be even, positive and at most rot_dim")
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            if mlp.get("kind") not in FEED_FORWARD_KINDS:
                raise ConfigError(f"{where}.mlp.kind {mlp.get('kind')!r} is not one of {', '.join(FEED_FORWARD_KINDS)}")
            router = mlp.get("router") or {}
            experts = _positive_int(router.get("experts"), f"{where}.mlp.router.experts")
            top = _positive_int(router.get("top"), f"{where}.mlp.router.top")
            if top > experts:
                raise ConfigError(f"{where}.mlp.router.top exceeds the number of experts")
            _positive_int((mlp.get("expert") or {}).get("ff"), f"{where}.mlp.expert.ff")
            if mlp.get("shared") is not None:
                _positive_int(mlp["shared"].get("ff"), f"{where}.mlp.shared.ff")
        if self.loop is not None:
            start, stop, times = self.loop
            if not (0 <= start < stop <= len(self.layers)) or times < 1:
                raise ConfigError(f"loop {{start {start}, stop {stop}, times {times}}} does not fit {len(self.layers)} layers")

    # ---- (de)serialisation -----------------------------------------------------------
    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "GedalixConfig":
        missing = [k for k in ("vocab", "width", "max_positions", "layers", "norm", "residual_mult", "embedding") if k not in raw]
        if missing:
            raise ConfigError("config.json is missing " + ", ".join(missing))
        loop = raw.get("loop")
        if loop is not None:
            for k in ("start", "stop", "times"):
                if not isinstance(loop.get(k), int) or isinstance(loop.get(k), bool):
                    raise ConfigError(f"loop.{k} must be an integer")
            loop = (loop["start"], loop["stop"], loop["times"])
        if not isinstance(raw["layers"], list):
            raise ConfigError("layers must be a list")
        cfg = cls(vocab=raw["vocab"], width=raw["width"], max_positions=raw["max_positions"],
                  embedding_scale=(raw["embedding"] or {}).get("scale", 1.0), norm_eps=(raw["norm"] or {}).get("eps"),
                  residual_mult=raw["residual_mult"], layers=tuple(copy.deepcopy(l) for l in raw["layers"]), loop=loop,
                  torch_dtype=raw.get("torch_dtype", "bfloat16"))
        cfg.validate()
        return cfg

    @classmethod
    def from_json(cls, path: str) -> "GedalixConfig":
        if os.path.isdir(path):
            path = os.path.join(path, "config.json")
        with open(path, "r", encoding="utf-8") as f:
            return cls.from_dict(json.load(f))

    def to_dict(self) -> Dict[str, Any]:
        d = {"architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width, "max_positions": self.max_positions,
             "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.norm_eps}, "residual_mult": self.residual_mult,
             "layers": [copy.deepcopy(l) for l in self.layers], "torch_dtype": self.torch_dtype}
        if self.loop is not None:
            d["loop"] = {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}
        return d

    def __hash__(self):
        return hash(json.dumps(self.to_dict(), sort_keys=True))


def _layer(heads, dim, rot_dim, vdim, kv_rank, experts, top, ff, shared_ff, base=10000.0, rot_dims=None, mlp=True):
    layer = {"type": "latent_attention",
             "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank,
                       "scale": 1.0 / math.sqrt(dim + rot_dim), "rot": {"base": base, "dims": rot_dims or rot_dim}},
             "mlp": None}
    if mlp:
        layer["mlp"] = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}
        if shared_ff:
            layer["mlp"]["shared"] = {"ff": shared_ff}
    return layer


def _preset(vocab, width, n_layers, max_positions, loop=None, **layer):
    return {"architecture": ARCHITECTURE, "vocab": vocab, "width": width, "max_positions": max_positions,
            "embedding": {"scale": 4.0}, "norm": {"eps": 1e-6}, "residual_mult": 0.5,
            "layers": [_layer(**layer) for _ in range(n_layers)], "loop": loop}


# Named presets: a tiny one for smoke runs, and three whose layers have the sizes of real models of this kind
# (random weights; `bench.py --model` takes them).
PRESETS: Dict[str, Dict[str, Any]] = {
    "gedalix-tiny": _preset(320, 96, 3, 256, loop={"start": 1, "stop": 3, "times": 2}, heads=3, dim=32, rot_dim=16, vdim=24,
                            kv_rank=40, experts=6, top=2, ff=48, shared_ff=80),
    "gedalix-small": _preset(32000, 1024, 8, 8192, heads=8, dim=64, rot_dim=32, vdim=64, kv_rank=256, experts=16, top=4,
                             ff=512, shared_ff=1024),
    "gedalix-16b-layers": _preset(102400, 2048, 8, 16384, heads=16, dim=128, rot_dim=64, vdim=128, kv_rank=512, experts=64,
                                  top=6, ff=1408, shared_ff=2816),
}


def gedalix_preset(name: str, **overrides) -> GedalixConfig:
    if name not in PRESETS:
        raise ConfigError(f"unknown preset {name!r}; known: {', '.join(sorted(PRESETS))}")
    raw = dict(PRESETS[name])
    raw.update(overrides)
    return GedalixConfig.from_dict(raw)
