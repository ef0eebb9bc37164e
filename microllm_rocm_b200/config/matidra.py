"""Typed configuration of the Matidra decoder, read from its own config.json keys.

  architecture          "Matidra"
  vocab, width          vocabulary and residual width
  norm.eps              eps of every norm of the model (layer norms and the per-head rms norms)
  postln_alpha          factor on the residual stream inside each post-norm sum
  layers[i]             type ("attention" | "parallel"), mixer (its sizes), mlp ({kind: "dense", ff} or null for none)
  max_positions         optional: the longest sequence the engine admits (no table depends on it)

Mixer "attention": heads, kv_heads, dim, vdim (= dim: the values are the projected keys), scale,
rot {base, dims, scaling {factor, original, fast, slow} | null}.
Mixer "parallel": left {heads, kv_heads, dim, vdim, scale, conv, q_temp {coef, every}},
right {heads, kv_heads, dim, vdim, conv, a_rank, g_rank}, left_scale, right_scale.  a_rank and g_rank (inner widths
of the decay's and the output gate's two-step projections) may be absent from config.json: they are then read from
the shapes of `<layer>.mix.right.a1` and `.g1` in the weight file (`sizes_from_tensors`).
Every size and constant comes from here or from a tensor's shape; nothing in the engine carries one.
"""
from __future__ import annotations

import copy
import json
import math
import os
from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Sequence, Tuple

from .qwen2 import ConfigError

ARCHITECTURE = "Matidra"
MIXER_KINDS = ("attention", "parallel")
DEFAULT_MAX_POSITIONS = 1 << 20


def _positive_int(value, what: str) -> int:
    if not isinstance(value, int) or isinstance(value, bool) or value <= 0:
        raise ConfigError(f"{what} must be a positive integer, got {value!r}")
    return value


def _number(value, what: str, positive: bool = False) -> float:
    if isinstance(value, bool) or not isinstance(value, (int, float)) or not math.isfinite(value) or (positive and value <= 0):
        raise ConfigError(f"{what} must be a finite{' positive' if positive else ''} number, got {value!r}")
    return float(value)


def _heads(m: Mapping[str, Any], where: str) -> None:
    if not isinstance(m, Mapping):
        raise ConfigError(f"{where} is missing")
    for key in ("heads", "kv_heads", "dim", "vdim"):
        _positive_int(m.get(key), f"{where}.{key}")
    if m["heads"] % m["kv_heads"]:
        raise ConfigError(f"{where}.heads must be a multiple of kv_heads")


@dataclass(frozen=True)
class MatidraConfig:
    vocab: int
    width: int
    norm_eps: float
    postln_alpha: float
    layers: Tuple[Dict[str, Any], ...]
    max_positions: int = DEFAULT_MAX_POSITIONS
    torch_dtype: str = "bfloat16"

    # ---- what the engine asks of any configuration ------------------------------------
    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def max_position_embeddings(self) -> int:
        return self.max_positions

    eos_token_id = None

    # ---- validation ----------------------------------------------------------------
    def validate(self) -> None:
        _positive_int(self.vocab, "vocab"); _positive_int(self.width, "width"); _positive_int(self.max_positions, "max_positions")
        _number(self.norm_eps, "norm.eps", positive=True); _number(self.postln_alpha, "postln_alpha")
        if not self.layers:
            raise ConfigError("layers must list at least one layer")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            kind = layer.get("type")
            if kind not in MIXER_KINDS:
                raise ConfigError(f"{where}.type {kind!r} is not one of {', '.join(MIXER_KINDS)}")
            m = layer.get("mixer")
            if not isinstance(m, Mapping):
                raise ConfigError(f"{where}.mixer is missing")
            if kind == "attention":
                _heads(m, f"{where}.mixer")
                _number(m.get("scale"), f"{where}.mixer.scale", positive=True)
                if m["vdim"] != m["dim"]:
                    raise ConfigError(f"{where}.mixer: the values are the projected keys, so vdim must equal dim")
                rot = m.get("rot")
                if rot is not None:
                    _number(rot.get("base"), f"{where}.mixer.rot.base", positive=True)
                    dims = rot.get("dims")
                    if not isinstance(dims, int) or isinstance(dims, bool) or dims <= 0 or dims % 2 or dims > m["dim"]:
                        raise ConfigError(f"{where}.mixer.rot.dims must be even, positive and at most dim")
                    sc = rot.get("scaling")
                    if sc is not None:
                        for key in ("factor", "original", "fast", "slow"):
                            _number(sc.get(key), f"{where}.mixer.rot.scaling.{key}", positive=True)
            else:
                left, right = m.get("left"), m.get("right")
                _heads(left, f"{where}.mixer.left"); _heads(right, f"{where}.mixer.right")
                _number(left.get("scale"), f"{where}.mixer.left.scale", positive=True)
                for side, s in (("left", left), ("right", right)):
                    conv = s.get("conv", 1)
                    if not isinstance(conv, int) or isinstance(conv, bool) or conv < 1:
                        raise ConfigError(f"{where}.mixer.{side}.conv must be a positive number of taps")
                qt = left.get("q_temp")
                if qt is not None:
                    _number(qt.get("coef"), f"{where}.mixer.left.q_temp.coef")
                    _positive_int(qt.get("every"), f"{where}.mixer.left.q_temp.every")
                for key in ("a_rank", "g_rank"):
                    _positive_int(right.get(key), f"{where}.mixer.right.{key} (or the shape of the matching tensor)")
                _number(m.get("left_scale"), f"{where}.mixer.left_scale"); _number(m.get("right_scale"), f"{where}.mixer.right_scale")
            mlp = layer.get("mlp")
            if mlp is not None:
                if mlp.get("kind") != "dense":
                    raise ConfigError(f"{where}.mlp.kind {mlp.get('kind')!r} is not 'dense'")
                _positive_int(mlp.get("ff"), f"{where}.mlp.ff")

    # ---- (de)serialisation -----------------------------------------------------------
    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "MatidraConfig":
        missing = [k for k in ("vocab", "width", "layers", "norm", "postln_alpha") if k not in raw]
        if missing:
            raise ConfigError("config.json is missing " + ", ".join(missing))
        if not isinstance(raw["layers"], list):
            raise ConfigError("layers must be a list")
        cfg = cls(vocab=raw["vocab"], width=raw["width"], norm_eps=(raw["norm"] or {}).get("eps"),
                  postln_alpha=raw["postln_alpha"], layers=tuple(copy.deepcopy(l) for l in raw["layers"]),
                  max_positions=raw.get("max_positions", DEFAULT_MAX_POSITIONS), torch_dtype=raw.get("torch_dtype", "bfloat16"))
        cfg.validate()
        return cfg

    @classmethod
    def from_json(cls, path: str) -> "MatidraConfig":
        if os.path.isdir(path):
            path = os.path.join(path, "config.json")
        with open(path, "r", encoding="utf-8") as f:
            return cls.from_dict(json.load(f))

    def to_dict(self) -> Dict[str, Any]:
        return {"architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
                "postln_alpha": self.postln_alpha, "layers": [copy.deepcopy(l) for l in self.layers],
                "max_positions": self.max_positions, "torch_dtype": self.torch_dtype}

    def __hash__(self):
        return hash(json.dumps(self.to_dict(), sort_keys=True))


def sizes_from_tensors(raw: Dict[str, Any], shapes: Mapping[str, Sequence[int]]) -> Dict[str, Any]:
    """config.json completed with the sizes that only the weight file knows (tensor name -> shape)."""
    raw = copy.deepcopy(raw)
    for i, layer in enumerate(raw.get("layers") or []):
        if not isinstance(layer, dict) or layer.get("type") != "parallel":
            continue
        right = (layer.get("mixer") or {}).get("right")
        if not isinstance(right, dict):
            continue
        for key, tensor in (("a_rank", f"l{i}.mix.right.a1"), ("g_rank", f"l{i}.mix.right.g1")):
            if key not in right and tensor in shapes and len(shapes[tensor]) == 2:
                right[key] = int(shapes[tensor][0])
    return raw


# ---- presets: a tiny one for smoke runs, and two whose layers have the sizes of real models' layers ---------------
def attention_layer(heads, kv_heads, dim, ff, rot_dims=None, base=1000000.0, scaling=None, scale=None):
    return {"type": "attention",
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale or dim ** -0.5,
                      "rot": {"base": base, "dims": rot_dims or dim, "scaling": scaling}},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


def parallel_layer(heads, kv_heads, dim, vdim, r_heads, r_kv_heads, r_dim, r_vdim, ff, conv=4, rank=None, left_scale=0.5,
                   right_scale=1.0, q_temp=(0.2, 128), scale=None):
    return {"type": "parallel",
            "mixer": {"left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale or dim ** -0.5,
                               "conv": conv, "q_temp": {"coef": q_temp[0], "every": q_temp[1]} if q_temp else None},
                      "right": {"heads": r_heads, "kv_heads": r_kv_heads, "dim": r_dim, "vdim": r_vdim, "conv": conv,
                                "a_rank": rank or r_dim, "g_rank": rank or r_dim},
                      "left_scale": left_scale, "right_scale": right_scale},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


def _preset(vocab, width, layers):
    return {"architecture": ARCHITECTURE, "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "postln_alpha": 2.0,
            "layers": layers}


_YARN = {"factor": 4.0, "original": 4096, "fast": 32.0, "slow": 1.0}
PRESETS: Dict[str, Dict[str, Any]] = {
    "matidra-tiny": _preset(320, 96, [attention_layer(4, 2, 32, 160, rot_dims=16, scaling=_YARN),
                                      parallel_layer(3, 3, 16, 32, 2, 1, 16, 32, 160, rank=8),
                                      parallel_layer(3, 3, 16, 32, 2, 1, 16, 32, 0, rank=8)]),
    "matidra-small": _preset(32000, 1024, [attention_layer(16, 4, 64, 2816, rot_dims=32, scaling=_YARN)]
                             + [parallel_layer(8, 8, 64, 128, 8, 8, 64, 128, 2816, rank=64) for _ in range(3)]),
    "matidra-3b-layers": _preset(102400, 2048, [attention_layer(16, 4, 128, 5632, rot_dims=64, scaling=_YARN)]
                                 + [parallel_layer(16, 16, 64, 128, 16, 16, 128, 128, 5632, rank=128) for _ in range(3)]),
}
