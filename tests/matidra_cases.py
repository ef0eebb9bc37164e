"""Small Matidra configurations for the tests, and random weights for them under the checkpoint's names.

The cases differ from one another in every size and option: the order of the layer kinds, heads and kv heads, key and
value widths (unequal, equal, not multiples of 8), convolution taps (none, two, five), the part of a head that is turned
and whether its frequencies are stretched, a query temperature or none, a layer without a feed-forward, the inner
widths of the two narrow projections, alpha and the branch weights (also 1, which a fault that drops them would hide
at other values only).
"""
from __future__ import annotations

import copy
import math
import os
from typing import Dict

import torch


def attention(heads, kv_heads, dim, ff, rot_dims=None, base=10000.0, scaling=None, scale=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale or dim ** -0.5}
    if rot_dims:
        m["rot"] = {"base": base, "dims": rot_dims, "scaling": scaling}
    return {"type": "attention", "mixer": m, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def parallel(left, right, ff, left_scale=0.7, right_scale=1.3):
    lh, lg, ld, lv, lconv, temp = left
    rh, rg, rd, rv, rconv = right
    l = {"heads": lh, "kv_heads": lg, "dim": ld, "vdim": lv, "scale": 1.0 / math.sqrt(ld), "conv": lconv}
    if temp:
        l["q_temp"] = {"coef": temp[0], "every": temp[1]}
    r = {"heads": rh, "kv_heads": rg, "dim": rd, "vdim": rv, "conv": rconv}         # a_rank / g_rank: from the tensors' shapes
    return {"type": "parallel", "mixer": {"left": l, "right": r, "left_scale": left_scale, "right_scale": right_scale},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


CASES = {
    # parallel first, attention in the middle, a layer without a feed-forward; unequal widths everywhere
    "a": {"architecture": "Matidra", "vocab": 200, "width": 64, "norm": {"eps": 1e-5}, "postln_alpha": 2.5,
          "layers": [parallel((3, 3, 16, 24, 3, (0.4, 7)), (4, 2, 16, 8, 2), 96),
                     attention(4, 2, 32, 80, rot_dims=12, base=5000.0, scaling={"factor": 4.0, "original": 64, "fast": 8.0, "slow": 2.0}),
                     parallel((3, 3, 16, 24, 3, (0.4, 7)), (4, 2, 16, 8, 2), 0)],
          "ranks": (5, 6)},
    # sizes that are not multiples of 8; one kv head for two query heads; no convolution on the left, five taps on the
    # right; equal key and value widths on the left; no temperature; alpha and both weights 1; plain frequencies
    "b": {"architecture": "Matidra", "vocab": 333, "width": 72, "norm": {"eps": 1e-3}, "postln_alpha": 1.0,
          "layers": [attention(3, 3, 10, 44, rot_dims=10, base=100.0),
                     parallel((2, 1, 24, 24, 1, None), (3, 1, 12, 20, 5), 100, left_scale=1.0, right_scale=1.0),
                     attention(1, 1, 18, 0, rot_dims=4, base=777.0, scaling={"factor": 1.5, "original": 16, "fast": 4.0, "slow": 1.0})],
          "ranks": (3, 9)},
    # sizes the tensor-core kernels like (heads of 64 with equal widths in the attention layer; 32 / 64 on the left)
    "c": {"architecture": "Matidra", "vocab": 256, "width": 128, "norm": {"eps": 2e-6}, "postln_alpha": 2.0,
          "layers": [attention(4, 2, 64, 256, rot_dims=32, base=5e5, scaling={"factor": 3.0, "original": 128, "fast": 16.0, "slow": 1.0}),
                     parallel((4, 2, 32, 64, 4, (0.25, 32)), (2, 2, 64, 64, 4), 256, left_scale=0.8, right_scale=0.9),
                     parallel((4, 2, 32, 64, 4, (0.25, 32)), (2, 2, 64, 64, 4), 256, left_scale=0.8, right_scale=0.9)],
          "ranks": (16, 16)},
    # one head each side, no rotation anywhere (the attention layer has none either, and no feed-forward), wide keys on the
    # right (several registers a lane)
    "d": {"architecture": "Matidra", "vocab": 150, "width": 48, "norm": {"eps": 1e-5}, "postln_alpha": 0.5,
          "layers": [parallel((1, 1, 40, 16, 2, (1.0, 3)), (1, 1, 136, 40, 3), 64, left_scale=2.0, right_scale=0.25),
                     parallel((1, 1, 40, 16, 2, (1.0, 3)), (1, 1, 136, 40, 3), 64, left_scale=2.0, right_scale=0.25),
                     attention(2, 2, 24, 0)],
          "ranks": (7, 4)},
    # wide heads: keys of 80 beside values of 160 on the left (stored at 256 on the tensor-core kernels), 72 / 72 in the
    # attention layer (stored at 128), all of a head turned; no convolution on the right; a temperature that steps at every position
    "e": {"architecture": "Matidra", "vocab": 120, "width": 96, "norm": {"eps": 1e-5}, "postln_alpha": 1.5,
          "layers": [parallel((2, 1, 80, 160, 3, (0.5, 1)), (2, 2, 24, 48, 1), 128, left_scale=0.9, right_scale=0.8),
                     attention(2, 1, 72, 128, rot_dims=72, base=2000.0)],
          "ranks": (8, 8)},
}


def raw_config(key: str) -> dict:
    raw = copy.deepcopy(CASES[key])
    raw.pop("ranks")
    return raw


def random_weights(raw: dict, seed: int, ranks=(5, 6), sharp: float = 1.0) -> Dict[str, torch.Tensor]:
    """Random float32 tensors under the checkpoint's names.  `sharp` multiplies the weights of the queries' norms,
    which makes the softmax peaky (single far keys then carry a position's output) whatever the norm does."""
    g = torch.Generator().manual_seed(seed)
    W = raw["width"]
    normal = lambda *shape, std=1.0: torch.randn(*shape, generator=g) * std
    out = {"embed": normal(raw["vocab"], W), "final.norm": 1 + normal(W, std=0.1), "final.norm.b": normal(W, std=0.1),
           "head": normal(raw["vocab"], W, std=W ** -0.5)}

    def softmax_side(p, m, conv, values, gate):
        H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        out[p + "q"] = normal(H * dk, W, std=W ** -0.5)
        out[p + "k"] = normal(G * dk, W, std=W ** -0.5)
        out[p + "q.norm"] = (1 + normal(dk, std=0.1)) * sharp
        out[p + "k.norm"] = 1 + normal(dk, std=0.1)
        out[p + "o"] = normal(W, H * dv, std=(H * dv) ** -0.5)
        if values:
            out[p + "v"] = normal(G * dv, W, std=W ** -0.5)
        if gate:
            out[p + "g"] = normal(H * dv, W, std=W ** -0.5)
        if conv > 1:
            for n, c in (("q", H * dk), ("k", G * dk), ("v", G * dv)):
                out[p + n + ".conv"] = normal(c, conv, std=0.6)

    for i, layer in enumerate(raw["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        out[p + "norm1"], out[p + "norm1.b"] = 1 + normal(W, std=0.1), normal(W, std=0.1)
        if layer["type"] == "attention":
            softmax_side(p + "mix.", m, 1, values=False, gate=False)
        else:
            softmax_side(p + "mix.left.", m["left"], m["left"].get("conv", 1), values=True, gate=True)
            r, q = m["right"], p + "mix.right."
            H, G, dk, dv, conv = r["heads"], r["kv_heads"], r["dim"], r["vdim"], r.get("conv", 1)
            ra, rg = r.get("a_rank", ranks[0]), r.get("g_rank", ranks[1])
            out[q + "q"], out[q + "k"] = normal(G * dk, W, std=W ** -0.5), normal(G * dk, W, std=W ** -0.5)
            out[q + "v"] = normal(H * dv, W, std=W ** -0.5)
            if conv > 1:
                for n, c in (("q", G * dk), ("k", G * dk), ("v", H * dv)):
                    out[q + n + ".conv"] = normal(c, conv, std=0.6)
            out[q + "b"] = normal(H, W, std=W ** -0.5)
            out[q + "a1"], out[q + "a2"] = normal(ra, W, std=W ** -0.5), normal(H * dk, ra, std=ra ** -0.5)
            out[q + "A_log"], out[q + "dt_bias"] = normal(H, std=0.7) - 1.0, normal(H * dk, std=0.7)
            out[q + "g1"], out[q + "g2"] = normal(rg, W, std=W ** -0.5), normal(H * dv, rg, std=rg ** -0.5)
            out[q + "norm"] = 1 + normal(dv, std=0.1)
            out[q + "o"] = normal(W, H * dv, std=(H * dv) ** -0.5)
        if layer.get("mlp"):
            ff = layer["mlp"]["ff"]
            out[p + "norm2"], out[p + "norm2.b"] = 1 + normal(W, std=0.1), normal(W, std=0.1)
            out[p + "mlp.gate"], out[p + "mlp.up"] = normal(ff, W, std=W ** -0.5), normal(ff, W, std=W ** -0.5)
            out[p + "mlp.down"] = normal(W, ff, std=ff ** -0.5)
    return out


def case(key: str, seed: int = 0, sharp: float = 1.0):
    """(raw config as config.json holds it, weights)."""
    raw = raw_config(key)
    return raw, random_weights(raw, seed or (len(key) + ord(key[0])), CASES[key]["ranks"], sharp)


def write_folder(folder: str, raw: dict, weights: Dict[str, torch.Tensor], storage: torch.dtype = torch.float32) -> str:
    import json

    from microllm_rocm_b200.weights.safetensors import save_file
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(raw, f)
    save_file({n: t.to(storage).contiguous() for n, t in weights.items()}, os.path.join(folder, "model.safetensors"), metadata={"format": "pt"})
    return folder
