"""Small Gedalix configurations for the tests, and random weights for them under the checkpoint's names.

The cases differ from one another in every size and option: heads, the four per-head sizes (all unequal), the part
of the rotated elements that is turned, experts and choices (one choice; as many choices as experts), a shared
expert or none, a layer without a feed-forward, no loop, a loop of one pass, a loop over one layer run three times.
"""
from __future__ import annotations

import copy
import math
import os
from typing import Dict

import torch


def _layer(heads, dim, rot_dim, vdim, kv_rank, rot_dims, base, experts=0, top=0, ff=0, shared_ff=0, scale=None):
    layer = {"type": "latent_attention",
             "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank,
                       "scale": scale or 1.0 / math.sqrt(dim + rot_dim), "rot": {"base": base, "dims": rot_dims}},
             "mlp": None}
    if experts:
        layer["mlp"] = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}
        if shared_ff:
            layer["mlp"]["shared"] = {"ff": shared_ff}
    return layer


CASES = {
    # three heads, every per-head size different, half of the rotated elements turned, a loop over two layers
    "a": {"architecture": "Gedalix", "vocab": 200, "width": 48, "max_positions": 320, "embedding": {"scale": 3.0},
          "norm": {"eps": 1e-5}, "residual_mult": 0.6,
          "layers": [_layer(3, 16, 8, 24, 20, 4, 1000.0, experts=5, top=2, ff=40, shared_ff=56),
                     _layer(3, 16, 8, 24, 20, 4, 1000.0, experts=5, top=2, ff=40, shared_ff=56),
                     _layer(2, 12, 6, 10, 36, 6, 50000.0, experts=4, top=4, ff=24)],
          "loop": {"start": 0, "stop": 2, "times": 2}},
    # one head beside five, a layer without a feed-forward, one choice of seven, one layer run three times
    "b": {"architecture": "Gedalix", "vocab": 333, "width": 80, "max_positions": 400, "embedding": {"scale": 0.5},
          "norm": {"eps": 1e-3}, "residual_mult": 1.25,
          "layers": [_layer(1, 32, 32, 16, 64, 32, 10000.0, experts=7, top=1, ff=72, shared_ff=32),
                     _layer(5, 8, 16, 8, 24, 16, 250000.0),
                     _layer(5, 8, 16, 8, 24, 8, 100.0, experts=3, top=2, ff=96)],
          "loop": {"start": 1, "stop": 2, "times": 3}},
    # no loop at all; sizes that the tensor-core kernels like (multiples of 16 and 32)
    "c": {"architecture": "Gedalix", "vocab": 256, "width": 128, "max_positions": 1100, "embedding": {"scale": 1.0},
          "norm": {"eps": 1e-6}, "residual_mult": 1.5,
          "layers": [_layer(4, 32, 16, 48, 64, 16, 10000.0, experts=6, top=3, ff=64, shared_ff=96),
                     _layer(4, 32, 16, 48, 64, 16, 10000.0, experts=6, top=3, ff=64, shared_ff=96)],
          "loop": None},
    # a loop of one pass (only the pass's vector is added)
    "d": {"architecture": "Gedalix", "vocab": 150, "width": 64, "max_positions": 300, "embedding": {"scale": 2.0},
          "norm": {"eps": 1e-5}, "residual_mult": 1.0,
          "layers": [_layer(2, 16, 16, 32, 32, 16, 5000.0, experts=8, top=3, ff=32, shared_ff=48),
                     _layer(2, 16, 16, 32, 32, 16, 5000.0, experts=8, top=3, ff=32, shared_ff=48)],
          "loop": {"start": 1, "stop": 2, "times": 1}},
    # awkward sizes: nothing is a multiple of 8 but the width (every kernel that moves 16-byte pieces must step aside)
    "e": {"architecture": "Gedalix", "vocab": 101, "width": 72, "max_positions": 260, "embedding": {"scale": 1.5},
          "norm": {"eps": 1e-5}, "residual_mult": 0.7,
          "layers": [_layer(3, 10, 6, 14, 18, 6, 777.0, experts=9, top=3, ff=20, shared_ff=28),
                     _layer(3, 10, 6, 14, 18, 6, 777.0, experts=9, top=3, ff=20, shared_ff=28)],
          "loop": {"start": 0, "stop": 2, "times": 2}},
}


def raw_config(key: str) -> dict:
    return copy.deepcopy(CASES[key])


def random_weights(raw: dict, seed: int, sharp: float = 1.0, sink: float = 1.0) -> Dict[str, torch.Tensor]:
    """Random float32 tensors under the checkpoint's names.  `sharp` multiplies the query projections, which makes
    the attention weights peaky (single far keys then carry a position's output); `sink` multiplies the sinks."""
    g = torch.Generator().manual_seed(seed)
    W = raw["width"]
    normal = lambda *shape, std=1.0: torch.randn(*shape, generator=g) * std
    out = {"embed": normal(raw["vocab"], W), "pos": normal(raw["max_positions"], W, std=0.3), "final.norm": 1 + normal(W, std=0.1),
           "head": normal(raw["vocab"], W, std=W ** -0.5)}
    if raw.get("loop"):
        out["loop.step"] = normal(raw["loop"]["times"], W, std=0.5)
    for i, layer in enumerate(raw["layers"]):
        m, p = layer["mixer"], f"l{i}."
        H, dim, rot, vdim, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
        out[p + "norm1"] = 1 + normal(W, std=0.1)
        out[p + "ls1"] = 1 + normal(W, std=0.2)
        out[p + "mix.q"] = normal(H * (dim + rot), W, std=sharp * W ** -0.5)
        out[p + "mix.dkv"] = normal(rank + rot, W, std=W ** -0.5)
        out[p + "mix.dkv.norm"] = 1 + normal(rank, std=0.1)
        out[p + "mix.uk"] = normal(H * dim, rank, std=rank ** -0.5)
        out[p + "mix.uv"] = normal(H * vdim, rank, std=rank ** -0.5)
        out[p + "mix.sink"] = normal(H) * sink
        out[p + "mix.g"] = normal(H * vdim, W, std=W ** -0.5)
        out[p + "mix.o"] = normal(W, H * vdim, std=(H * vdim) ** -0.5)
        mlp = layer["mlp"]
        if not mlp:
            continue
        out[p + "norm2"] = 1 + normal(W, std=0.1)
        out[p + "ls2"] = 1 + normal(W, std=0.2)
        E, ff = mlp["router"]["experts"], mlp["expert"]["ff"]
        for e in range(E):
            out[p + f"mlp.e{e}.gate"] = normal(ff, W, std=W ** -0.5)
            out[p + f"mlp.e{e}.up"] = normal(ff, W, std=W ** -0.5)
            out[p + f"mlp.e{e}.down"] = normal(W, ff, std=ff ** -0.5)
        out[p + "mlp.router"] = normal(E, W, std=W ** -0.5)
        out[p + "mlp.router.b"] = normal(E, std=0.5)
        if mlp.get("shared"):
            sf = mlp["shared"]["ff"]
            out[p + "mlp.shared.gate"] = normal(sf, W, std=W ** -0.5)
            out[p + "mlp.shared.up"] = normal(sf, W, std=W ** -0.5)
            out[p + "mlp.shared.down"] = normal(W, sf, std=sf ** -0.5)
            out[p + "mlp.shared.sg"] = normal(1, W, std=W ** -0.5)
    return out


def write_folder(folder: str, raw: dict, weights: Dict[str, torch.Tensor], storage: torch.dtype = torch.float32) -> str:
    import json

    from microllm_rocm_b200.weights.safetensors import save_file
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(raw, f)
    save_file({n: t.to(storage).contiguous() for n, t in weights.items()}, os.path.join(folder, "model.safetensors"), metadata={"format": "pt"})
    return folder
