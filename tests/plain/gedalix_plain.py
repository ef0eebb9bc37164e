"""Plain, slow restatement of the Gedalix decoder: one function per mechanism, whole sequences
at once, float64 on the CPU.  It shares no code with the package: it reads a raw configuration
(the keys of config.json) and a dict of tensors under the checkpoint's names.

  embedding      x_p = scale * E[token_p] + P[p]
  layer          x += m * ls1 * mixer(rms(x) * n1);  x += m * ls2 * ff(rms(x) * n2)
  loop           layers start..stop-1 run `times` times with the same weights; pass t first
                 adds the embedding output (t > 0) and the row t of the step table
  latent mixer   q = Wq h; [c | kr] = Wdkv h; c = rms(c) * nc; per head k = Wuk c, v = Wuv c;
                 rotated parts of q and kr turned by the position; causal softmax whose
                 denominator also holds exp(sink_h); heads * sigmoid(Wg h); Wo
  feed-forward   routed experts (largest `top` logits of Wr h + b, softmax over the chosen)
                 plus a shared expert times sigmoid(Wsg h)
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F = torch.float64


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rotate_half(x: torch.Tensor, positions: torch.Tensor, base: float, dims: int) -> torch.Tensor:
    """x [..., T, n]: the first `dims` of the last axis are turned, i paired with i + dims/2."""
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F)
    a = positions.to(F)[:, None] * f[None, :]
    cos, sin = torch.cos(a), torch.sin(a)
    u, v = x[..., :half], x[..., half:dims]
    out = x.clone()
    out[..., :half] = u * cos - v * sin
    out[..., half:dims] = v * cos + u * sin
    return out


def swiglu_expert(h: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor) -> torch.Tensor:
    g = h @ gate.T
    return ((g * torch.sigmoid(g)) * (h @ up.T)) @ down.T


def sink_softmax_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                           sink: Optional[torch.Tensor], window: Optional[int] = None) -> torch.Tensor:
    """q, k [H, T, dk], v [H, T, dv] of one sequence; position i sees j <= i (with a window: the last `window` of
    them, itself included); returns [T, H, dv]."""
    H, T, _ = q.shape
    s = torch.einsum("hid,hjd->hij", q, k) * scale
    mask = torch.ones(T, T, dtype=torch.bool).tril()
    if window is not None:
        mask &= ~torch.ones(T, T, dtype=torch.bool).tril(-int(window))
    s = s.masked_fill(~mask, -math.inf)
    if sink is not None:
        s = torch.cat([s, sink.to(F)[:, None, None].expand(H, T, 1)], dim=-1)
    p = torch.softmax(s, dim=-1)
    if sink is not None:
        p = p[..., :T]
    return torch.einsum("hij,hjd->ihd", p, v)


def latent_attention(h: torch.Tensor, positions: torch.Tensor, w: Dict[str, torch.Tensor], prefix: str, mixer: dict,
                     eps: float) -> torch.Tensor:
    H, dim, rot_dim = mixer["heads"], mixer["dim"], mixer["rot_dim"]
    vdim, rank = mixer["vdim"], mixer["kv_rank"]
    rot = mixer["rot"]
    T = h.shape[0]
    g = lambda n: w[prefix + n].to(F)
    q = (h @ g("q").T).view(T, H, dim + rot_dim)
    dkv = h @ g("dkv").T
    c = rms(dkv[:, :rank], eps) * g("dkv.norm")
    k_rot = rotate_half(dkv[:, rank:], positions, rot["base"], rot["dims"])              # [T, rot_dim], shared
    q_rot = rotate_half(q[..., dim:].transpose(0, 1), positions, rot["base"], rot["dims"])   # [H, T, rot_dim]
    k_plain = (c @ g("uk").T).view(T, H, dim).transpose(0, 1)
    value = (c @ g("uv").T).view(T, H, vdim).transpose(0, 1)
    qq = torch.cat([q[..., :dim].transpose(0, 1), q_rot], dim=-1)
    kk = torch.cat([k_plain, k_rot[None].expand(H, T, rot_dim)], dim=-1)
    o = sink_softmax_attention(qq, kk, value, mixer["scale"], w.get(prefix + "sink"), mixer.get("window")).reshape(T, H * vdim)
    if prefix + "g" in w:
        o = o * torch.sigmoid(h @ g("g").T)
    return o @ g("o").T


def routed_feed_forward(h: torch.Tensor, w: Dict[str, torch.Tensor], prefix: str, mlp: dict) -> torch.Tensor:
    g = lambda n: w[prefix + n].to(F)
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    z = h @ g("router").T + g("router.b")
    chosen = torch.topk(z, top, dim=-1)
    weights = torch.softmax(chosen.values, dim=-1)
    out = torch.zeros(h.shape[0], g("e0.down").shape[0], dtype=F)
    for t in range(h.shape[0]):
        for j in range(top):
            e = int(chosen.indices[t, j])
            out[t] += weights[t, j] * swiglu_expert(h[t:t + 1], g(f"e{e}.gate"), g(f"e{e}.up"), g(f"e{e}.down"))[0]
    if mlp.get("shared"):
        shared = swiglu_expert(h, g("shared.gate"), g("shared.up"), g("shared.down"))
        out = out + shared * torch.sigmoid(h @ g("shared.sg").T)
    return out


def layer_order(cfg: dict) -> List[tuple]:
    """(layer, pass number if this run opens a pass else None) in execution order."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    start, stop, times = loop["start"], loop["stop"], loop["times"]
    order = [(i, None) for i in range(start)]
    for t in range(times):
        order += [(i, t if i == start else None) for i in range(start, stop)]
    return order + [(i, None) for i in range(stop, n)]


def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: List[int], collect: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] (float64) of one whole sequence.  `collect` receives the residual after every run."""
    eps, m = cfg["norm"]["eps"], cfg["residual_mult"]
    T = len(tokens)
    positions = torch.arange(T)
    x = w["embed"].to(F)[torch.tensor(tokens)] * cfg["embedding"]["scale"] + w["pos"].to(F)[:T]
    x0 = x.clone()
    for i, opens in layer_order(cfg):
        layer = cfg["layers"][i]
        p = f"l{i}."
        if opens is not None:
            if opens > 0:
                x = x + x0
            x = x + w["loop.step"].to(F)[opens]
        if layer["type"] != "latent_attention":
            raise ValueError(layer["type"])
        mixed = latent_attention(rms(x, eps) * w[p + "norm1"].to(F), positions, w, p + "mix.", layer["mixer"], eps)
        x = x + m * (mixed * w[p + "ls1"].to(F))
        if layer.get("mlp"):
            ff = routed_feed_forward(rms(x, eps) * w[p + "norm2"].to(F), w, p + "mlp.", layer["mlp"])
            x = x + m * (ff * w[p + "ls2"].to(F))
        if collect is not None:
            collect.append(x.clone())
    x = rms(x, eps) * w["final.norm"].to(F)
    return x @ w["head"].to(F).T
