"""Plain, slow restatement of the Matidra decoder: one function per mechanism, whole sequences at
once, float64 on the CPU.  It shares no code with the package: it reads a raw configuration (the
keys of config.json) and a dict of tensors under the checkpoint's names.

  layer            x = LN1(alpha x + mixer(x));  x = LN2(alpha x + ff(x))   (the sublayers read x itself)
  mixer attention  q = Wq x, k = Wk x, v = k (as projected); per-head rms norm of q and k; interleaved rotation of the
                   first `dims` elements with stretched frequencies; causal softmax; Wo
  mixer parallel   a_left * left(x) + a_right * right(x)
     left          q, k, v = Wq x, Wk x, Wv x, each through a short causal convolution; rms norm of q and k; q times a
                   temperature that grows with the logarithm of the position; causal softmax;
                   heads * sigmoid(Wg x); Wo
     right         q, k, v through short convolutions and silu; q, k unit vectors; per-channel decay;
                   S = diag(g) S;  u = beta (v - S^T k);  S += k u^T;  o = S^T q;  rms(o) * n * sigmoid(Wg2 Wg1 x);  Wo
  feed-forward     Wdown (gelu_tanh(Wgate x) * (Wup x))
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F = torch.float64


def layer_norm(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor, eps: float) -> torch.Tensor:
    mean = x.mean(-1, keepdim=True)
    var = ((x - mean) ** 2).mean(-1, keepdim=True)
    return (x - mean) / torch.sqrt(var + eps) * w + b


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def short_convolution(u: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """u [T, C], w [C, taps]: y_t = sum_j w[:, j] u_(t - taps + 1 + j), zeros before the start."""
    T, C = u.shape
    taps = w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=u.dtype), u], 0)
    y = torch.zeros_like(u)
    for j in range(taps):
        y += padded[j:j + T] * w[:, j]
    return y


def stretched_frequencies(dims: int, base: float, scaling: Optional[dict]):
    """(frequencies [dims/2], factor on cos and sin)."""
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    if not scaling:
        return torch.tensor(f, dtype=F), 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])
    where = lambda turns: dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(where(float(scaling["fast"]))), 0)
    hi = min(math.ceil(where(float(scaling["slow"]))), dims - 1)
    out = []
    for i, fi in enumerate(f):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(fi / factor * ramp + fi * (1.0 - ramp))
    return torch.tensor(out, dtype=F), 0.1 * math.log(factor) + 1.0


def rotate_pairs(x: torch.Tensor, positions: torch.Tensor, dims: int, freq: torch.Tensor, magnitude: float) -> torch.Tensor:
    """x [T, heads, n]: elements (2i, 2i+1), i < dims/2, are turned by position * freq_i."""
    a = positions.to(F)[:, None] * freq[None, :]
    cos, sin = (torch.cos(a) * magnitude)[:, None, :], (torch.sin(a) * magnitude)[:, None, :]
    out = x.clone()
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * cos - v * sin
    out[..., 1:dims:2] = v * cos + u * sin
    return out


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float) -> torch.Tensor:
    """q [T, H, dk], k [T, G, dk], v [T, G, dv]; query head h reads key/value head h // (H / G).  Returns [T, H, dv]."""
    T, H, _ = q.shape
    G = k.shape[1]
    rep = H // G
    out = torch.zeros(T, H, v.shape[-1], dtype=F)
    mask = torch.ones(T, T, dtype=torch.bool).tril()
    for h in range(H):
        s = (q[:, h] @ k[:, h // rep].T) * scale
        s = s.masked_fill(~mask, -math.inf)
        out[:, h] = torch.softmax(s, -1) @ v[:, h // rep]
    return out


def delta_rule(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, g: torch.Tensor, beta: torch.Tensor,
               state: Optional[torch.Tensor] = None):
    """q, k, g [T, H, dk], v [T, H, dv], beta [T, H]; returns (o [T, H, dv], final state [H, dk, dv])."""
    T, H, dk = q.shape
    dv = v.shape[-1]
    S = torch.zeros(H, dk, dv, dtype=F) if state is None else state.clone()
    o = torch.zeros(T, H, dv, dtype=F)
    for t in range(T):
        S = S * g[t][:, :, None]
        u = beta[t][:, None] * (v[t] - torch.einsum("hkv,hk->hv", S, k[t]))
        S = S + k[t][:, :, None] * u[:, None, :]
        o[t] = torch.einsum("hkv,hk->hv", S, q[t])
    return o, S


def softmax_mixer(h, positions, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float, conv: bool, values_are_keys: bool):
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q, k = h @ w[p + "q"].T, h @ w[p + "k"].T
    v = k if values_are_keys else h @ w[p + "v"].T
    if conv and p + "q.conv" in w:
        q, k, v = (short_convolution(x, w[p + n + ".conv"]) for x, n in ((q, "q"), (k, "k"), (v, "v")))
    v = v.view(T, G, dv)
    q = rms(q.view(T, H, dk), eps) * w[p + "q.norm"]
    k = rms(k.view(T, G, dk), eps) * w[p + "k.norm"]
    if m.get("rot"):
        freq, magnitude = stretched_frequencies(m["rot"]["dims"], m["rot"]["base"], m["rot"].get("scaling"))
        q = rotate_pairs(q, positions, m["rot"]["dims"], freq, magnitude)
        k = rotate_pairs(k, positions, m["rot"]["dims"], freq, magnitude)
    if m.get("q_temp"):
        t = 1.0 + m["q_temp"]["coef"] * torch.log(torch.floor((positions.to(F) + 1) / m["q_temp"]["every"]) + 1.0)
        q = q * t[:, None, None]
    o = causal_attention(q, k, v, float(m["scale"])).reshape(T, H * dv)
    if p + "g" in w:
        o = o * torch.sigmoid(h @ w[p + "g"].T)
    return o @ w[p + "o"].T


def delta_mixer(h, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float):
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    silu = lambda x: x * torch.sigmoid(x)
    conv = lambda x, n: short_convolution(x, w[p + n + ".conv"]) if p + n + ".conv" in w else x
    q = silu(conv(h @ w[p + "q"].T, "q")).view(T, G, dk)
    k = silu(conv(h @ w[p + "k"].T, "k")).view(T, G, dk)
    v = silu(conv(h @ w[p + "v"].T, "v")).view(T, H, dv)
    unit = lambda x: x / torch.sqrt((x * x).sum(-1, keepdim=True) + 1e-6)
    q, k = unit(q) * dk ** -0.5, unit(k)
    rep = H // G
    q, k = q.repeat_interleave(rep, 1), k.repeat_interleave(rep, 1)
    beta = torch.sigmoid(h @ w[p + "b"].T)
    pre = (h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "dt_bias"]
    g = torch.exp(-torch.exp(w[p + "A_log"])[None, :, None] * torch.nn.functional.softplus(pre).view(T, H, dk))
    o, _ = delta_rule(q, k, v, g, beta)
    o = rms(o, eps) * w[p + "norm"] * torch.sigmoid((h @ w[p + "g1"].T) @ w[p + "g2"].T).view(T, H, dv)
    return o.reshape(T, H * dv) @ w[p + "o"].T


def dense_ff(h, w, p):
    return (gelu_tanh(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def forward(raw: dict, weights: Dict[str, torch.Tensor], tokens: List[int], layers_out: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence from position 0; `layers_out` receives the stream after every layer."""
    w = {k: v.to(F) for k, v in weights.items()}
    eps, alpha = float(raw["norm"]["eps"]), float(raw["postln_alpha"])
    positions = torch.arange(len(tokens))
    x = w["embed"][torch.tensor(tokens)]
    for i, layer in enumerate(raw["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        if layer["type"] == "attention":
            mixed = softmax_mixer(x, positions, w, p + "mix.", m, eps, conv=False, values_are_keys=True)
        elif layer["type"] == "parallel":
            left = softmax_mixer(x, positions, w, p + "mix.left.", m["left"], eps, conv=True, values_are_keys=False)
            right = delta_mixer(x, w, p + "mix.right.", m["right"], eps)
            mixed = float(m["left_scale"]) * left + float(m["right_scale"]) * right
        else:
            raise ValueError(layer["type"])
        x = layer_norm(alpha * x + mixed, w[p + "norm1"], w[p + "norm1.b"], eps)
        if layer.get("mlp") is not None:
            x = layer_norm(alpha * x + dense_ff(x, w, p + "mlp."), w[p + "norm2"], w[p + "norm2.b"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    x = layer_norm(x, w["final.norm"], w["final.norm.b"], eps)
    return x @ w["head"].T
