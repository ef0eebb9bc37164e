"""Gated delta rule: a linear-attention mixer whose state is one matrix per head, decayed per key channel.

  q, k = Wq x, Wk x  (kv_heads x dim),  v = Wv x  (heads x vdim); head h reads q/k head h // (heads / kv_heads)
  each through a short causal convolution over time per channel (optional, `conv` taps) and silu
  q, k unit vectors per head: x / sqrt(sum x^2 + 1e-6); q also times dim^-1/2
  beta = sigmoid(Wb x)                                        one per head
  g = exp(-exp(A_log[h]) * softplus(Wa2 (Wa1 x) + dt_bias))   one per head and key channel
  per head, S [dim, vdim] from zero:  S <- diag(g) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
  o / rms(o) per head * weight * sigmoid(Wg2 (Wg1 x)),  then Wo

Every projection that reads x (q, k, v, b, a1, g1) is one fused product; the second steps of the two narrow
projections (Wa2, Wg2: `a_rank` and `g_rank` columns) are applied inside the kernels that need their results, in
fp32.  The state (S, fp32) and the convolution's last taps - 1 inputs live in the request's state slot.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..kernels import gemm_bf16, recurrent
from ..kernels.linear import linear
from .base import (CompositeNeed, FixedStateNeed, Mixer, PositionEncoding, Runtime, StepContext, WeightSpec, register_mixer)


@register_mixer("gated_delta_rule")
class GatedDeltaRule(Mixer):
    graph_safe = True

    def __init__(self, params: dict, rt: Runtime, position: Optional[PositionEncoding] = None):
        self.prefix = params.get("prefix", "")
        self.hidden = int(params["hidden_size"])
        self.nh, self.nkv = int(params["num_heads"]), int(params["num_kv_heads"])
        self.dk, self.dv = int(params["dim"]), int(params["vdim"])
        self.taps = int(params.get("conv", 1))
        self.a_rank, self.g_rank = int(params["a_rank"]), int(params["g_rank"])
        self.eps = float(params.get("eps", 1e-6))
        if self.nh % self.nkv:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        if not (0 < self.dk <= recurrent.MAX_WIDTH and 0 < self.dv <= recurrent.MAX_WIDTH):
            raise ValueError(f"gated_delta_rule: widths {self.dk}/{self.dv} must be in 1..{recurrent.MAX_WIDTH}")
        names = dict(q="q_proj.weight", k="k_proj.weight", v="v_proj.weight", o="o_proj.weight", q_conv="q_conv.weight",
                     k_conv="k_conv.weight", v_conv="v_conv.weight", beta="b_proj.weight", a1="a_proj.0.weight",
                     a2="a_proj.1.weight", a_log="A_log", dt_bias="dt_bias", g1="g_proj.0.weight", g2="g_proj.1.weight",
                     norm="o_norm.weight")
        names.update(params.get("names", {}))
        self.names = names
        self.rt = rt
        # columns of the fused input projection: q | k | v | beta | a1 | g1
        self.q_cols = self.k_cols = self.nkv * self.dk
        self.v_cols = self.nh * self.dv
        self.conv_cols = self.q_cols + self.k_cols + self.v_cols
        self.beta_col = self.conv_cols
        self.a_col = self.beta_col + self.nh
        self.g_col = self.a_col + self.a_rank
        self.in_rows = self.g_col + self.g_rank
        # the second steps of the two narrow projections run as products when their inner widths suit the product
        # kernels (multiples of 8), else inside the kernels that need their results
        self.a_product, self.g_product = self.a_rank % 8 == 0, self.g_rank % 8 == 0
        self.w_in = self.w_o = self.w_conv = self.w_a2 = self.w_g2 = self.a_log = self.dt_bias = self.norm_w = None

    # --- declarations -----------------------------------------------------------------
    def cache_need(self):
        items = [("state", FixedStateNeed((self.nh, self.dk, self.dv), torch.float32))]
        if self.taps > 1:
            items.append(("conv", FixedStateNeed((self.taps - 1, self.conv_cols), torch.float32)))
        return CompositeNeed(tuple(items))

    def _pieces(self):
        n = self.names
        return [(n["q"], 0), (n["k"], self.q_cols), (n["v"], self.q_cols + self.k_cols), (n["beta"], self.beta_col),
                (n["a1"], self.a_col), (n["g1"], self.g_col)]

    def weight_specs(self) -> Dict[str, WeightSpec]:
        n, W = self.names, self.hidden
        specs = {n["q"]: WeightSpec((self.q_cols, W)), n["k"]: WeightSpec((self.k_cols, W)), n["v"]: WeightSpec((self.v_cols, W)),
                 n["beta"]: WeightSpec((self.nh, W)), n["a1"]: WeightSpec((self.a_rank, W)), n["g1"]: WeightSpec((self.g_rank, W)),
                 n["a2"]: WeightSpec((self.nh * self.dk, self.a_rank), role="matrix" if self.a_product else "vector", init=("normal", 0.1)),
                 n["g2"]: WeightSpec((self.nh * self.dv, self.g_rank), role="matrix" if self.g_product else "vector", init=("normal", 0.1)),
                 n["a_log"]: WeightSpec((self.nh,), role="vector", init=("normal", 0.5)),
                 n["dt_bias"]: WeightSpec((self.nh * self.dk,), role="vector", init=("normal", 0.5)),
                 n["norm"]: WeightSpec((self.dv,), role="vector", init=("one_plus_normal", 0.1)),
                 n["o"]: WeightSpec((W, self.v_cols))}
        if self.taps > 1:
            for key, cols in (("q_conv", self.q_cols), ("k_conv", self.k_cols), ("v_conv", self.v_cols)):
                specs[n[key]] = WeightSpec((cols, self.taps), role="vector", init=("normal", 0.5))
        return specs

    def fused_tensors(self):
        fused = {"in_proj.weight": (WeightSpec((self.in_rows, self.hidden)), self._pieces())}
        if self.taps > 1:
            n = self.names
            fused["conv.weight"] = (WeightSpec((self.conv_cols, self.taps), role="vector"),
                                    [(n["q_conv"], 0), (n["k_conv"], self.q_cols), (n["v_conv"], self.q_cols + self.k_cols)])
        return fused

    def kernel_sources(self):
        own = recurrent.delta_sources() + recurrent.conv_sources()
        return own if self.rt.is_fp32 else own + gemm_bf16.sources(engine_only=True)

    def bind(self, tensors):
        n = self.names
        if "in_proj.weight" in tensors:
            self.w_in = tensors["in_proj.weight"]
        else:
            self.w_in = torch.cat([tensors[name] for name, _ in self._pieces()], 0).contiguous()
        if self.taps > 1:
            self.w_conv = tensors["conv.weight"] if "conv.weight" in tensors else torch.cat(
                [tensors[n[k]] for k in ("q_conv", "k_conv", "v_conv")], 0).contiguous()
        else:       # no convolution: one tap of weight 1 keeps one path (the activation still applies)
            self.w_conv = torch.ones((self.conv_cols, 1), dtype=torch.float32, device=self.rt.device)
        self.w_a2, self.w_g2 = tensors[n["a2"]], tensors[n["g2"]]
        self.a_log, self.dt_bias, self.norm_w = tensors[n["a_log"]], tensors[n["dt_bias"]], tensors[n["norm"]]
        self.w_o = tensors[n["o"]]

    def replay_key(self):
        if not self.rt.is_fp32 and not gemm_bf16._direct_library(self.rt.device):
            return None
        return ("gated_delta_rule", self.hidden, self.nh, self.nkv, self.dk, self.dv, self.taps, self.a_rank, self.g_rank, self.eps)

    def own_tensors(self):
        return [self.w_in, self.w_o, self.w_conv, self.w_a2, self.w_g2, self.a_log, self.dt_bias, self.norm_w]

    # --- compute ------------------------------------------------------------------------
    def forward(self, x: torch.Tensor, ctx: StepContext, cache) -> torch.Tensor:
        T, flag, f32 = x.shape[0], ctx.error_flag, torch.float32
        state = cache["state"]
        proj = linear(x, self.w_in, None, f32, partials_ok=True, error_flag=flag,
                      alloc=lambda shape, dtype: ctx.buffer("delta_rule.proj", shape, dtype))
        qkv = ctx.buffer("delta_rule.qkv", (T, self.conv_cols), f32)
        conv = cache.get("conv")
        recurrent.short_conv(proj, 0, self.w_conv, conv.storage if conv is not None else None, state.slots, ctx, qkv, silu=True,
                             update_state=state.writable)
        qn = ctx.buffer("delta_rule.qn", (T, self.q_cols), f32)
        kn = ctx.buffer("delta_rule.kn", (T, self.k_cols), f32)
        g = ctx.buffer("delta_rule.g", (T, self.nh * self.dk), f32)
        beta = ctx.buffer("delta_rule.beta", (T, self.nh), f32)
        a_pre = g_pre = None
        if self.a_product:
            narrow = ctx.buffer("delta_rule.a", (T, self.a_rank), self.rt.dtype)
            recurrent.take_columns(proj, self.a_col, narrow)
            a_pre = linear(narrow, self.w_a2, None, f32, partials_ok=True, error_flag=flag,
                           alloc=lambda shape, dtype: ctx.buffer("delta_rule.a_pre", shape, dtype))
        if self.g_product:
            narrow = ctx.buffer("delta_rule.g_in", (T, self.g_rank), self.rt.dtype)
            recurrent.take_columns(proj, self.g_col, narrow)
            g_pre = linear(narrow, self.w_g2, None, f32, partials_ok=True, error_flag=flag,
                           alloc=lambda shape, dtype: ctx.buffer("delta_rule.g_pre", shape, dtype))
        recurrent.delta_prepare(qkv, proj, self.beta_col, self.a_col, None if self.a_product else self.w_a2, self.dt_bias, self.a_log,
                                qn, kn, g, beta, self.nh, self.nkv, self.dk, pre=a_pre)
        o = ctx.buffer("delta_rule.o", (T, self.v_cols), f32)
        recurrent.delta_scan(qn, kn, g, beta, qkv[:, self.q_cols + self.k_cols:], o, state.storage, state.slots, ctx, self.nh,
                             self.nkv, self.dk, self.dv)
        gated = ctx.buffer("delta_rule.gated", (T, self.v_cols), self.rt.dtype)
        recurrent.delta_output(o, self.norm_w, proj, self.g_col, None if self.g_product else self.w_g2, gated, self.nh, self.dv, self.eps,
                               pre=g_pre)
        return linear(gated, self.w_o, None, f32, partials_ok=True, error_flag=flag,
                      alloc=lambda shape, dtype: ctx.buffer("delta_rule.out", shape, dtype))
