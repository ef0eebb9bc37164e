"""Latent attention: keys and values of all heads are expanded from one small vector per token, and only that
vector (with a rotated key part that all heads share) is cached.

  q = Wq x                           per head: `dim` plain elements, then `rot_dim` rotated ones
  [l | kr] = Wdkv x                  c = rms(l) * n  (fp32; `rank` elements),  kr: `rot_dim` elements, rotated
  head h:  k_h = Wuk_h c,  v_h = Wuv_h c
           score(i, j) = (q_h,plain(i) . k_h(j) + q_h,rot(i) . kr(j)) * scale,   j <= i
           softmax whose denominator also holds exp(sink_h) (optional, a learned number per head)
  out = Wo (concat_h o_h  *  sigmoid(Wg x))        the gate is optional

The cache holds c and kr only (`PagedRowsNeed(rank + rot_dim)`).  k_h and v_h are never expanded: with
a_h = Wuk_h^T q_h,plain the score is (a_h . c + q_h,rot . kr) * scale, and o_h = Wuv_h (sum_j p_j c_j); both extra
products run per head over all tokens (`kernels/grouped.py`), the second with the gate as its epilogue.  Wq, Wdkv
and Wg are one fused product.  The rotation comes from the position encoding this mixer is given: its first
`rotary_dim` rotated elements are turned, pairs (i, i + rotary_dim / 2).
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..kernels import gemm_bf16, grouped, latent
from ..kernels.linear import linear
from .base import Mixer, PagedKVView, PagedRowsNeed, PositionEncoding, Runtime, StepContext, WeightSpec, register_mixer


@register_mixer("latent_attention")
class LatentAttention(Mixer):
    graph_safe = True

    def __init__(self, params: dict, rt: Runtime, position: Optional[PositionEncoding] = None):
        self.prefix = params.get("prefix", "")
        self.hidden = int(params["hidden_size"])
        self.heads = int(params["num_heads"])
        self.dim = int(params["dim"])
        self.rot_dim = int(params["rot_dim"])
        self.vdim = int(params["vdim"])
        self.rank = int(params["kv_rank"])
        self.scale = float(params["scale"])
        self.eps = float(params["eps"])
        self.window = params.get("window")
        self.has_sink = bool(params.get("sink", False))
        self.has_gate = bool(params.get("gate", False))
        # local names in the checkpoint
        names = dict(q="q_proj.weight", dkv="kv_a_proj.weight", dkv_norm="kv_a_norm.weight", uk="k_b_proj.weight",
                     uv="v_b_proj.weight", o="o_proj.weight", sink="sink", gate="gate_proj.weight")
        names.update(params.get("names", {}))
        self.names = names
        latent.check_sizes(self.rank, self.rot_dim)
        self.rt = rt
        table = position.rotary_table(self.rot_dim) if position is not None and self.rot_dim else None
        if table is not None and table.magnitude != 1.0:
            raise ValueError("latent attention takes plain cosines and sines")
        if table is not None and table.interleaved:
            raise ValueError("latent attention pairs element i with i + rotary_dim / 2")
        self.inv_freq = table.inv_freq if table is not None else torch.zeros(0, dtype=torch.float32, device=rt.device)
        self.rot_dims = table.rotary_dim if table is not None else 0
        self.q_width = self.heads * (self.dim + self.rot_dim)
        self.kv_width = self.rank + self.rot_dim
        self.gate_width = self.heads * self.vdim if self.has_gate else 0
        self.w_in = self.w_uk_t = self.w_uv = self.w_o = self.kv_norm = self.sink = None

    # --- declarations -----------------------------------------------------------------
    def cache_need(self):
        return PagedRowsNeed(self.kv_width, self.window)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        n = self.names
        specs = {n["q"]: WeightSpec((self.q_width, self.hidden)), n["dkv"]: WeightSpec((self.kv_width, self.hidden)),
                 n["dkv_norm"]: WeightSpec((self.rank,), role="vector", init=("one_plus_normal", 0.1)),
                 n["uk"]: WeightSpec((self.heads * self.dim, self.rank)), n["uv"]: WeightSpec((self.heads * self.vdim, self.rank)),
                 n["o"]: WeightSpec((self.hidden, self.heads * self.vdim))}
        if self.has_sink:
            specs[n["sink"]] = WeightSpec((self.heads,), role="vector", init=("normal", 1.0))
        if self.has_gate:
            specs[n["gate"]] = WeightSpec((self.gate_width, self.hidden))
        return specs

    def _in_pieces(self):
        pieces = [(self.names["q"], 0), (self.names["dkv"], self.q_width)]
        if self.has_gate:
            pieces.append((self.names["gate"], self.q_width + self.kv_width))
        return pieces

    def fused_tensors(self):
        rows = self.q_width + self.kv_width + self.gate_width
        return {"in_proj.weight": (WeightSpec((rows, self.hidden)), self._in_pieces())}

    def kernel_sources(self):
        own = latent.sources() + grouped.sources()
        return own if self.rt.is_fp32 else own + latent.mma_sources(self.rank, self.rot_dim) + gemm_bf16.sources(engine_only=True)

    def bind(self, tensors):
        n = self.names
        if "in_proj.weight" in tensors:
            self.w_in = tensors["in_proj.weight"]
        else:
            self.w_in = torch.cat([tensors[name] for name, _ in self._in_pieces()], 0).contiguous()
        # a_h = Wuk_h^T q_h: as a product with a weight stored [out, in] that is the transposed block, [heads, rank, dim]
        self.w_uk_t = tensors[n["uk"]].view(self.heads, self.dim, self.rank).transpose(1, 2).contiguous()
        self.w_uv = tensors[n["uv"]].view(self.heads, self.vdim, self.rank)
        self.w_o = tensors[n["o"]]
        self.kv_norm = tensors[n["dkv_norm"]]
        self.sink = tensors[n["sink"]] if self.has_sink else None

    def replay_key(self):
        if not self.rt.is_fp32 and not gemm_bf16._direct_library(self.rt.device):
            return None                  # the library product would go through the tensor framework
        return ("latent_attention", self.hidden, self.heads, self.dim, self.rot_dim, self.vdim, self.rank, self.scale,
                self.eps, self.window, self.has_sink, self.has_gate, self.rot_dims)

    def own_tensors(self):
        return [self.w_in, self.w_uk_t, self.w_uv, self.w_o, self.kv_norm, self.sink, self.inv_freq]

    # --- launch plans frozen into a captured decode step ----------------------------------
    def plan_stale(self, ctx: StepContext, max_seq_len: int) -> bool:
        return latent.plan_stale(ctx, max_seq_len)

    def forget_plans(self, ctx: StepContext) -> None:
        latent.forget_plans(ctx)

    def plan_group(self):
        return ("latent_attention", self.rt.device)

    # --- compute ------------------------------------------------------------------------
    def forward(self, x: torch.Tensor, ctx: StepContext, cache: PagedKVView) -> torch.Tensor:
        T, H, dt = x.shape[0], self.heads, self.rt.dtype
        flag = ctx.error_flag
        proj = linear(x, self.w_in, None, torch.float32, partials_ok=True, error_flag=flag,
                      alloc=lambda shape, dtype: ctx.buffer("latent.proj", shape, dtype))
        q_plain = ctx.buffer("latent.q_plain", (T, H * self.dim), dt)
        q_full = ctx.buffer("latent.q_full", (T, H * self.kv_width), dt)
        gate = ctx.buffer("latent.gate", (T, self.gate_width), torch.float32) if self.has_gate else None
        latent.prepare(proj, q_col=0, kv_col=self.q_width, gate_col=self.q_width + self.kv_width, norm_weight=self.kv_norm,
                       eps=self.eps, positions=ctx.positions, token_seq=ctx.token_seq, block_table=cache.block_table,
                       inv_freq=self.inv_freq, rot_dims=self.rot_dims, q_plain=q_plain, q_full=q_full,
                       pages=cache.pages if cache.writable else None, gate_out=gate, heads=H, dim=self.dim,
                       rot_dim=self.rot_dim, rank=self.rank, error_flag=flag)
        row_tile = grouped.row_tile_for(T, H, False, grouped.mma_supported(q_plain, self.w_uk_t, self.dim))
        # a_h = Wuk_h^T q_h,plain into the first `rank` columns of each head's query row
        grouped.grouped_linear(q_plain, self.w_uk_t, q_full, rows=T, a_group_cols=self.dim, c_group_cols=self.kv_width,
                               row_tile=row_tile)
        o_latent = ctx.buffer("latent.o_latent", (T, H * self.rank), dt)
        latent.attention(q_full, cache.pages, o_latent, self.sink, ctx, cache.block_table, H, self.rank, self.rot_dim,
                         self.scale, self.window)
        # o_h = Wuv_h (sum_j p_j c_j), times the gate
        o = ctx.buffer("latent.o", (T, H * self.vdim), dt)
        grouped.grouped_linear(o_latent, self.w_uv, o, rows=T, a_group_cols=self.rank, c_group_cols=self.vdim, factor=gate,
                               row_tile=row_tile)
        return linear(o, self.w_o, None, torch.float32, partials_ok=True, error_flag=flag,
                      alloc=lambda shape, dtype: ctx.buffer("latent.out", shape, dtype))
