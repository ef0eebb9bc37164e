"""Latent attention's own kernels (`csrc/latent.cu`): what follows the fused input projection (norm of the latent,
rotation, cache store, query split, gate activation) and the attention over the compressed cache."""
from __future__ import annotations

from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Optional

import torch

from . import build, ops
from .build import KernelError

SOURCE = "latent.cu"
ops.register_signatures(SOURCE, {
    "mlb_latent_prepare": [c_void_p, c_longlong, c_int, c_longlong, c_longlong, c_longlong, c_longlong, c_void_p, c_float,
                           c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int,
                           c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
    "mlb_latent_attention_plain": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                   c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p],
})

MAX_RANK = 512
MAX_KEY_WIDTH = 640


def sources():
    return [(SOURCE, {})]


def check_sizes(rank: int, rot_dim: int) -> None:
    if rank <= 0 or rank > MAX_RANK or rank + rot_dim > MAX_KEY_WIDTH:
        raise KernelError(f"latent attention: a latent of {rank} and a rotated part of {rot_dim} exceed {MAX_RANK} / {MAX_KEY_WIDTH}")


def prepare(proj: torch.Tensor, *, q_col: int, kv_col: int, gate_col: int, norm_weight: torch.Tensor, eps: float,
            positions: torch.Tensor, token_seq: torch.Tensor, block_table: Optional[torch.Tensor], inv_freq: torch.Tensor,
            rot_dims: int, q_plain: torch.Tensor, q_full: torch.Tensor, pages: Optional[torch.Tensor],
            gate_out: Optional[torch.Tensor], heads: int, dim: int, rot_dim: int, rank: int,
            error_flag: Optional[torch.Tensor]) -> None:
    """proj: the fused projection [T, N] fp32 or its [S, T, N] partial sums; see csrc/latent.cu for what goes where.
    pages [num_pages, page_size, rank + rot_dim]; None: a run that reads another run's cache stores nothing."""
    n_partials, stride = 1, 0
    first = proj
    if proj.dim() == 3:
        ops._need(proj, "proj", torch.float32, 3)
        n_partials, stride = proj.shape[0], proj.shape[1] * proj.shape[2]
        first = proj[0]
    ops._need(first, "proj", torch.float32, 2)
    T = first.shape[0]
    ops._need(q_plain, "q_plain", dims=2); ops._need(q_full, "q_full", q_plain.dtype, 2)
    ops._need(norm_weight, "norm_weight", torch.float32, 1); ops._need(inv_freq, "inv_freq", torch.float32, 1)
    ops._need(positions, "positions", torch.int32, 1); ops._need(token_seq, "token_seq", torch.int32, 1)
    if (tuple(q_plain.shape) != (T, heads * dim) or tuple(q_full.shape) != (T, heads * (rank + rot_dim))
            or norm_weight.shape[0] != rank or inv_freq.shape[0] * 2 != rot_dims or positions.shape[0] != T):
        raise KernelError("latent.prepare: shapes do not agree")
    gate_width = 0
    if gate_out is not None:
        ops._need(gate_out, "gate_out", torch.float32, 2)
        gate_width = gate_out.shape[1]
        if gate_out.shape[0] != T:
            raise KernelError("latent.prepare: one gate row per token")
    if max(q_col + heads * (dim + rot_dim), kv_col + rank + rot_dim, gate_col + gate_width) > first.shape[1]:
        raise KernelError("latent.prepare: a column range runs past the projection")
    num_pages = page_size = max_blocks = 0
    if pages is not None:
        ops._need(pages, "pages", dims=3); ops._need(block_table, "block_table", torch.int32, 2)
        num_pages, page_size, width = pages.shape
        if width != rank + rot_dim:
            raise KernelError(f"latent.prepare: pages {tuple(pages.shape)} do not hold rows of {rank} + {rot_dim}")
        max_blocks = block_table.shape[1]
    L = ops.lib(SOURCE)
    build.check(L, L.mlb_latent_prepare(
        first.data_ptr(), first.stride(0), n_partials, stride, q_col, kv_col, gate_col, norm_weight.data_ptr(), float(eps),
        positions.data_ptr(), token_seq.data_ptr(), ops._ptr(block_table), max_blocks, inv_freq.data_ptr(), int(rot_dims),
        q_plain.data_ptr(), q_full.data_ptr(), ops.dtype_tag(q_plain), ops._ptr(pages),
        ops.dtype_tag(pages) if pages is not None else ops.F32, ops._ptr(gate_out), num_pages, page_size, T, heads, dim,
        rot_dim, rank, gate_width, ops._ptr(error_flag), ops._stream()))


def attention_plain(q: torch.Tensor, pages: torch.Tensor, out: torch.Tensor, sink: Optional[torch.Tensor],
                    positions: torch.Tensor, token_seq: torch.Tensor, block_table: torch.Tensor, heads: int, rank: int,
                    rot_dim: int, scale: float, window: Optional[int], error_flag: Optional[torch.Tensor]) -> None:
    """q [T, heads * (rank + rot_dim)], pages [num_pages, page_size, rank + rot_dim], out [T, heads * rank]."""
    ops._need(q, "q", dims=2); ops._need(pages, "pages", dims=3); ops._need(out, "out", dims=2)
    ops._need(block_table, "block_table", torch.int32, 2)
    T = q.shape[0]
    num_pages, page_size, width = pages.shape
    if width != rank + rot_dim or q.shape[1] != heads * width or tuple(out.shape) != (T, heads * rank) or positions.shape[0] != T:
        raise KernelError("latent.attention_plain: shapes do not agree")
    if sink is not None:
        ops._need(sink, "sink", torch.float32, 1)
        if sink.shape[0] != heads:
            raise KernelError("latent.attention_plain: one sink per head")
    L = ops.lib(SOURCE)
    build.check(L, L.mlb_latent_attention_plain(
        q.data_ptr(), ops.dtype_tag(q), pages.data_ptr(), ops.dtype_tag(pages), out.data_ptr(), ops.dtype_tag(out), ops._ptr(sink),
        positions.data_ptr(), token_seq.data_ptr(), block_table.data_ptr(), block_table.shape[1], num_pages, page_size, T,
        heads, rank, rot_dim, int(window or 0), float(scale), ops._ptr(error_flag), ops._stream()))
