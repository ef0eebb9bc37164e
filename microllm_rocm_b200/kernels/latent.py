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

MMA_SOURCE = "latent_mma.cu"
ops.register_signatures(MMA_SOURCE, {
    "mlb_latent_mma_widths": [c_int],
    "mlb_latent_attention_mma": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                 c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p],
})
ROWS_PER_TILE = 16                  # (token, head) rows of one sequence that a CTA of the tensor-core kernel owns
KEYS_PER_TILE = 32
MIN_KEY_TILES_PER_SPLIT = 4         # a CTA that shares a work item's keys streams 128 of them at least
MAX_SPLITS = 64
USE_TENSOR_CORES = True             # tests set it to False to run the plain kernel on the same inputs


def mma_supported(rank: int, rot_dim: int) -> bool:
    return rank % 32 == 0 and (rank + rot_dim) % 16 == 0 and rank <= MAX_RANK


def mma_sources(rank: int, rot_dim: int):
    return [(MMA_SOURCE, {"LAT_R": rank, "LAT_DR": rot_dim})] if mma_supported(rank, rot_dim) else []


def key_splits(num_work: int, max_seq_len: int, sms: int) -> int:
    """How many CTAs share the keys of one work item: enough to give every multiprocessor two CTAs, while each still
    streams a few key tiles."""
    key_tiles = max(1, -(-max_seq_len // KEYS_PER_TILE))
    return max(1, min((2 * sms) // max(1, num_work), key_tiles // MIN_KEY_TILES_PER_SPLIT, MAX_SPLITS))


def _plan(ctx, heads: int):
    """Work items of a step ((sequence, first row) per 16 rows of a sequence's new (token, head) rows; long causal
    ranges first) and the key split, shared by every layer with this many heads."""
    from .device import sm_count
    key = ("latent_mma", heads)
    plan = ctx.extras.get(key)
    if plan is not None:
        return plan
    starts = ctx.seq_starts_host
    work = []
    for a in range(ctx.num_seqs):
        rows = (starts[a + 1] - starts[a]) * heads
        pos0 = ctx.seq_pos0_host[a] if ctx.seq_pos0_host else 0
        work += [(pos0 + first // heads, a, first) for first in range(0, rows, ROWS_PER_TILE)]
    if not ctx.decode_only:
        work.sort(key=lambda item: -item[0])
    device = ctx.positions.device
    work_dev = ops.upload([x for _, a, first in work for x in (a, first)], "int32", device)
    splits = key_splits(len(work), ctx.max_seq_len, sm_count(device)) if ctx.decode_only or len(work) <= 32 else 1
    plan = ctx.extras[key] = (work_dev, len(work), splits)
    return plan


def plan_stale(ctx, max_seq_len: int) -> bool:
    from .device import sm_count
    for key, plan in ctx.extras.items():
        if isinstance(key, tuple) and key and key[0] == "latent_mma":
            if key_splits(plan[1], max_seq_len, sm_count(ctx.positions.device)) != plan[2]:
                return True
    return False


def forget_plans(ctx) -> None:
    for key in [k for k in ctx.extras if isinstance(k, tuple) and k and k[0] == "latent_mma"]:
        del ctx.extras[key]


def attention(q: torch.Tensor, pages: torch.Tensor, out: torch.Tensor, sink: Optional[torch.Tensor], ctx,
              block_table: torch.Tensor, heads: int, rank: int, rot_dim: int, scale: float, window: Optional[int]) -> None:
    """The step's attention over the compressed cache: bf16 on the tensor cores when the widths suit them, else (and
    always in fp32) the plain kernel."""
    if not (USE_TENSOR_CORES and q.dtype == torch.bfloat16 and pages.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
            and mma_supported(rank, rot_dim)):
        attention_plain(q, pages, out, sink, ctx.positions, ctx.token_seq, block_table, heads, rank, rot_dim, scale, window,
                        ctx.error_flag)
        return
    ops._need(q, "q", torch.bfloat16, 2); ops._need(pages, "pages", torch.bfloat16, 3); ops._need(out, "out", torch.bfloat16, 2)
    T = q.shape[0]
    num_pages, page_size, width = pages.shape
    if width != rank + rot_dim or q.shape[1] != heads * width or tuple(out.shape) != (T, heads * rank):
        raise KernelError("latent.attention: shapes do not agree")
    work, num_work, splits = _plan(ctx, heads)
    part_o = part_ml = None
    if splits > 1:
        part_o = ctx.buffer("latent.part_o", (splits, T * heads, rank), torch.float32)
        part_ml = ctx.buffer("latent.part_ml", (splits, T * heads, 2), torch.float32)
    L = ops.lib(MMA_SOURCE, {"LAT_R": rank, "LAT_DR": rot_dim})
    build.check(L, L.mlb_latent_attention_mma(
        q.data_ptr(), pages.data_ptr(), out.data_ptr(), ops._ptr(sink), ctx.seq_starts.data_ptr(), ctx.seq_pos0.data_ptr(),
        block_table.data_ptr(), work.data_ptr(), num_work, ops._ptr(part_o), ops._ptr(part_ml), block_table.shape[1], num_pages,
        page_size, heads, int(window or 0), splits, T * heads, float(scale), ops._ptr(ctx.error_flag), ops._stream()))


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
