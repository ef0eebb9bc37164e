"""Grouped matrix products: one product per group over that group's rows (`csrc/grouped_gemm.cu`).

Two uses: the experts of a routed feed-forward (groups = experts, rows = the tokens routed to each, known only on
the device) and the per-head products of latent attention (groups = heads, every group takes all rows).  fp32
operands run in true fp32 with a fixed summation order; bf16 operands accumulate in fp32.
"""
from __future__ import annotations

from ctypes import c_int, c_longlong, c_void_p
from typing import Optional

import torch

from . import build, ops
from .build import KernelError

SOURCE = "grouped_gemm.cu"
ops.register_signatures(SOURCE, {
    "mlb_grouped_gemm": [c_void_p, c_longlong, c_longlong, c_void_p, c_longlong, c_longlong, c_void_p, c_longlong, c_longlong,
                         c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_longlong, c_int, c_int, c_int, c_int, c_int, c_int,
                         c_int, c_void_p],
})


MMA_SOURCE = "grouped_mma.cu"
ops.register_signatures(MMA_SOURCE, {
    "mlb_grouped_mma": [c_void_p, c_longlong, c_longlong, c_void_p, c_longlong, c_longlong, c_void_p, c_longlong, c_longlong,
                        c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_longlong, c_longlong, c_int, c_int, c_int, c_int, c_int,
                        c_int, c_void_p],
})

# Tests set it to False to send bf16 products to the CUDA-core kernel and compare.
USE_TENSOR_CORES = True


def sources():
    return [(SOURCE, {}), (MMA_SOURCE, {})]


def mma_supported(a: torch.Tensor, weight: torch.Tensor, a_group_cols: int = 0) -> bool:
    """The tensor-core kernel moves 16-byte pieces: bf16 operands whose K, row pitches and column blocks are multiples
    of 8 elements."""
    return (USE_TENSOR_CORES and a.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and weight.shape[2] % 8 == 0
            and a.stride(0) % 8 == 0 and weight.stride(1) % 8 == 0 and weight.stride(0) % 8 == 0 and a_group_cols % 8 == 0
            and a.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0)


def row_tile_for(rows: int, groups: int, listed: bool, tensor_cores: bool) -> int:
    """Rows of a CTA's tile: 16 while a group holds few rows (decoding: a CTA should not multiply rows that do not
    exist), 128 on the tensor cores once the groups are large (twice the reuse of every weight tile), else 64."""
    per_group = rows / max(1, groups) if listed else rows
    if per_group <= 16:
        return 16
    return 128 if tensor_cores and per_group >= 96 else 64


def grouped_linear(a: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, *, rows: int, a_group_cols: int = 0,
                   c_group_cols: int = 0, group_offsets: Optional[torch.Tensor] = None, a_rows: Optional[torch.Tensor] = None,
                   c_rows: Optional[torch.Tensor] = None, a_row_div: int = 1, factor: Optional[torch.Tensor] = None,
                   row_tile: int = 64) -> None:
    """weight [G, N, K]; a [*, lda] and out [*, ldc] are 2-D and row-major.

    group g multiplies the K columns of `a` that start at g * a_group_cols with weight[g] and writes N columns of
    `out` starting at g * c_group_cols.  With `group_offsets` ([G + 1] int32 on the device) group g owns the places
    offsets[g]..offsets[g+1]-1 of a sorted list of `rows` places; `a_rows[place] // a_row_div` is the row read and
    `c_rows[place]` the row written (None: the place itself).  Without it every group takes rows 0..rows-1.
    `factor` (fp32, the shape of `out`): the result is multiplied by it element by element."""
    ops._need(a, "a", dims=2); ops._need(weight, "weight", dims=3); ops._need(out, "out", dims=2)
    if a.dtype != weight.dtype:
        raise KernelError(f"grouped_linear: operands are {a.dtype} and {weight.dtype}")
    G, N, K = weight.shape
    if a_group_cols * (G - 1) + K > a.shape[1] or c_group_cols * (G - 1) + N > out.shape[1]:
        raise KernelError("grouped_linear: a group's columns run past its matrix")
    for name, t in (("group_offsets", group_offsets), ("a_rows", a_rows), ("c_rows", c_rows)):
        if t is not None:
            ops._need(t, name, torch.int32, 1)
    if group_offsets is not None and group_offsets.shape[0] != G + 1:
        raise KernelError("grouped_linear: group_offsets must have one entry per group and one more")
    if factor is not None:
        ops._need(factor, "factor", torch.float32, 2)
        if factor.shape[1] < out.shape[1]:
            raise KernelError("grouped_linear: the factor matrix is narrower than the output")
    if row_tile == 128 and not mma_supported(a, weight, a_group_cols):
        row_tile = 64
    if mma_supported(a, weight, a_group_cols):
        L = ops.lib(MMA_SOURCE)
        build.check(L, L.mlb_grouped_mma(
            a.data_ptr(), a.stride(0), a_group_cols, weight.data_ptr(), weight.stride(1), weight.stride(0), out.data_ptr(),
            out.stride(0), c_group_cols, ops._ptr(group_offsets), ops._ptr(a_rows), ops._ptr(c_rows), int(a_row_div),
            ops._ptr(factor), factor.stride(0) if factor is not None else 0, 0, int(rows), N, K, G, ops.dtype_tag(out),
            int(row_tile), ops._stream()))
        return
    L = ops.lib(SOURCE)
    build.check(L, L.mlb_grouped_gemm(
        a.data_ptr(), a.stride(0), a_group_cols, weight.data_ptr(), weight.stride(1), weight.stride(0), out.data_ptr(),
        out.stride(0), c_group_cols, ops._ptr(group_offsets), ops._ptr(a_rows), ops._ptr(c_rows), int(a_row_div),
        ops._ptr(factor), factor.stride(0) if factor is not None else 0, int(rows), N, K, G, ops.dtype_tag(a),
        ops.dtype_tag(out), int(row_tile), ops._stream()))


def grouped_silu_mul(a: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, *, rows: int, group_offsets: torch.Tensor,
                     a_rows: Optional[torch.Tensor] = None, a_row_div: int = 1, row_tile: int = 64, alloc=None) -> None:
    """weight [G, 2 * F, K]: per group F gate rows over F up rows; out[place] = silu(a gate^T) * (a up^T), [rows, F].
    On the tensor cores both products and the activation are one kernel; otherwise the fused product leaves
    [rows, 2 * F] (from `alloc(shape, dtype)`) and the activation kernel follows."""
    ops._need(a, "a", dims=2); ops._need(weight, "weight", dims=3); ops._need(out, "out", dims=2)
    G, two_f, K = weight.shape
    F = two_f // 2
    if two_f % 2 or tuple(out.shape) != (rows, F):
        raise KernelError("grouped_silu_mul: the weight holds gate rows over up rows, the output one column per pair")
    if mma_supported(a, weight):
        ops._need(group_offsets, "group_offsets", torch.int32, 1)
        if a_rows is not None:
            ops._need(a_rows, "a_rows", torch.int32, 1)
        L = ops.lib(MMA_SOURCE)
        build.check(L, L.mlb_grouped_mma(
            a.data_ptr(), a.stride(0), 0, weight.data_ptr(), weight.stride(1), weight.stride(0), out.data_ptr(), out.stride(0), 0,
            group_offsets.data_ptr(), ops._ptr(a_rows), None, int(a_row_div), None, 0, F, int(rows), F, K, G,
            ops.dtype_tag(out), int(row_tile), ops._stream()))
        return
    row_tile = min(row_tile, 64)
    gate_up = alloc((rows, two_f), a.dtype) if alloc is not None else torch.empty((rows, two_f), dtype=a.dtype, device=a.device)
    grouped_linear(a, weight, gate_up, rows=rows, group_offsets=group_offsets, a_rows=a_rows, a_row_div=a_row_div, row_tile=row_tile)
    ops.silu_mul(gate_up, out)
