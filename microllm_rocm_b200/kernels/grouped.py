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


def sources():
    return [(SOURCE, {})]


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
    L = ops.lib(SOURCE)
    build.check(L, L.mlb_grouped_gemm(
        a.data_ptr(), a.stride(0), a_group_cols, weight.data_ptr(), weight.stride(1), weight.stride(0), out.data_ptr(),
        out.stride(0), c_group_cols, ops._ptr(group_offsets), ops._ptr(a_rows), ops._ptr(c_rows), int(a_row_div),
        ops._ptr(factor), factor.stride(0) if factor is not None else 0, int(rows), N, K, G, ops.dtype_tag(a),
        ops.dtype_tag(out), int(row_tile), ops._stream()))
