"""Routing of tokens to experts on the device (`csrc/moe.cu`): router logits, choice and weights; the list of
(token, choice) pairs sorted by expert; the weighted sum of the experts' results."""
from __future__ import annotations

from ctypes import c_int, c_longlong, c_void_p
from typing import Optional

import torch

from . import build, ops
from .build import KernelError

SOURCE = "moe.cu"
ops.register_signatures(SOURCE, {
    "mlb_moe_route": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p,
                      c_void_p],
    "mlb_moe_align": [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p],
    "mlb_moe_combine": [c_void_p, c_void_p, c_void_p, c_int, c_longlong, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                        c_void_p],
})


def sources():
    return [(SOURCE, {})]


def route(x: torch.Tensor, router: torch.Tensor, bias: Optional[torch.Tensor], top: int, ids: torch.Tensor,
          weights: torch.Tensor, shared_gate: Optional[torch.Tensor] = None, gate_out: Optional[torch.Tensor] = None) -> None:
    """x [T, W] and router [E, W] in one dtype; bias [E] fp32.  ids [T, top] int32 and weights [T, top] fp32 receive the
    chosen experts in order of their logits and the softmax over the chosen logits.  shared_gate [1, W] (x's dtype)
    and gate_out [T] fp32: sigmoid(x . shared_gate) per token."""
    ops._need(x, "x", dims=2); ops._need(router, "router", x.dtype, 2)
    ops._need(ids, "ids", torch.int32, 2); ops._need(weights, "weights", torch.float32, 2)
    T, W = x.shape
    E = router.shape[0]
    if router.shape[1] != W or tuple(ids.shape) != (T, top) or tuple(weights.shape) != (T, top):
        raise KernelError("moe.route: shapes do not agree")
    if bias is not None:
        ops._need(bias, "bias", torch.float32, 1)
        if bias.shape[0] != E:
            raise KernelError("moe.route: one bias per expert")
    if (shared_gate is None) != (gate_out is None):
        raise KernelError("moe.route: the shared gate's row and its output come together")
    if shared_gate is not None:
        ops._need(shared_gate, "shared_gate", x.dtype); ops._need(gate_out, "gate_out", torch.float32, 1)
        if shared_gate.numel() != W or gate_out.shape[0] != T:
            raise KernelError("moe.route: the shared gate is one row of the input's width, its output one number per token")
    L = ops.lib(SOURCE)
    build.check(L, L.mlb_moe_route(x.data_ptr(), router.data_ptr(), ops._ptr(bias), ops._ptr(shared_gate), ops.dtype_tag(x),
                                   T, W, E, int(top), ids.data_ptr(), weights.data_ptr(), ops._ptr(gate_out), ops._stream()))


def align(ids: torch.Tensor, experts: int, offsets: torch.Tensor, sorted_pairs: torch.Tensor,
          error_flag: Optional[torch.Tensor] = None) -> None:
    """ids [T, top] -> offsets [experts + 1], sorted_pairs [T * top] (indices t * top + j grouped by expert)."""
    ops._need(ids, "ids", torch.int32); ops._need(offsets, "offsets", torch.int32, 1)
    ops._need(sorted_pairs, "sorted_pairs", torch.int32, 1)
    if offsets.shape[0] != experts + 1 or sorted_pairs.shape[0] != ids.numel():
        raise KernelError("moe.align: shapes do not agree")
    L = ops.lib(SOURCE)
    build.check(L, L.mlb_moe_align(ids.data_ptr(), ids.numel(), int(experts), offsets.data_ptr(), sorted_pairs.data_ptr(),
                                   ops._ptr(error_flag), ops._stream()))


def combine(y: torch.Tensor, weights: torch.Tensor, out: torch.Tensor, shared: Optional[torch.Tensor] = None,
            gate: Optional[torch.Tensor] = None, col_scale: Optional[torch.Tensor] = None) -> None:
    """out[t] = (sum_j weights[t, j] * y[t * top + j] + gate[t] * shared[t]) * col_scale; shared may be [S, T, W]
    partial sums."""
    ops._need(y, "y", torch.float32, 2); ops._need(weights, "weights", torch.float32, 2); ops._need(out, "out", torch.float32, 2)
    T, top = weights.shape
    W = out.shape[1]
    if out.shape[0] != T or tuple(y.shape) != (T * top, W):
        raise KernelError("moe.combine: shapes do not agree")
    n_shared, stride = 0, 0
    if shared is not None:
        n_shared, stride = ops._partials(shared, out.shape, "moe.combine shared")
    for name, t, n in (("gate", gate, T), ("col_scale", col_scale, W)):
        if t is not None:
            ops._need(t, name, torch.float32, 1)
            if t.shape[0] != n:
                raise KernelError(f"moe.combine: {name} has the wrong length")
    L = ops.lib(SOURCE)
    build.check(L, L.mlb_moe_combine(y.data_ptr(), weights.data_ptr(), ops._ptr(shared), n_shared, stride, ops._ptr(gate),
                                     ops._ptr(col_scale), out.data_ptr(), T, W, top, ops._stream()))
