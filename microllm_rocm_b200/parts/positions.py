"""Learned additive positions: row p of a table is added to the embedded token at position p, unscaled, in fp32.
Mixers get no rotation table from it; a mixer that rotates brings an encoding of its own."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..kernels import ops
from .base import PositionEncoding, Runtime, StepContext, WeightSpec, register_position_encoding


@register_position_encoding("learned")
class LearnedPositions(PositionEncoding):
    def __init__(self, params: dict, rt: Runtime):
        self.prefix = params.get("prefix", "")
        self.name = params.get("name", "weight")
        self.rows = int(params["max_position"])
        self.hidden = int(params["hidden_size"])
        self.rt = rt
        self.table: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {self.name: WeightSpec((self.rows, self.hidden), role="table")}

    def bind(self, tensors):
        self.table = tensors[self.name]

    def kernel_sources(self):
        return [("residual.cu", {})]

    def on_embedding(self, x: torch.Tensor, ctx: StepContext) -> None:
        ops.add_table_rows(x, self.table, ctx.positions)
