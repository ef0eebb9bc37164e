"""What a pass of looped layers adds to the residual stream before its first layer: row `row` of a table with one
row per pass, and (for every pass but the first) the embedding output of the step once more."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..kernels import ops
from .base import RunEntry, Runtime, StepContext, WeightSpec, register_run_entry


@register_run_entry("pass_entry")
class PassEntry(RunEntry):
    def __init__(self, params: dict, rt: Runtime):
        self.prefix = params.get("prefix", "")
        self.name = params["name"]
        self.rows = int(params["rows"])
        self.row = int(params["row"])
        self.hidden = int(params["hidden_size"])
        self.needs_embedding = bool(params.get("add_embedding", False))
        if not 0 <= self.row < self.rows:
            raise ValueError(f"pass entry: row {self.row} of a table of {self.rows}")
        self.rt = rt
        self.vector: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {self.name: WeightSpec((self.rows, self.hidden), role="vector")}

    def kernel_sources(self):
        return [("residual.cu", {})]

    def bind(self, tensors):
        self.vector = tensors[self.name][self.row]          # a contiguous row of the fp32 table

    def forward(self, residual: torch.Tensor, ctx: StepContext, embedding_output: Optional[torch.Tensor]) -> None:
        if self.needs_embedding and embedding_output is None:
            raise RuntimeError("pass entry: the embedding output was not kept")
        ops.stream_entry(residual, embedding_output if self.needs_embedding else None, self.vector)
