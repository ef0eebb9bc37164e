"""Several mixers side by side: every branch reads the same input, and the results are added with fixed weights,

  out = sum_b  scale_b * branch_b(x).

`branches` = ((name, scale, PartSpec of a mixer), ...); a branch's tensors live under `<name>.`-prefixed names (the
prefix in its own params), its caches under the sub-name `name`.  A block that can add weighted terms itself asks for
them (`forward_terms`) and spares the pass that `forward` needs to add them up.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from ..kernels import ops
from .base import MIXERS, CompositeNeed, Mixer, PositionEncoding, Runtime, StepContext, WeightSpec, make, register_mixer, sub_views


@register_mixer("parallel")
class ParallelMixers(Mixer):
    def __init__(self, params: dict, rt: Runtime, position: Optional[PositionEncoding] = None):
        from .base import POSITION_ENCODINGS
        self.prefix = params.get("prefix", "")
        self.hidden = int(params["hidden_size"])
        self.rt = rt
        self.branches: List[Tuple[str, float, str, Mixer]] = []       # (name, scale, tensor prefix, mixer)
        self._positions = []
        for name, scale, spec in params["branches"]:
            if spec.kind not in MIXERS:
                raise KeyError(f"unknown mixer kind {spec.kind!r}; registered: {', '.join(sorted(MIXERS))}")
            own_position = position
            if "position" in spec.params:            # a branch may bring its own encoding
                own_position = make(POSITION_ENCODINGS, "position encoding", spec.params["position"], rt)
                self._positions.append((spec.params.get("prefix", "") + spec.params["position"].params.get("prefix", ""), own_position))
            self.branches.append((name, float(scale), spec.params.get("prefix", ""), MIXERS[spec.kind](spec.params, rt, own_position)))
        if not self.branches:
            raise ValueError("parallel: at least one branch")
        self.graph_safe = all(m.graph_safe for _, _, _, m in self.branches)

    def _parts(self):
        return [(prefix, mixer) for _, _, prefix, mixer in self.branches] + list(self._positions)

    # --- declarations: everything is the branches', under their prefixes -------------------
    def cache_need(self):
        items = tuple((name, mixer.cache_need()) for name, _, _, mixer in self.branches)
        return CompositeNeed(items) if any(need is not None for _, need in items) else None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {prefix + local: ws for prefix, part in self._parts() for local, ws in part.weight_specs().items()}

    def fused_tensors(self):
        out = {}
        for prefix, part in self._parts():
            for dest, (spec, pieces) in part.fused_tensors().items():
                out[prefix + dest] = (spec, [(prefix + local, row) for local, row in pieces])
        return out

    def kernel_sources(self):
        out = [("residual.cu", {})]
        for _, part in self._parts():
            out += [item for item in part.kernel_sources() if item not in out]
        return out

    def bind(self, tensors):
        for prefix, part in self._parts():
            part.bind({name[len(prefix):]: t for name, t in tensors.items() if name.startswith(prefix)})

    def replay_key(self):
        keys = [m.replay_key() for _, _, _, m in self.branches]
        return None if any(k is None for k in keys) else ("parallel", tuple((n, s) for n, s, _, _ in self.branches), *keys)

    def own_tensors(self):
        return [t for _, _, _, m in self.branches for t in m.own_tensors()]

    def plan_stale(self, ctx: StepContext, max_seq_len: int) -> bool:
        return any(m.plan_stale(ctx, max_seq_len) for _, _, _, m in self.branches)

    def forget_plans(self, ctx: StepContext) -> None:
        for _, _, _, m in self.branches:
            m.forget_plans(ctx)

    def plan_group(self):
        return ("parallel", tuple(m.plan_group() for _, _, _, m in self.branches))

    # --- compute ------------------------------------------------------------------------
    def forward_terms(self, x: torch.Tensor, ctx: StepContext, cache):
        """[(scale, result of the branch [T, H] fp32 or its [S, T, H] partial results), ...]"""
        views = cache or {}
        return [(scale, mixer.forward(x, ctx, sub_views(views, name))) for name, scale, _, mixer in self.branches]

    def forward(self, x: torch.Tensor, ctx: StepContext, cache) -> torch.Tensor:
        out = ctx.buffer("parallel.out", (x.shape[0], self.hidden), torch.float32)
        out.zero_()
        for scale, term in self.forward_terms(x, ctx, cache):
            key = ("parallel.scale", scale)
            column_scale = ctx.extras.get(key)
            if column_scale is None:
                column_scale = ctx.extras[key] = torch.full((self.hidden,), scale, dtype=torch.float32, device=x.device)
            ops.add_scaled_inplace(out, term, column_scale)
        return out
