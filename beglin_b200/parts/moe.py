"""Routed experts: every token goes through `top` of `experts` small feed-forwards, chosen by the largest router scores.

A step's (token, rank) assignments are laid out expert by expert on the device, the experts' products run as ONE grouped
product each (up with the activation in its epilogue, then down), and the results are added per token in rank order.
Nothing is read back to the host and every grid depends on the step's shapes alone, so the step can be captured.  The
router's logits are float whatever the compute type; its matrix is kept in float32.  A row's result is a function of that
row alone (each output summed over the inner size in index order), so it does not depend on what else the step holds.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List

import torch

from ..csrc import ops
from .context import BuildContext
from .registry import register_feed_forward
from .spec import RoutedExpertsSpec, TensorRole


@dataclass
class RoutedRows:
    """The experts' results before they are added up per token: rows [T * top, hidden] float32 laid out expert by expert,
    `row_of[t * top + j]` the row of token t's rank j, `weights` the chosen scores, `scale` whether they still multiply.
    A norm that stands behind the experts adds the rows up itself (`RMSNorm.norm_add`)."""
    rows: torch.Tensor
    row_of: torch.Tensor
    weights: torch.Tensor
    top: int
    scale: bool


@register_feed_forward("routed_experts")
class RoutedExperts:
    @staticmethod
    def expected_tensors(spec: RoutedExpertsSpec) -> List[TensorRole]:
        roles = [TensorRole("router.weight", (spec.experts, spec.hidden), True, True)]
        for e in range(spec.experts):
            roles += [TensorRole(f"experts.{e}.up.weight", (spec.intermediate, spec.hidden), True, True),
                      TensorRole(f"experts.{e}.down.weight", (spec.hidden, spec.intermediate), True, True)]
        return roles

    gives_rows = True          # forward(..., summed=False) hands out RoutedRows

    def __init__(self, spec: RoutedExpertsSpec, tensors: Dict[str, torch.Tensor], ctx: BuildContext):
        if spec.activation not in ops.EXPERT_ACTIVATIONS or spec.activation == "none":
            raise ValueError(f"unknown activation '{spec.activation}' of an expert (relu2)")
        if spec.router_activation not in ("sigmoid", "none"):
            raise ValueError(f"unknown router activation '{spec.router_activation}' (sigmoid, none)")
        if not 1 <= spec.top <= min(spec.experts, 32):
            raise ValueError(f"top={spec.top} must be between 1 and the number of experts ({spec.experts}), at most 32")
        self.spec, self.ctx = spec, ctx
        self.router = tensors["router.weight"].to(device=ctx.device, dtype=torch.float32).contiguous()
        self.up = torch.stack([ctx.matrix(tensors[f"experts.{e}.up.weight"]) for e in range(spec.experts)]).contiguous()
        self.down = torch.stack([ctx.matrix(tensors[f"experts.{e}.down.weight"]) for e in range(spec.experts)]).contiguous()
        self.tensor_cores = ctx.gemm != "library"

    def forward(self, h: torch.Tensor, batch, summed: bool = True):
        """h [T, hidden] in the compute type -> the sum of the chosen experts' results, float32 [T, hidden]; or, with
        `summed` False, the results as `RoutedRows`, for a consumer that adds them up itself."""
        if not isinstance(h, torch.Tensor):
            h = h.tensor()
        s, dev, ct = self.spec, h.device, self.ctx.compute_dtype
        T, A = h.shape[0], h.shape[0] * s.top
        ints = torch.empty((3 * A + s.experts + 1,), dtype=torch.int32, device=dev)
        ids, row_of, src_of, offsets = ints[:A].view(T, s.top), ints[A:2 * A], ints[2 * A:3 * A], ints[3 * A:]
        weights = torch.empty((T, s.top), dtype=torch.float32, device=dev)
        ops.route(h, self.router, s.top, ids, weights, sigmoid=s.router_activation == "sigmoid", renorm=s.renormalize)
        ops.route_sort(ids.view(-1), s.experts, offsets, row_of, src_of)
        xp = torch.empty((A, s.hidden), dtype=ct, device=dev)
        ops.route_gather(h, weights.view(-1), src_of, xp, s.top, scale=s.scale_input)
        hp = torch.empty((A, s.intermediate), dtype=ct, device=dev)
        ops.gemm_grouped(xp, self.up, offsets, hp, s.activation, self.ctx.status, self.tensor_cores)
        yp = torch.empty((A, s.hidden), dtype=torch.float32, device=dev)
        ops.gemm_grouped(hp, self.down, offsets, yp, "none", self.ctx.status, self.tensor_cores)
        if not summed:
            return RoutedRows(yp, row_of, weights.view(-1), s.top, not s.scale_input)
        out = torch.empty((T, s.hidden), dtype=torch.float32, device=dev)
        ops.route_combine(yp, weights.view(-1), row_of, out, s.top, scale=not s.scale_input)
        return out
