"""The depth-weighted average.  Call R_0 the scaled embedding rows and R_(j+1) the stream as layer j's sublayers
leave it (no averaging applied yet).  Layer i hands on  sum_{j = 0 .. i+1} w[j] R_j  with a learned vector w of
its own.  The R_j of a step are kept, float, in the stream's `history`; one kernel per layer adds what the
layer's last part still owes to the stream, stores the sum as R_(i+1) and overwrites the stream with the
weighted sum."""
from __future__ import annotations

from typing import Dict, List

import torch

from ..csrc import ops
from .context import BuildContext
from .registry import register_combiner
from .spec import DepthAverageSpec, TensorRole
from .stream import ResidualStream


@register_combiner("depth_average")
class DepthAverage:
    @staticmethod
    def expected_tensors(spec: DepthAverageSpec) -> List[TensorRole]:
        return [TensorRole("weight", (spec.terms,), role="average")]

    def __init__(self, spec: DepthAverageSpec, tensors: Dict[str, torch.Tensor], ctx: BuildContext):
        if not 2 <= spec.terms <= spec.total:
            raise ValueError(f"a depth average over {spec.terms} of {spec.total} results")
        self.spec, self.ctx = spec, ctx
        self.weight = ctx.vector(tensors["weight"])

    def begin(self, stream: ResidualStream) -> None:
        """Before the first averaged layer's sublayers run: keep the embedding output."""
        if stream.history is None:
            if stream.pending is not None:
                raise ops.KernelError("the depth average starts from a stream to which nothing is owed")
            stream.history = torch.empty((self.spec.total,) + tuple(stream.x.shape), dtype=torch.float32, device=stream.x.device)
            stream.history[0].copy_(stream.x)

    def forward(self, stream: ResidualStream, batch) -> None:
        ops.depth_mix(stream.x, stream.pending, stream.history, self.weight, self.spec.terms)
        stream.updated(None)
