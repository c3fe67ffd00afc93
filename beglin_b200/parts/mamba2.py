"""The Mamba-2 mixer: a recurrence with a matrix-valued state per head.

One product of the mixer's input gives, side by side, the gate z, the inputs x, B and C of the recurrence and
the step sizes dt.  x, B and C pass a short causal convolution per channel and SiLU; then, per head h (with
B and C of the head's group), for each token in turn
    dt = softplus(dt + dt_bias[h]);  S = exp(-exp(A_log[h]) dt) S + dt B x^T;  y = S^T C + D[h] x.
The gated rows y * silu(z) are RMS-normed in equal parts of the row and go through the output product.

The state S and the last conv - 1 inputs of the convolution are per-request state of fixed size (one slot of
the cache manager's slab, float32, zero when the request starts): a step continues each request from its
slot, however the request's tokens are cut into steps and whatever else the step holds.  Everything that
enters the recurrence is float in both number formats.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..csrc import ops
from .cache_need import FixedStateNeed, FixedStateView
from .context import BuildContext
from .linear import Linear
from .registry import register_mixer
from .spec import Mamba2Spec, TensorRole
from .stream import NormedInput, ResidualStream


def _sizes(spec: Mamba2Spec):
    inner = spec.n_heads * spec.vdim
    channels = inner + 2 * spec.groups * spec.state
    return inner, channels


@register_mixer("mamba2")
class Mamba2:
    @staticmethod
    def expected_tensors(spec: Mamba2Spec) -> List[TensorRole]:
        inner, channels = _sizes(spec)
        H = spec.n_heads
        return [TensorRole("in_proj.weight", (inner + channels + H, spec.hidden), True, True),
                TensorRole("conv.weight", (channels, spec.conv)),
                TensorRole("conv.bias", (channels,), role="bias"),
                TensorRole("dt_bias", (H,), role="bias"),
                TensorRole("A_log", (H,)),
                TensorRole("D", (H,)),
                TensorRole("norm.weight", (inner,), role="scale"),
                TensorRole("o_proj.weight", (spec.hidden, inner), True, True)]

    @staticmethod
    def cache_need(spec: Mamba2Spec) -> FixedStateNeed:
        inner, channels = _sizes(spec)
        return FixedStateNeed((spec.n_heads * spec.state * spec.vdim + (spec.conv - 1) * channels,), "float32")

    def __init__(self, spec: Mamba2Spec, tensors: Dict[str, torch.Tensor], ctx: BuildContext):
        if spec.n_heads % spec.groups:
            raise ValueError(f"{spec.n_heads} heads are not a multiple of {spec.groups} groups")
        inner, channels = _sizes(spec)
        if inner % spec.norm_groups:
            raise ValueError(f"{inner} features do not fall into {spec.norm_groups} equal parts")
        if spec.conv < 1:
            raise ValueError("the convolution has at least one tap")
        self.spec, self.ctx = spec, ctx
        self.inner, self.channels = inner, channels
        self.in_proj = Linear(tensors["in_proj.weight"], None, ctx, label="proj_in")
        self.o_proj = Linear(tensors["o_proj.weight"], None, ctx, label="proj_o")
        same = lambda t: t.to(device=ctx.device, dtype=ctx.compute_dtype).contiguous()
        self.conv_w, self.conv_b = same(tensors["conv.weight"]), same(tensors["conv.bias"])
        self.dt_bias, self.A_log, self.D = same(tensors["dt_bias"]), same(tensors["A_log"]), same(tensors["D"])
        self.norm_w = ctx.vector(tensors["norm.weight"])
        self.conv_off = spec.n_heads * spec.state * spec.vdim

    takes_stream = True        # forward takes a NormedInput and may add its result to the stream itself

    def forward(self, h, batch, cache: FixedStateView, stream: Optional[ResidualStream] = None) -> Optional[torch.Tensor]:
        """h: the normed rows, or a NormedInput.  With `stream` the result is added to it (or left owed to it) and None
        is returned; without, the addend is returned."""
        if isinstance(h, NormedInput):
            h = h.tensor()
        s, ctx = self.spec, self.ctx
        T = batch.n_rows
        proj = self.in_proj(h, out_dtype=torch.float32)                 # [T, z | x B C | dt]
        reqs, n_req = batch.query_blocks(1 << 30)                       # one (request, first row, rows) per request
        xbc = torch.empty((T, self.channels), dtype=torch.float32, device=h.device)
        ops.conv_silu(proj, self.inner, self.channels, self.conv_w, self.conv_b, cache.state, self.conv_off, cache.slots,
                      batch.row_req, reqs, n_req, xbc)
        y = torch.empty((T, self.inner), dtype=torch.float32, device=h.device)
        ops.ssm_scan(xbc, proj, self.inner + self.channels, self.dt_bias, self.A_log, self.D, cache.state, cache.slots,
                     reqs, n_req, y, s.n_heads, s.vdim, s.state, s.groups)
        out = torch.empty((T, self.inner), dtype=ctx.compute_dtype, device=h.device)
        ops.gated_group_rmsnorm(y, proj, 0, self.norm_w, s.eps, s.norm_groups, out)
        if stream is None:
            return self.o_proj.partial(out)
        self.o_proj.into(out, stream)
        return None
