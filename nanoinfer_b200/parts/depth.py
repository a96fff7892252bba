"""Depth-weighted average of a step's residual streams.

With ``X_0`` the embedding output and ``X_j`` the result of the j-th layer run, the stream that goes on after the
layer that produced ``X_(n-1)`` is ``sum_{j<n} coef[j] X_j``. The earlier streams of the step are kept in a 32-bit
buffer that lives in the step's context; the sum is made in 32-bit, ascending j.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..registry import register_part
from .base import PENDING_STREAM_OP, Part, Runtime, StepContext
from .spec import PartSpec, TensorSpec

_KEY = "depth_average.history"


class DepthAverage(Part):
    """params: ``inputs`` (n: how many streams are summed, the newest included), ``capacity`` (the most streams any
    layer of the model sums). tensors: ``coef [inputs]``."""

    graph_safe = True   # launches do not depend on which requests are in the batch

    @staticmethod
    def spec(name: str, inputs: int, capacity: int) -> PartSpec:
        return PartSpec("depth_average", {"inputs": inputs, "capacity": capacity},
                        {"coef": TensorSpec(name, (inputs,), "mix")})

    def __init__(self, spec: PartSpec, tensors: Dict[str, torch.Tensor], rt: Runtime):
        super().__init__(spec, tensors, rt)
        self.inputs, self.capacity = int(spec.params["inputs"]), int(spec.params["capacity"])
        if not (2 <= self.inputs <= self.capacity):
            raise ValueError(f"a depth average of {self.inputs} streams with room for {self.capacity}")
        self.coef = rt.vector32(tensors["coef"])

    def begin(self, x32: torch.Tensor, ctx: StepContext) -> None:
        """Before the layer runs: the first layer of a step keeps its input as stream 0."""
        if self.inputs == 2:
            hist = torch.empty((self.capacity,) + tuple(x32.shape), dtype=torch.float32, device=x32.device)
            hist[0].copy_(x32)
            ctx.scratch[_KEY] = hist

    def forward(self, x32: torch.Tensor, ctx: StepContext) -> None:
        """After the layer: x32 (the layer's result) is to join the streams and to be replaced by their weighted sum. The
        work is left pending in the step's context (``parts.base.PENDING_STREAM_OP``): whoever reads the stream next
        either runs it (``run``) or, if it norms the stream twice anyway, lets one kernel do both (``run_with_norms``)."""
        ctx.scratch[PENDING_STREAM_OP] = self

    def run(self, x32: torch.Tensor, ctx: StepContext) -> None:
        self.ops.depth_mix(ctx.scratch[_KEY], x32, self.coef, self.inputs)

    def run_with_norms(self, x32: torch.Tensor, ctx: StepContext, norm_a, norm_b):
        """The pending sum and the two RMS norms of its result (equal size and eps) in one pass; returns (h_a, h_b)."""
        a = torch.empty((x32.shape[0], norm_a.size), dtype=self.rt.dtype, device=x32.device)
        b = torch.empty_like(a)
        self.ops.depth_mix_norm_pair(ctx.scratch[_KEY], x32, self.coef, self.inputs, norm_a.gain, norm_b.gain, norm_a.eps, a, b)
        return a, b


register_part("depth_average", DepthAverage)
