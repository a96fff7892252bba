"""A recurrent block around a real-gated linear recurrent unit.

Two branches of ``width`` channels: ``y = gelu_tanh(W_y h + b_y)`` and ``u = conv(W_x h + b_x)``, a causal convolution
per channel over the last ``taps`` positions (zeros before the start of a request, no activation). ``u`` is cut into
``blocks`` equal parts; in part b ``r = sigmoid(A_b u_b + a_b)`` and ``i = sigmoid(B_b u_b + b_b)`` with square
matrices. Then per channel, in 32-bit, from S = 0:

    a = exp(-8 r softplus(lam)),        S <- a S + sqrt(1 - a^2) (i u),        out = W_o (S * y).

A request's state is S and the convolution's last ``taps - 1`` inputs.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..registry import register_part
from .base import LayerCache, Mixer, Runtime, StateNeed, StepContext
from .spec import PartSpec, TensorSpec


class GatedLinearRecurrence(Mixer):
    """params: ``hidden``, ``width``, ``taps``, ``blocks``. tensors: ``y x [width, hidden]``, ``y_b x_b``,
    ``conv [width, taps]`` (last column = the current token), ``conv_b``, ``ra ri [blocks, bw, bw]`` ([out, in]),
    ``ra_b ri_b [blocks, bw]``, ``lam [width]``, ``o [hidden, width]``."""

    graph_safe = True   # launches do not depend on which requests are in the batch

    @staticmethod
    def spec(prefix: str, hidden: int, width: int, taps: int, blocks: int) -> PartSpec:
        bw = width // blocks
        t = {
            "y": TensorSpec(f"{prefix}.y", (width, hidden)), "y_b": TensorSpec(f"{prefix}.y.b", (width,), "bias"),
            "x": TensorSpec(f"{prefix}.x", (width, hidden)), "x_b": TensorSpec(f"{prefix}.x.b", (width,), "bias"),
            "conv": TensorSpec(f"{prefix}.conv", (width, taps), "unit"), "conv_b": TensorSpec(f"{prefix}.conv.b", (width,), "bias"),
            "ra": TensorSpec(f"{prefix}.ra", (blocks, bw, bw)), "ra_b": TensorSpec(f"{prefix}.ra.b", (blocks, bw), "bias"),
            "ri": TensorSpec(f"{prefix}.ri", (blocks, bw, bw)), "ri_b": TensorSpec(f"{prefix}.ri.b", (blocks, bw), "bias"),
            "lam": TensorSpec(f"{prefix}.lam", (width,), "unit"),
            "o": TensorSpec(f"{prefix}.o", (hidden, width)),
        }
        return PartSpec("rglru", {"hidden": hidden, "width": width, "taps": taps, "blocks": blocks}, t)

    def __init__(self, spec: PartSpec, tensors: Dict[str, torch.Tensor], rt: Runtime):
        super().__init__(spec, tensors, rt)
        p = spec.params
        self.hidden, self.width, self.taps, self.blocks = int(p["hidden"]), int(p["width"]), int(p["taps"]), int(p["blocks"])
        if self.width % self.blocks:
            raise ValueError(f"width {self.width} is not a multiple of blocks {self.blocks}")
        self.bw = self.width // self.blocks
        # One product for both branches: rows [x | y]. One product per block for both gates: rows [recurrence | input].
        self.w_in = rt.matrix(torch.cat([tensors["x"], tensors["y"]], dim=0))
        self.b_in = rt.vector32(torch.cat([tensors["x_b"], tensors["y_b"]], dim=0))
        self.conv_w, self.conv_b = rt.vector32(tensors["conv"]), rt.vector32(tensors["conv_b"])
        self.w_gate = rt.matrix(torch.cat([tensors["ra"], tensors["ri"]], dim=1))              # [blocks, 2 bw, bw]
        self.b_gate = rt.vector32(torch.cat([tensors["ra_b"], tensors["ri_b"]], dim=1))        # [blocks, 2 bw]
        self.softplus_lam = rt.vector32(torch.nn.functional.softplus(tensors["lam"].to(torch.float32)))
        self.w_o = rt.matrix(tensors["o"])

    def state_need(self) -> StateNeed:
        # row 0: S; rows 1 .. taps-1: the convolution's last inputs, oldest first
        return StateNeed((self.taps, self.width), torch.float32)

    def forward(self, h: torch.Tensor, residual32: torch.Tensor, ctx: StepContext, cache: LayerCache) -> None:
        m, dev, w, ops = h.shape[0], h.device, self.width, self.ops
        xy32 = torch.empty((m, 2 * w), dtype=torch.float32, device=dev)
        ops.linear(h, self.w_in, self.b_in, xy32, "f32")
        u32 = torch.empty((m, w), dtype=torch.float32, device=dev)
        u_blocks = torch.empty((self.blocks, m, self.bw), dtype=self.rt.dtype, device=dev)
        ops.causal_conv(xy32[:, :w], self.conv_w, self.conv_b, cache.state, 1, ctx, u32, u_blocks, self.taps, self.blocks)
        gates = torch.empty((self.blocks, m, 2 * self.bw), dtype=torch.float32, device=dev)
        ops.block_diag_linear(u_blocks, self.w_gate, self.b_gate, gates, a32=u32)
        out = torch.empty((m, w), dtype=self.rt.dtype, device=dev)
        ops.rglru_scan(u32, gates, xy32[:, w:], xy32[:, :w], self.softplus_lam, cache.state, ctx, out, self.taps, self.blocks)
        ops.linear(out, self.w_o, None, residual32, "add")


register_part("rglru", GatedLinearRecurrence)
