"""The generalized delta rule: a recurrent mixer with a matrix state per head.

With ``r, k, v`` the head's projections of the token (``d`` elements each), a decay per key channel
``w = exp(-exp(-1/2) * sigmoid(W_w2 tanh(W_w1 h) + w0))``, a removal rate per key channel ``a = sigmoid(W_a h + b_a)``
and the unit key ``u = k / sqrt(sum(k^2) + 1e-6)``, the state ``S`` (key channel x value channel, zero at the start of
a request, 32-bit) moves as

    S <- diag(w) S - (a * u)(u^T S) + k v^T        (both products read the old S),        o = S^T r.

Each head's ``o`` is divided by its root mean square, multiplied by a gain (all heads' size) and by
``sigmoid(W_g h)``; then ``W_o``, added to the residual stream. Everything that enters the recurrence is 32-bit: the
projections leave the matrix kernels as floats.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..registry import register_part
from .base import LayerCache, Mixer, Runtime, StateNeed, StepContext
from .spec import PartSpec, TensorSpec


class GeneralizedDeltaRule(Mixer):
    """params: ``hidden``, ``heads``, ``dim``, ``decay_rank`` (inner width of the decay's two-layer map), ``eps``
    (of the per-head norm). tensors: ``r k v g a [heads*dim, hidden]``, ``a_b``, ``w1 [decay_rank, hidden]``,
    ``w2 [heads*dim, decay_rank]``, ``w0``, ``norm [heads*dim]``, ``o [hidden, heads*dim]``."""

    graph_safe = True   # launches do not depend on which requests are in the batch

    @staticmethod
    def spec(prefix: str, hidden: int, heads: int, dim: int, decay_rank: int, eps: float) -> PartSpec:
        n = heads * dim
        t = {name: TensorSpec(f"{prefix}.{name}", (n, hidden)) for name in ("r", "k", "v", "g", "a")}
        t["a_b"] = TensorSpec(f"{prefix}.a.b", (n,), "bias")
        t["w1"] = TensorSpec(f"{prefix}.w1", (decay_rank, hidden))
        t["w2"] = TensorSpec(f"{prefix}.w2", (n, decay_rank))
        t["w0"] = TensorSpec(f"{prefix}.w0", (n,), "unit")
        t["norm"] = TensorSpec(f"{prefix}.norm", (n,), "gain")
        t["o"] = TensorSpec(f"{prefix}.o", (hidden, n))
        return PartSpec("general_delta", {"hidden": hidden, "heads": heads, "dim": dim, "decay_rank": decay_rank, "eps": eps}, t)

    def __init__(self, spec: PartSpec, tensors: Dict[str, torch.Tensor], rt: Runtime):
        super().__init__(spec, tensors, rt)
        p = spec.params
        self.hidden, self.heads, self.dim = int(p["hidden"]), int(p["heads"]), int(p["dim"])
        self.decay_rank, self.eps = int(p["decay_rank"]), float(p["eps"])
        n = self.n = self.heads * self.dim
        # One product for everything that reads h: rows [r | k | v | a | g | w1]; only a has a bias.
        self.w_in = rt.matrix(torch.cat([tensors[x] for x in ("r", "k", "v", "a", "g", "w1")], dim=0))
        bias = torch.zeros(5 * n + self.decay_rank, dtype=torch.float32)
        bias[3 * n:4 * n] = tensors["a_b"].to(torch.float32)
        self.b_in = rt.vector32(bias)
        self.w_2, self.w_0 = rt.matrix(tensors["w2"]), rt.vector32(tensors["w0"])
        self.gain = rt.vector32(tensors["norm"])
        self.w_o = rt.matrix(tensors["o"])

    def state_need(self) -> StateNeed:
        # per head [value channel, key channel]: a value column's key channels lie together
        return StateNeed((self.heads, self.dim, self.dim), torch.float32)

    def forward(self, h: torch.Tensor, residual32: torch.Tensor, ctx: StepContext, cache: LayerCache) -> None:
        m, dev, n, ops = h.shape[0], h.device, self.n, self.ops
        p32 = torch.empty((m, 5 * n + self.decay_rank), dtype=torch.float32, device=dev)
        ops.linear(h, self.w_in, self.b_in, p32, "f32")
        inner = torch.empty((m, self.decay_rank), dtype=self.rt.dtype, device=dev)
        ops.unary(p32[:, 5 * n:], inner, "tanh")
        w_logit = torch.empty((m, n), dtype=torch.float32, device=dev)
        ops.linear(inner, self.w_2, self.w_0, w_logit, "f32")
        o32 = torch.empty((m, n), dtype=torch.float32, device=dev)
        ops.delta_rule_scan(p32[:, :n], p32[:, n:2 * n], p32[:, 2 * n:3 * n], p32[:, 3 * n:4 * n], w_logit, cache.state,
                            ctx, o32, self.heads, self.dim)
        gated = torch.empty((m, n), dtype=self.rt.dtype, device=dev)
        ops.head_norm_gate(o32, p32[:, 4 * n:5 * n], self.gain, self.eps, self.heads, self.dim, gated)
        ops.linear(gated, self.w_o, None, residual32, "add")


register_part("general_delta", GeneralizedDeltaRule)
