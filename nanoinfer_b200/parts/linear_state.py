"""Mixers whose memory is a matrix per head that decays and takes one outer product per token:

    S_t = diag(w_t) S_(t-1) + k_t v_t^T          (S: key channel x value channel, 32-bit, zero at a request's start)

read either after the update (``o_t = S_t^T q_t``) or before it with a bonus for the current token
(``o_t = (S_(t-1) + diag(u) k_t v_t^T)^T q_t``). One kernel walks all of them (``ops.linear_state_scan``); the classes
differ in where q, k, v and the decay come from and in what happens to o:

* ``GatedLinearAttention``: ``q = W_q h / sqrt(dim)``, ``k = W_k h``, ``v = W_v h``, decay per key channel
  ``sigmoid(W_a2 W_a1 h + b)^(1/tau)``; o is RMS-normed per head (gain of ``vdim``, shared by the heads), times
  ``silu(W_g h)``, then ``W_o``.
* ``ShiftedTimeMix``: each of r, k, v, g, w reads ``h + (h_prev - h) * mu_s`` (``h_prev``: the token before, zeros at the
  start; the last h of a request is kept in its state); decay ``exp(-exp(W_w2 tanh(W_w1 x_w) + w0))``; read before the
  update with the bonus ``u``; o is divided by its root mean square per head, times a gain of all heads' size, times
  ``silu(W_g x_g)``, then ``W_o``.
* ``Mamba2Mixer``: ``W_in h = [z | x | B | C | dt]``; x, B, C pass a short causal convolution with bias and silu (its
  last inputs are kept in the state); ``dt = softplus(dt + dt_bias)``; per head the decay is the scalar
  ``exp(-exp(A_log) dt)``, ``k = B`` and ``q = C`` of the head's group, ``v = dt x``; ``y = o + D x``, times ``silu(z)``,
  RMS-normed in ``norm_groups`` equal parts, times a gain, then ``W_o``.

Everything that enters the walk is 32-bit: the projections leave the matrix kernels as floats. Each adds
``out_scale`` times its result to the residual stream.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..registry import register_part
from .base import LayerCache, Mixer, Runtime, StateNeed, StepContext, as_tensor
from .spec import PartSpec, TensorSpec


class GatedLinearAttention(Mixer):
    """params: ``hidden heads dim vdim decay_rank tau eps out_scale``. tensors: ``q k [heads*dim, hidden]``,
    ``v g [heads*vdim, hidden]``, ``a1 [decay_rank, hidden]``, ``a2 [heads*dim, decay_rank]``, ``a2_b``, ``norm [vdim]``,
    ``o [hidden, heads*vdim]``."""

    graph_safe = True   # launches do not depend on which requests are in the batch

    @staticmethod
    def spec(prefix: str, hidden: int, heads: int, dim: int, vdim: int, decay_rank: int, tau: float, eps: float,
             out_scale: float = 1.0) -> PartSpec:
        nk, nv = heads * dim, heads * vdim
        t = {"q": TensorSpec(f"{prefix}.q", (nk, hidden)), "k": TensorSpec(f"{prefix}.k", (nk, hidden)),
             "v": TensorSpec(f"{prefix}.v", (nv, hidden)), "g": TensorSpec(f"{prefix}.g", (nv, hidden)),
             "a1": TensorSpec(f"{prefix}.a1", (decay_rank, hidden)), "a2": TensorSpec(f"{prefix}.a2", (nk, decay_rank)),
             "a2_b": TensorSpec(f"{prefix}.a2.b", (nk,), "unit"), "norm": TensorSpec(f"{prefix}.norm", (vdim,), "gain"),
             "o": TensorSpec(f"{prefix}.o", (hidden, nv))}
        return PartSpec("gated_linear_attention", {"hidden": hidden, "heads": heads, "dim": dim, "vdim": vdim,
                                                   "decay_rank": decay_rank, "tau": float(tau), "eps": float(eps),
                                                   "out_scale": float(out_scale)}, t)

    def __init__(self, spec: PartSpec, tensors: Dict[str, torch.Tensor], rt: Runtime):
        super().__init__(spec, tensors, rt)
        p = spec.params
        self.heads, self.dim, self.vdim, self.rank = int(p["heads"]), int(p["dim"]), int(p["vdim"]), int(p["decay_rank"])
        self.tau, self.eps, self.out_scale = float(p["tau"]), float(p["eps"]), float(p.get("out_scale", 1.0))
        self.nk, self.nv = self.heads * self.dim, self.heads * self.vdim
        # One product for everything that reads h: rows [q | k | v | g | a1].
        self.w_in = rt.matrix(torch.cat([tensors[x] for x in ("q", "k", "v", "g", "a1")], dim=0))
        self.w_a2, self.b_a2 = rt.matrix(tensors["a2"]), rt.vector32(tensors["a2_b"])
        self.gain = rt.vector32(tensors["norm"])
        self.w_o = rt.matrix(tensors["o"])

    def state_need(self) -> StateNeed:
        return StateNeed((self.heads * self.vdim * self.dim,), torch.float32)

    def forward(self, h: torch.Tensor, residual32: torch.Tensor, ctx: StepContext, cache: LayerCache) -> None:
        h = as_tensor(h)
        m, dev, ops, nk, nv = h.shape[0], h.device, self.ops, self.nk, self.nv
        p32 = torch.empty((m, 2 * nk + 2 * nv + self.rank), dtype=torch.float32, device=dev)
        ops.linear(h, self.w_in, None, p32, "f32")
        inner = torch.empty((m, self.rank), dtype=self.rt.dtype, device=dev)
        ops.unary(p32[:, 2 * nk + 2 * nv:], inner, "copy")
        z32 = torch.empty((m, nk), dtype=torch.float32, device=dev)
        ops.linear(inner, self.w_a2, self.b_a2, z32, "f32")
        decay = torch.empty((m, nk), dtype=torch.float32, device=dev)
        ops.decay_map(z32, decay, "sigmoid_root", self.tau)
        o32 = torch.empty((m, nv), dtype=torch.float32, device=dev)
        ops.linear_state_scan(p32[:, :nk], p32[:, nk:2 * nk], p32[:, 2 * nk:2 * nk + nv], decay, cache.state, 0, ctx, o32,
                              self.heads, self.heads, self.dim, self.vdim, q_scale=self.dim ** -0.5)
        gated = torch.empty((m, nv), dtype=self.rt.dtype, device=dev)
        ops.gated_norm(o32, gated, groups=self.heads, eps=self.eps, gain32=self.gain, gate32=p32[:, 2 * nk + nv:2 * nk + 2 * nv],
                       gate_kind="silu", out_scale=self.out_scale)
        ops.linear(gated, self.w_o, None, residual32, "add")


class ShiftedTimeMix(Mixer):
    """params: ``hidden heads dim vdim decay_rank eps out_scale``. tensors: ``mu_r mu_k mu_v mu_g mu_w [hidden]``,
    ``r k [heads*dim, hidden]``, ``v g [heads*vdim, hidden]``, ``w1 [decay_rank, hidden]``, ``w2 [heads*dim, decay_rank]``,
    ``w0 [heads*dim]``, ``u [heads, dim]``, ``norm [heads*vdim]``, ``o [hidden, heads*vdim]``."""

    graph_safe = True   # launches do not depend on which requests are in the batch
    STREAMS = ("r", "k", "v", "g", "w")

    @staticmethod
    def spec(prefix: str, hidden: int, heads: int, dim: int, vdim: int, decay_rank: int, eps: float,
             out_scale: float = 1.0) -> PartSpec:
        nk, nv = heads * dim, heads * vdim
        t = {f"mu_{s}": TensorSpec(f"{prefix}.mu.{s}", (hidden,), "mix01") for s in ShiftedTimeMix.STREAMS}
        t.update({"r": TensorSpec(f"{prefix}.r", (nk, hidden)), "k": TensorSpec(f"{prefix}.k", (nk, hidden)),
                  "v": TensorSpec(f"{prefix}.v", (nv, hidden)), "g": TensorSpec(f"{prefix}.g", (nv, hidden)),
                  "w1": TensorSpec(f"{prefix}.w1", (decay_rank, hidden)), "w2": TensorSpec(f"{prefix}.w2", (nk, decay_rank)),
                  "w0": TensorSpec(f"{prefix}.w0", (nk,), "unit"), "u": TensorSpec(f"{prefix}.u", (heads, dim), "unit"),
                  "norm": TensorSpec(f"{prefix}.norm", (nv,), "gain"), "o": TensorSpec(f"{prefix}.o", (hidden, nv))})
        return PartSpec("time_mix", {"hidden": hidden, "heads": heads, "dim": dim, "vdim": vdim, "decay_rank": decay_rank,
                                     "eps": float(eps), "out_scale": float(out_scale)}, t)

    def __init__(self, spec: PartSpec, tensors: Dict[str, torch.Tensor], rt: Runtime):
        super().__init__(spec, tensors, rt)
        p = spec.params
        self.hidden, self.heads, self.dim, self.vdim = int(p["hidden"]), int(p["heads"]), int(p["dim"]), int(p["vdim"])
        self.rank, self.eps, self.out_scale = int(p["decay_rank"]), float(p["eps"]), float(p.get("out_scale", 1.0))
        self.nk, self.nv = self.heads * self.dim, self.heads * self.vdim
        self.mu = rt.vector32(torch.stack([tensors[f"mu_{s}"] for s in self.STREAMS], dim=0))       # [5, hidden]
        self.w = {s: rt.matrix(tensors[s]) for s in ("r", "k", "v", "g", "w1", "w2")}
        self.w0, self.bonus = rt.vector32(tensors["w0"]), rt.vector32(tensors["u"])
        self.gain = rt.vector32(tensors["norm"])
        self.w_o = rt.matrix(tensors["o"])

    def state_need(self) -> StateNeed:
        # [the request's last h | S as [head, value channel, key channel]]
        return StateNeed((self.hidden + self.heads * self.vdim * self.dim,), torch.float32)

    def forward(self, h: torch.Tensor, residual32: torch.Tensor, ctx: StepContext, cache: LayerCache) -> None:
        h = as_tensor(h)
        m, dev, ops, nk, nv = h.shape[0], h.device, self.ops, self.nk, self.nv
        mixes = torch.empty((5, m, self.hidden), dtype=self.rt.dtype, device=dev)
        ops.token_shift(h, self.mu, cache.state, 0, ctx, mixes)
        proj = {}
        for i, s in enumerate(("r", "k", "v", "g")):        # four products: every stream has an input of its own
            proj[s] = torch.empty((m, self.w[s].shape[0]), dtype=torch.float32, device=dev)
            ops.linear(mixes[i], self.w[s], None, proj[s], "f32")
        t32 = torch.empty((m, self.rank), dtype=torch.float32, device=dev)
        ops.linear(mixes[4], self.w["w1"], None, t32, "f32")
        inner = torch.empty((m, self.rank), dtype=self.rt.dtype, device=dev)
        ops.unary(t32, inner, "tanh")
        z32 = torch.empty((m, nk), dtype=torch.float32, device=dev)
        ops.linear(inner, self.w["w2"], self.w0, z32, "f32")
        decay = torch.empty((m, nk), dtype=torch.float32, device=dev)
        ops.decay_map(z32, decay, "exp_neg_exp", 1.0)
        o32 = torch.empty((m, nv), dtype=torch.float32, device=dev)
        ops.linear_state_scan(proj["r"], proj["k"], proj["v"], decay, cache.state, self.hidden, ctx, o32,
                              self.heads, self.heads, self.dim, self.vdim, bonus32=self.bonus)
        gated = torch.empty((m, nv), dtype=self.rt.dtype, device=dev)
        ops.gated_norm(o32, gated, groups=self.heads, eps=self.eps, gain32=self.gain, gate32=proj["g"], gate_kind="silu",
                       out_scale=self.out_scale)
        ops.linear(gated, self.w_o, None, residual32, "add")


class Mamba2Mixer(Mixer):
    """params: ``hidden heads vdim state groups norm_groups conv eps out_scale``. tensors: ``in [2*inner + 2*groups*state +
    heads, hidden]``, ``conv [inner + 2*groups*state, taps]``, ``conv_b``, ``dt_bias A_log D [heads]``, ``norm [inner]``,
    ``o [hidden, inner]`` with ``inner = heads * vdim``."""

    graph_safe = True   # launches do not depend on which requests are in the batch

    @staticmethod
    def spec(prefix: str, hidden: int, heads: int, vdim: int, state: int, groups: int, norm_groups: int, conv: int, eps: float,
             out_scale: float = 1.0) -> PartSpec:
        inner, gn = heads * vdim, groups * state
        t = {"in": TensorSpec(f"{prefix}.in", (2 * inner + 2 * gn + heads, hidden)),
             "conv": TensorSpec(f"{prefix}.conv", (inner + 2 * gn, conv), "unit"),
             "conv_b": TensorSpec(f"{prefix}.conv.b", (inner + 2 * gn,), "bias"),
             "dt_bias": TensorSpec(f"{prefix}.dt_bias", (heads,), "unit"), "A_log": TensorSpec(f"{prefix}.A_log", (heads,), "unit"),
             "D": TensorSpec(f"{prefix}.D", (heads,), "gain"), "norm": TensorSpec(f"{prefix}.norm", (inner,), "gain"),
             "o": TensorSpec(f"{prefix}.o", (hidden, inner))}
        return PartSpec("mamba2", {"hidden": hidden, "heads": heads, "vdim": vdim, "state": state, "groups": groups,
                                   "norm_groups": norm_groups, "conv": conv, "eps": float(eps), "out_scale": float(out_scale)}, t)

    def __init__(self, spec: PartSpec, tensors: Dict[str, torch.Tensor], rt: Runtime):
        super().__init__(spec, tensors, rt)
        p = spec.params
        self.heads, self.vdim, self.n, self.groups = int(p["heads"]), int(p["vdim"]), int(p["state"]), int(p["groups"])
        self.norm_groups, self.taps = int(p["norm_groups"]), int(p["conv"])
        self.eps, self.out_scale = float(p["eps"]), float(p.get("out_scale", 1.0))
        self.inner, self.gn = self.heads * self.vdim, self.groups * self.n
        if self.heads % self.groups or self.inner % self.norm_groups:
            raise ValueError("heads must be a multiple of groups, and heads * vdim of norm_groups")
        self.w_in = rt.matrix(tensors["in"])
        self.conv_w, self.conv_b = rt.vector32(tensors["conv"]), rt.vector32(tensors["conv_b"])
        self.dt_bias, self.a_log, self.skip = rt.vector32(tensors["dt_bias"]), rt.vector32(tensors["A_log"]), rt.vector32(tensors["D"])
        self.gain = rt.vector32(tensors["norm"])
        self.w_o = rt.matrix(tensors["o"])
        self.conv_state = (self.taps - 1) * (self.inner + 2 * self.gn)

    def state_need(self) -> StateNeed:
        # [the convolution's last taps-1 inputs | S as [head, value channel, state channel]]
        return StateNeed((self.conv_state + self.heads * self.vdim * self.n,), torch.float32)

    def forward(self, h: torch.Tensor, residual32: torch.Tensor, ctx: StepContext, cache: LayerCache) -> None:
        h = as_tensor(h)
        m, dev, ops, inner, gn = h.shape[0], h.device, self.ops, self.inner, self.gn
        p32 = torch.empty((m, 2 * inner + 2 * gn + self.heads), dtype=torch.float32, device=dev)
        ops.linear(h, self.w_in, None, p32, "f32")
        xbc_in = p32[:, inner:2 * inner + 2 * gn]
        xbc = torch.empty((m, inner + 2 * gn), dtype=torch.float32, device=dev)
        ops.conv_step(xbc_in, self.conv_w, self.conv_b, "silu", cache.state, 0, ctx, xbc, self.taps)
        dt = torch.empty((m, self.heads), dtype=torch.float32, device=dev)
        decay = torch.empty((m, self.heads), dtype=torch.float32, device=dev)
        ops.step_sizes(p32[:, 2 * inner + 2 * gn:], self.dt_bias, self.a_log, dt, decay)
        o32 = torch.empty((m, inner), dtype=torch.float32, device=dev)
        x = xbc[:, :inner]
        ops.linear_state_scan(xbc[:, inner + gn:], xbc[:, inner:inner + gn], x, decay, cache.state, self.conv_state, ctx, o32,
                              self.heads, self.groups, self.n, self.vdim, v_scale32=dt)
        gated = torch.empty((m, inner), dtype=self.rt.dtype, device=dev)
        ops.gated_norm(o32, gated, groups=self.norm_groups, eps=self.eps, gain32=self.gain, gate32=p32[:, :inner], gate_kind="silu",
                       gate_first=True, skip32=x, skip_coef32=self.skip, out_scale=self.out_scale)
        ops.linear(gated, self.w_o, None, residual32, "add")


register_part("gated_linear_attention", GatedLinearAttention)
register_part("time_mix", ShiftedTimeMix)
register_part("mamba2", Mamba2Mixer)
