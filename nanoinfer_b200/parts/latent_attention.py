"""Attention whose keys and values come out of a cached low-rank latent.

Per token the cache holds ONE row for all heads: the latent ``c = rmsnorm(W_dkv h)[:rank]`` and a rotated key part
``kr`` of ``rot`` elements (the last rows of ``W_dkv h``, not normed, rotated by the token's position) that every
head shares. Queries go through a latent too: ``q = W_uq rmsnorm(W_dq h)``, laid out head by head as
``[plain | rotated]``. Head ``n``: key ``[W_uk,n c | kr]``, value ``W_uv,n c``, score
``(q_plain . W_uk,n c + q_rot . kr) * scale`` over the positions the window lets it see, softmax in 32-bit, then
``W_o`` over the concatenated heads, added to the residual stream.

The kernels never expand keys or values per cached position: the query is carried into the latent space
(``W_uk,n^T q_plain``), scored against the cached rows as they are, and ``W_uv,n`` is applied to the weighted sum of
latents. A layer may read the rows that an earlier layer cached (its schedule entry names that entry) and has then no
down projection for keys and values of its own.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..registry import register_part
from .base import CacheNeed, LayerCache, Mixer, PagedTensor, PositionEncoding, Runtime, StepContext
from .spec import PartSpec, TensorSpec


class LatentAttention(Mixer):
    """params: ``hidden``, ``heads``, ``dim`` (plain query/key width of a head), ``rot_dim`` (rotated width),
    ``vdim`` (value width), ``q_rank``, ``kv_rank``, ``scale``, ``window`` (0 = all keys), ``keep`` (how many of the
    last positions the cache has to keep: the largest window of the layers that read it; 0 = all), ``eps``,
    ``position`` (name of a shared ``frequency_rotary`` encoding), ``owns_kv`` (False: the rows of another entry).
    tensors: ``dq dq_norm uq uk uv o`` and, with ``owns_kv``, ``dkv dkv_norm``."""

    graph_safe = True   # launches do not depend on which requests are in the batch

    @staticmethod
    def spec(prefix: str, hidden: int, heads: int, dim: int, rot_dim: int, vdim: int, q_rank: int, kv_rank: int,
             scale: float, window: int, keep: int, eps: float, position: str, owns_kv: bool = True) -> PartSpec:
        t = {
            "dq": TensorSpec(f"{prefix}.dq", (q_rank, hidden)),
            "dq_norm": TensorSpec(f"{prefix}.dq.norm", (q_rank,), "gain"),
            "uq": TensorSpec(f"{prefix}.uq", (heads * (dim + rot_dim), q_rank)),
            "uk": TensorSpec(f"{prefix}.uk", (heads * dim, kv_rank)),
            "uv": TensorSpec(f"{prefix}.uv", (heads * vdim, kv_rank)),
            "o": TensorSpec(f"{prefix}.o", (hidden, heads * vdim)),
        }
        if owns_kv:
            t["dkv"] = TensorSpec(f"{prefix}.dkv", (kv_rank + rot_dim, hidden))
            t["dkv_norm"] = TensorSpec(f"{prefix}.dkv.norm", (kv_rank,), "gain")
        return PartSpec("latent_attention", {
            "hidden": hidden, "heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank,
            "kv_rank": kv_rank, "scale": scale, "window": window, "keep": keep, "eps": eps, "position": position,
            "owns_kv": owns_kv}, t)

    def __init__(self, spec: PartSpec, tensors: Dict[str, torch.Tensor], rt: Runtime):
        super().__init__(spec, tensors, rt)
        p = spec.params
        self.hidden, self.heads = int(p["hidden"]), int(p["heads"])
        self.dim, self.rot_dim, self.vdim = int(p["dim"]), int(p["rot_dim"]), int(p["vdim"])
        self.q_rank, self.kv_rank = int(p["q_rank"]), int(p["kv_rank"])
        self.scale, self.eps = float(p["scale"]), float(p["eps"])
        self.window, self.keep = int(p.get("window", 0)), int(p.get("keep", 0))
        if self.keep and (not self.window or self.window > self.keep):
            raise ValueError("the cache keeps fewer positions than the window reads")
        self.owns_kv = bool(p.get("owns_kv", True))
        self.position_name = str(p["position"])
        self.w_dq, self.g_dq = rt.matrix(tensors["dq"]), rt.vector32(tensors["dq_norm"])
        self.w_uq, self.w_uk, self.w_uv = rt.matrix(tensors["uq"]), rt.matrix(tensors["uk"]), rt.matrix(tensors["uv"])
        self.w_o = rt.matrix(tensors["o"])
        self.w_dkv = self.g_dkv = None
        if self.owns_kv:
            self.w_dkv, self.g_dkv = rt.matrix(tensors["dkv"]), rt.vector32(tensors["dkv_norm"])
        self._freq = None

    def cache_need(self) -> CacheNeed:
        return CacheNeed((PagedTensor("latent", 1, self.kv_rank + self.rot_dim),), self.keep)

    def bind_positions(self, positions: Dict[str, PositionEncoding]) -> None:
        freq = getattr(positions[self.position_name], "frequencies", None)
        if freq is None:
            raise ValueError("latent attention binds to a position encoding that gives frequencies")
        self._freq = freq()
        if self._freq[2] != self.rot_dim:
            raise ValueError(f"the position encoding rotates {self._freq[2]} elements, the mixer {self.rot_dim}")

    def forward(self, h: torch.Tensor, residual32: torch.Tensor, ctx: StepContext, cache: LayerCache) -> None:
        m, dev, ops = h.shape[0], h.device, self.ops
        freq, mag, _ = self._freq
        pages = cache.pages["latent"]
        if cache.writes:
            z32 = torch.empty((m, self.kv_rank + self.rot_dim), dtype=torch.float32, device=dev)
            ops.linear(h, self.w_dkv, None, z32, "f32")
            ops.latent_store(z32, self.g_dkv, self.eps, freq, mag, ctx, cache.block_table, cache.page_size, pages,
                             self.kv_rank, self.rot_dim)
        cq32 = torch.empty((m, self.q_rank), dtype=torch.float32, device=dev)
        ops.linear(h, self.w_dq, None, cq32, "f32")
        cq = torch.empty((m, self.q_rank), dtype=self.rt.dtype, device=dev)
        ops.rmsnorm(cq32, self.g_dq, self.eps, cq)
        q32 = torch.empty((m, self.heads * (self.dim + self.rot_dim)), dtype=torch.float32, device=dev)
        ops.linear(cq, self.w_uq, None, q32, "f32")
        q_width, q_dtype = ops.latent_query_layout(pages.dtype, self.kv_rank, self.rot_dim)     # what the attention kernel reads
        qa = torch.empty((m, self.heads * q_width), dtype=q_dtype, device=dev)
        ops.latent_query(q32, self.w_uk, freq, mag, ctx.positions, qa, self.heads, self.dim, self.kv_rank, self.rot_dim)
        lat32 = torch.empty((m, self.heads * self.kv_rank), dtype=torch.float32, device=dev)
        ops.latent_attention(qa, lat32, ctx, cache.block_table, cache.page_size, pages, self.heads, self.kv_rank,
                             self.rot_dim, self.scale, self.window)
        attn = torch.empty((m, self.heads * self.vdim), dtype=self.rt.dtype, device=dev)
        ops.latent_value(lat32, self.w_uv, attn, self.heads, self.vdim, self.kv_rank)
        ops.linear(attn, self.w_o, None, residual32, "add")


register_part("latent_attention", LatentAttention)
