"""Two mixers side by side: both read the same normed input and add their results to the residual stream, each with
the factor it was given (``out_scale`` of the mixer's own parameters). What the pair keeps per request is the union of
what its halves keep: the pages of the half that caches per position (at most one may), and one flat 32-bit state
whose first part belongs to the left half and the rest to the right one.
"""
from __future__ import annotations

from dataclasses import replace
from typing import Dict, Optional

import torch

from ..registry import get_part, register_part
from .base import CacheNeed, LayerCache, Mixer, Runtime, StateNeed, StepContext, as_tensor
from .spec import PartSpec


class SideBySide(Mixer):
    """params: ``left``, ``right`` (the halves' ``PartSpec``). tensors: the halves' tensors with the roles
    ``left.<role>`` and ``right.<role>``."""

    @staticmethod
    def spec(left: PartSpec, right: PartSpec) -> PartSpec:
        tensors = {f"left.{r}": ts for r, ts in left.tensors.items()}
        tensors.update({f"right.{r}": ts for r, ts in right.tensors.items()})
        return PartSpec("side_by_side", {"left": left, "right": right}, tensors)

    def __init__(self, spec: PartSpec, tensors: Dict[str, torch.Tensor], rt: Runtime):
        super().__init__(spec, tensors, rt)
        self.halves = []
        for side in ("left", "right"):
            sub: PartSpec = spec.params[side]
            mine = {r[len(side) + 1:]: t for r, t in tensors.items() if r.startswith(side + ".")}
            self.halves.append(get_part(sub.kind)(sub, mine, rt))
        needs = [m.cache_need() for m in self.halves]
        if sum(n is not None for n in needs) > 1:
            raise ValueError("at most one half of a pair may cache per position")
        self._offsets = []
        off = 0
        for m in self.halves:
            st = m.state_need()
            if st is not None and (st.dtype != torch.float32 or len(st.shape) != 1):
                raise ValueError("the halves of a pair keep their state as one row of 32-bit floats")
            n = 0 if st is None else int(st.shape[0])
            self._offsets.append((off, n))
            off += n
        self._state_size = off

    @property
    def graph_safe(self) -> bool:
        return all(getattr(m, "graph_safe", False) for m in self.halves)

    def cache_need(self) -> Optional[CacheNeed]:
        for m in self.halves:
            need = m.cache_need()
            if need is not None:
                return need
        return None

    def state_need(self) -> Optional[StateNeed]:
        return StateNeed((self._state_size,), torch.float32) if self._state_size else None

    def bind_positions(self, positions) -> None:
        for m in self.halves:
            m.bind_positions(positions)

    def forward(self, h: torch.Tensor, residual32: torch.Tensor, ctx: StepContext, cache: LayerCache) -> None:
        h = as_tensor(h)
        for m, (off, n) in zip(self.halves, self._offsets):
            state = cache.state[:, off:off + n] if n else None      # rows of the slots, a slice of their columns
            m.forward(h, residual32, ctx, replace(cache, state=state, writes=cache.writes and m.cache_need() is not None))


register_part("side_by_side", SideBySide)
