"""Two mixers side by side: both read the same input, and their results are added with fixed factors,
``left_scale * left(h) + right_scale * right(h)``.

``params``: ``left`` and ``right`` (``PartSpec`` of any registered mixers; their tensors live under ``left_prefix`` /
``right_prefix`` behind this mixer's own prefix, default ``left.`` / ``right.``), ``left_scale``, ``right_scale``.  At most
one of the two keeps keys and values; the fixed-size states of both are kept side by side under names that start with
``left.`` / ``right.``.  A block arrangement that sums several results into the stream itself takes the two results
unsummed through ``forward_terms``; ``forward`` forms the weighted sum in 32-bit and rounds it once.
"""

from __future__ import annotations

from typing import Dict, List, Mapping, Optional, Tuple

import torch

from ..cache.store import KVNeed, StateNeed
from ..config.spec import PartSpec
from ..ops import kernels as K
from .base import MIXERS, Runtime, StepContext, TensorInfo, register_mixer

_SIDES = ("left", "right")


@register_mixer("side_by_side")
class SideBySide:
    @staticmethod
    def _prefix(params: Mapping, prefix: str, side: str) -> str:
        return prefix + params.get(side + "_prefix", side + ".")

    @staticmethod
    def tensors(params: Mapping, prefix: str) -> Dict[str, TensorInfo]:
        out: Dict[str, TensorInfo] = {}
        for side in _SIDES:
            spec: PartSpec = params[side]
            out.update(MIXERS.get(spec.kind).tensors(spec.params, SideBySide._prefix(params, prefix, side)))
        return out

    def __init__(self, params: Mapping, prefix: str, weights, rt: Runtime):
        self.rt = rt
        self.parts = {}
        for side in _SIDES:
            spec: PartSpec = params[side]
            self.parts[side] = MIXERS.get(spec.kind)(spec.params, self._prefix(params, prefix, side), weights, rt)
        self.scales = {side: float(params.get(side + "_scale", 1.0)) for side in _SIDES}
        needs = [s for s in _SIDES if self.parts[s].kv_need() is not None]
        if len(needs) > 1:
            raise ValueError("side_by_side: one run step has one cache entry; only one of the two mixers may keep keys and values")
        self.kv_side = needs[0] if needs else None
        tiles = [getattr(p, "prefill_tile") for p in self.parts.values() if hasattr(p, "prefill_tile")]
        if tiles:
            self.prefill_tile = min(tiles)
        self.uses_fresh_steps = any(getattr(p, "uses_fresh_steps", False) for p in self.parts.values())
        K.stream_par_lib()

    def kv_need(self) -> Optional[KVNeed]:
        return self.parts[self.kv_side].kv_need() if self.kv_side else None

    def state_need(self):
        need: Dict[str, StateNeed] = {}
        for side, part in self.parts.items():
            st = part.state_need()
            if isinstance(st, StateNeed):
                need[side] = st
            elif st:
                need.update({f"{side}.{name}": v for name, v in st.items()})
        return need or None

    def _state_of(self, side: str, state):
        if state is None:
            return None
        if side in state:
            return state[side]
        sub = {name[len(side) + 1:]: t for name, t in state.items() if name.startswith(side + ".")}
        return sub or None

    def forward_terms(self, h: torch.Tensor, ctx: StepContext, cache, state, owns_cache: bool = True) -> List[Tuple[torch.Tensor, float]]:
        """``[(left(h), left_scale), (right(h), right_scale)]``: the caller forms the sum."""
        def job(side):
            part = self.parts[side]
            return lambda: part.forward(h, ctx, cache if side == self.kv_side else None, self._state_of(side, state), owns_cache)

        jobs = [job(side) for side in _SIDES]
        # few rows: the two mixers run on streams of their own (the first side stream is the enclosing arrangement's)
        ys = self.rt.run_branches(jobs, first_stream=1) if self.rt.branches(h.shape[0]) else [j() for j in jobs]
        return [(y, self.scales[side]) for y, side in zip(ys, _SIDES)]

    def forward(self, h: torch.Tensor, ctx: StepContext, cache, state, owns_cache: bool = True) -> torch.Tensor:
        terms = self.forward_terms(h, ctx, cache, state, owns_cache)
        acc = torch.zeros(terms[0][0].shape, dtype=torch.float32, device=h.device)
        K.stream_sum(acc, terms)
        return acc if h.dtype == torch.float32 else acc.to(h.dtype)
