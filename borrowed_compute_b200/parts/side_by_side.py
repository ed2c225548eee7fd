"""Two mixers side by side: both read the same input and both add into the residual stream, each with a
factor of its own (which it applies itself, ahead of its output product, through its ``out_scale``).

The pair is a mixer like any other.  At most one of the two may ask for token-indexed pages (the cache gives
a run one set of planes); each one's per-sequence state, and whatever further state it asks for, is passed
on under its side's name ("left", "right").
"""

from __future__ import annotations

from typing import Any, Dict, Mapping, Optional

import torch

from .base import MIXERS, CacheNeed, Mixer, RunMemory, Runtime, StateNeed, StepContext, TensorSpec

SIDES = ("left", "right")


@MIXERS.register("side_by_side")
class SideBySide(Mixer):
    def __init__(self, left: Mapping[str, Any], right: Mapping[str, Any]):
        """``left`` and ``right``: {"kind": a mixer's name, ...its parameters}; their tensors carry "left." and "right."."""
        super().__init__(left=left, right=right)
        self.sides: Dict[str, Mixer] = {}
        for side, spec in zip(SIDES, (left, right)):
            params = dict(spec)
            self.sides[side] = MIXERS.get(params.pop("kind"))(**params)
        if all(m.cache_need() is not None for m in self.sides.values()):
            raise ValueError("only one of two mixers side by side may keep token-indexed pages")
        self.graph_safe = all(m.graph_safe for m in self.sides.values())

    def tensors(self) -> Dict[str, TensorSpec]:
        return {f"{side}.{name}": spec for side, m in self.sides.items() for name, spec in m.tensors().items()}

    def load(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        super().load(tensors, rt)
        for side, m in self.sides.items():
            m.load({name[len(side) + 1:]: t for name, t in tensors.items() if name.startswith(side + ".")}, rt)

    def cache_need(self) -> Optional[CacheNeed]:
        return next((need for need in (m.cache_need() for m in self.sides.values()) if need is not None), None)

    def more_state_needs(self) -> Dict[str, StateNeed]:
        out: Dict[str, StateNeed] = {}
        for side, m in self.sides.items():
            if m.state_need() is not None:
                out[side] = m.state_need()
            out.update({f"{side}.{name}": need for name, need in m.more_state_needs().items()})
        return out

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx: StepContext, mem: RunMemory) -> None:
        for side, m in self.sides.items():
            pages = m.cache_need() is not None
            mine = RunMemory(planes=mem.planes if pages else (), page_table=mem.page_table if pages else None,
                             state=mem.states.get("mixer." + side), writes=mem.writes,
                             states={"mixer." + name[len(side) + 7:]: t for name, t in mem.states.items() if name.startswith(f"mixer.{side}.")})
            m.forward(x, residual, ctx, mine)
