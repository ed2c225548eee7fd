"""Block arrangements.

The pre-norm residual block: x += mixer(norm1(x)); x += feed_forward(norm2(x))
(crates/bc-infer/src/model.rs:323-345).

The parallel block: x += mixer(conv(norm1(x))) + feed_forward(norm2(x)), both branches reading
the same x, the mixer's input first passing a short causal convolution over time whose last
inputs are per-sequence state.  The feed-forward (and its norm) may be left out."""

from __future__ import annotations

import torch

from typing import Dict, Mapping

from .base import BLOCKS, CONVOLUTIONS, FEED_FORWARDS, MIXERS, NORMS, Block, RunMemory, Runtime, StateNeed, StepContext


@BLOCKS.register("prenorm")
class PreNormBlock(Block):
    ROLES = {"norm1": NORMS, "mixer": MIXERS, "norm2": NORMS, "feed_forward": FEED_FORWARDS}

    def forward(self, residual: torch.Tensor, ctx: StepContext, mem: RunMemory, rt: Runtime) -> None:
        h = torch.empty((residual.shape[0], self.hidden_size), dtype=rt.dtype, device=residual.device)
        self.norm1.forward(residual, h)
        self.mixer.forward(h, residual, ctx, mem)
        self.norm2.forward(residual, h)
        self.feed_forward.forward(h, residual, ctx)


@BLOCKS.register("parallel")
class ParallelBlock(Block):
    ROLES = {"norm1": NORMS, "conv": CONVOLUTIONS, "mixer": MIXERS, "norm2": NORMS, "feed_forward": FEED_FORWARDS}
    OPTIONAL = ("conv", "norm2", "feed_forward")

    def __init__(self, parts, hidden_size: int):
        super().__init__(parts, hidden_size)
        if (self.norm2 is None) != (self.feed_forward is None):
            raise ValueError("a parallel block has a feed-forward and its norm, or neither")

    def state_needs(self) -> Dict[str, StateNeed]:
        need = None if self.conv is None else self.conv.state_need()
        return {} if need is None else {"conv": need}

    def forward(self, residual: torch.Tensor, ctx: StepContext, mem: RunMemory, rt: Runtime) -> None:
        rows = residual.shape[0]
        # Both branches read the stream as it is now, so both norms run before either adds to it.
        h = torch.empty((rows, self.hidden_size), dtype=rt.dtype, device=residual.device)
        self.norm1.forward(residual, h)
        if self.feed_forward is not None:
            h2 = torch.empty((rows, self.hidden_size), dtype=rt.dtype, device=residual.device)
            self.norm2.forward(residual, h2)
        if self.conv is not None:
            hc = torch.empty_like(h)
            self.conv.forward(h, hc, ctx, mem.states.get("conv"), mem.writes)
            h = hc
        self.mixer.forward(h, residual, ctx, mem)
        if self.feed_forward is not None:
            self.feed_forward.forward(h2, residual, ctx)
