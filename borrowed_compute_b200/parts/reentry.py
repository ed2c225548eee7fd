"""Where a stretch of layers that runs several times is entered: before each pass the stream is mixed with
the embedding's output, x <- W [x; x0] + step[number of the pass], W being [width, 2 width] with the stream's
columns first.  The concatenation takes the activation type for the product; the stream stays float."""

from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import ops
from . import products
from .base import JUNCTIONS, Junction, Runtime, StepContext, TensorSpec


@JUNCTIONS.register("mix_with_embedding")
class MixWithEmbedding(Junction):
    needs_embedding = True

    def __init__(self, hidden_size: int, passes: int, matrix: str = "in", steps: str = "step"):
        super().__init__(hidden_size=hidden_size, passes=passes, matrix=matrix, steps=steps)
        self.hidden_size, self.passes, self.names = int(hidden_size), int(passes), (str(matrix), str(steps))

    def tensors(self) -> Dict[str, TensorSpec]:
        e = self.hidden_size
        return {self.names[0]: TensorSpec((e, 2 * e)), self.names[1]: TensorSpec((self.passes, e), role="vector", init="zeros")}

    def load(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        super().load(tensors, rt)
        self.weight, self.steps = tensors[self.names[0]].contiguous(), tensors[self.names[1]].contiguous()

    def forward(self, residual: torch.Tensor, embedded: Optional[torch.Tensor], ctx: StepContext, number: int) -> None:
        if embedded is None:
            raise RuntimeError("the junction was given no embedding output")
        if not 0 <= number < self.passes:
            raise ValueError(f"pass {number} of {self.passes}")
        cat = torch.empty((residual.shape[0], 2 * self.hidden_size), dtype=self.rt.dtype, device=residual.device)
        ops.reentry(residual, embedded, self.steps[number], cat)        # the stream now holds the pass's vector
        products.linear(cat, self.weight, residual, products.EPI_ADD_F32, "re-entry product")
