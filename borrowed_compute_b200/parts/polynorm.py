"""A dense feed-forward with the PolyNorm activation: down( act( up x ) ), added into the
residual stream, with

    act(z) = a N(z) + b N(z^2) + c N(z^3) + e

where powers are taken element by element, N divides a row's vector of values by its root
mean square (eps inside the root), and a, b, c, e are four learned numbers.  The up product
hands its float accumulators to the activation, whose three statistics are float.
"""

from __future__ import annotations

from typing import Dict

import torch

from .. import ops
from . import products
from .base import FEED_FORWARDS, FeedForward, Runtime, StepContext, TensorSpec


@FEED_FORWARDS.register("polynorm_mlp")
class PolyNormMLP(FeedForward):
    def __init__(self, hidden_size: int, intermediate_size: int, eps: float, up: str = "up", down: str = "down", coefficients: str = "act"):
        super().__init__(hidden_size=hidden_size, intermediate_size=intermediate_size, eps=eps, up=up, down=down, coefficients=coefficients)
        self.hidden_size, self.intermediate_size, self.eps = int(hidden_size), int(intermediate_size), float(eps)
        self.names = (str(up), str(down), str(coefficients))

    def tensors(self) -> Dict[str, TensorSpec]:
        e, f = self.hidden_size, self.intermediate_size
        up, down, coef = self.names
        return {up: TensorSpec((f, e)), down: TensorSpec((e, f)), coef: TensorSpec((4,), role="vector", init="ones")}

    def load(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        super().load(tensors, rt)
        up, down, coef = self.names
        self.w_up, self.w_down, self.coef = tensors[up].contiguous(), tensors[down].contiguous(), tensors[coef].contiguous()

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx: StepContext) -> None:
        z = torch.empty((x.shape[0], self.intermediate_size), dtype=torch.float32, device=x.device)
        products.linear(x, self.w_up, z, products.EPI_STORE_F32, "up product")
        y = torch.empty((x.shape[0], self.intermediate_size), dtype=x.dtype, device=x.device)
        ops.polynorm(z, self.coef, y, self.eps)
        products.linear(y, self.w_down, residual, products.EPI_ADD_F32, "down product")
