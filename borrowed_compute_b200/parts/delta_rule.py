"""The generalized delta rule: a recurrent mixer with one [D, D] float state a head.

With r, k, v = W_r h, W_k h, W_v h (heads x D each), a decay and a removal rate per head
and key channel

    w = exp(-decay_scale * sigmoid(W_w2 tanh(W_w1 h) + w0))        a = sigmoid(W_a h + a_b)

and the unit key u = k / sqrt(sum(k^2) + key_eps) of each head, the state moves as

    S_t = diag(w) S_(t-1) - (a * u) (u^T S_(t-1)) + k v^T          o_t = S_t^T r

(both corrections read the old state).  Each head's o is divided by its root mean square,
the heads are multiplied by a weight and by sigmoid(W_g h), and W_o adds the result into the
residual stream.  The state starts at zero and is carried from token to token for every
sequence, in the cache's per-sequence state.  The six projections of h are one product
that keeps its float accumulators; everything up to the output product is float.
"""

from __future__ import annotations

import math
from typing import Dict, Optional

import torch

from .. import ops
from . import products
from .base import MIXERS, Mixer, RunMemory, Runtime, StateNeed, StepContext, TensorSpec


split_steps = False      # tests: steps of single rows through the three kernels of a prompt step


@MIXERS.register("generalized_delta")
class GeneralizedDelta(Mixer):
    def __init__(self, hidden_size: int, heads: int, head_dim: int, decay_rank: int, norm_eps: float,
                 decay_scale: float = math.exp(-0.5), key_eps: float = 1e-6):
        super().__init__(hidden_size=hidden_size, heads=heads, head_dim=head_dim, decay_rank=decay_rank, norm_eps=norm_eps,
                         decay_scale=decay_scale, key_eps=key_eps)
        if not 0 < int(head_dim) <= 256:
            raise ValueError(f"a head of {head_dim} channels is outside what the recurrence kernel takes (1 to 256)")
        self.hidden_size, self.heads, self.head_dim, self.decay_rank = int(hidden_size), int(heads), int(head_dim), int(decay_rank)
        self.norm_eps, self.decay_scale, self.key_eps = float(norm_eps), float(decay_scale), float(key_eps)

    def tensors(self) -> Dict[str, TensorSpec]:
        e, hd, rank = self.hidden_size, self.heads * self.head_dim, self.decay_rank
        return {
            "r": TensorSpec((hd, e)), "k": TensorSpec((hd, e)), "v": TensorSpec((hd, e)), "g": TensorSpec((hd, e)),
            "a": TensorSpec((hd, e)), "a.b": TensorSpec((hd,), role="vector", init="zeros"),
            "w1": TensorSpec((rank, e)), "w2": TensorSpec((hd, rank), role="vector"), "w0": TensorSpec((hd,), role="vector", init="zeros"),
            "norm": TensorSpec((hd,), role="vector", init="ones"), "o": TensorSpec((e, hd)),
        }

    def state_need(self) -> Optional[StateNeed]:
        return StateNeed((self.heads, self.head_dim, self.head_dim), torch.float32)

    def load(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        super().load(tensors, rt)
        # One product for all that is read from h: r, k, v, the gate, the removal rate, the decay's inner projection.
        self.w_in = torch.cat([tensors[n] for n in ("r", "k", "v", "g", "a", "w1")], dim=0).contiguous()
        self.w_o = tensors["o"].contiguous()
        self.a_bias, self.w0, self.norm_weight = (tensors[n].contiguous() for n in ("a.b", "w0", "norm"))
        self.w2_t = tensors["w2"].t().contiguous()      # [rank, heads * dim]: the threads of a head read neighbouring values

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx: StepContext, mem: RunMemory) -> None:
        if mem.state is None:
            raise RuntimeError("the delta rule was given no state: the cache does not serve this run")
        rows, H, D = x.shape[0], self.heads, self.head_dim
        hd, f32, dev = H * D, torch.float32, x.device
        proj = torch.empty((rows, self.w_in.shape[0]), dtype=f32, device=dev)
        products.linear(x, self.w_in, proj, products.EPI_STORE_F32, "delta projections")
        y = torch.empty((rows, hd), dtype=x.dtype, device=dev)
        if ctx.decode and not split_steps and ops.delta_step_accepts(D):
            # One row a sequence: the three kernels below as one launch (the same bits).
            ops.delta_step(proj, self.w2_t, self.w0, self.a_bias, self.norm_weight, mem.state, ctx.row_slot, y, H, D, self.decay_scale,
                           self.key_eps, self.norm_eps, write_state=mem.writes)
            products.linear(y, self.w_o, residual, products.EPI_ADD_F32, "output product")
            return
        decay, unit, removal = (torch.empty((rows, hd), dtype=f32, device=dev) for _ in range(3))
        dots = torch.empty((rows, H, 2), dtype=f32, device=dev)
        ops.delta_prepare(proj, self.w2_t, self.w0, self.a_bias, decay, unit, removal, dots, H, D, self.decay_scale, self.key_eps)
        o = torch.empty((rows, hd), dtype=f32, device=dev)
        ops.delta_scan(proj, decay, unit, removal, dots, mem.state, ctx.seq_rows, ctx.seq_slot, o, ctx.seqs, H, D, write_state=mem.writes)
        ops.delta_finish(o, proj, 3 * hd, self.norm_weight, y, H, D, self.norm_eps)
        products.linear(y, self.w_o, residual, products.EPI_ADD_F32, "output product")
