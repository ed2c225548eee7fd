"""Recurrent mixers whose float state takes an outer product a token and decays channel by channel:

    S_t = diag(a_t) S_(t-1) + (c_t k_t) v_t^T          o_t = f S_t^T q_t + d v_t

per head, S being [key channels, value channels], zero at a sequence's start and carried from token to
token in the cache's per-sequence state.  Two mixers are this recurrence (``csrc/linear_scan.cu`` runs it,
the same kernel for prompts and single rows, so that both give the same bits):

``gated_linear_attention``: q, k (heads x dim) and v (heads x vdim) from h; a decay per key channel
a = sigmoid(z)^(1/tau) with z = W_a2 (W_a1 h) + b; c = 1, d = 0, f = dim^(-1/2).  Each head's o over its root
mean square times a weight of vdim values shared by the heads, times silu(W_g h), then W_o.

``state_space_dual`` (Mamba-2): W_in h = [z | x | B | C | dt]; x, B, C pass a short causal convolution
with bias and silu whose last inputs are per-sequence state too; dt = softplus(dt + dt_bias), a = exp(-exp(A_log) dt)
one number a head, c = dt, k = B and q = C of the head's group, v = x, d = D.  The heads' outputs times silu(z), then
an RMS norm in ``norm_groups`` equal parts times a weight, then W_o.

The projections keep their float accumulators; decays, step sizes, gates, norms and the state are float on both
paths.  ``out_scale`` multiplies the mixer's result (a mixer that runs beside another).
"""

from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import ops
from . import products
from .base import MIXERS, Mixer, RunMemory, Runtime, StateNeed, StepContext, TensorSpec


@MIXERS.register("gated_linear_attention")
class GatedLinearAttention(Mixer):
    def __init__(self, hidden_size: int, heads: int, head_dim: int, value_dim: int, decay_rank: int, tau: float, norm_eps: float,
                 out_scale: float = 1.0):
        super().__init__(hidden_size=hidden_size, heads=heads, head_dim=head_dim, value_dim=value_dim, decay_rank=decay_rank, tau=tau,
                         norm_eps=norm_eps, out_scale=out_scale)
        if not 0 < int(head_dim) <= 256:
            raise ValueError(f"a head of {head_dim} key channels is outside what the recurrence kernel takes (1 to 256)")
        self.hidden_size, self.heads, self.head_dim, self.value_dim = int(hidden_size), int(heads), int(head_dim), int(value_dim)
        self.decay_rank, self.tau, self.norm_eps, self.out_scale = int(decay_rank), float(tau), float(norm_eps), float(out_scale)
        if self.tau <= 0.0:
            raise ValueError(f"tau must be positive, got {tau}")

    def tensors(self) -> Dict[str, TensorSpec]:
        e, hd, hp, rank = self.hidden_size, self.heads * self.head_dim, self.heads * self.value_dim, self.decay_rank
        return {
            "q": TensorSpec((hd, e)), "k": TensorSpec((hd, e)), "v": TensorSpec((hp, e)), "g": TensorSpec((hp, e)),
            "a1": TensorSpec((rank, e)), "a2": TensorSpec((hd, rank), role="vector"), "a2.b": TensorSpec((hd,), role="vector", init="zeros"),
            "norm": TensorSpec((self.value_dim,), role="vector", init="ones"), "o": TensorSpec((e, hp)),
        }

    def state_need(self) -> Optional[StateNeed]:
        return StateNeed((self.heads, self.value_dim, self.head_dim), torch.float32)      # value channel by value channel

    def load(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        super().load(tensors, rt)
        # One product for all that is read from h: q, k, v, the gate, the decay's inner projection.
        self.w_in = torch.cat([tensors[n] for n in ("q", "k", "v", "g", "a1")], dim=0).contiguous()
        self.w_o = tensors["o"].contiguous()
        self.a2_t = tensors["a2"].t().contiguous()          # [rank, heads * dim]: neighbouring threads read neighbouring values
        self.a2_b, self.norm_weight = tensors["a2.b"].contiguous(), tensors["norm"].contiguous()

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx: StepContext, mem: RunMemory) -> None:
        if mem.state is None:
            raise RuntimeError("gated linear attention was given no state: the cache does not serve this run")
        rows, H, D, P = x.shape[0], self.heads, self.head_dim, self.value_dim
        hd, hp, dev = H * D, H * P, x.device
        proj = torch.empty((rows, self.w_in.shape[0]), dtype=torch.float32, device=dev)
        products.linear(x, self.w_in, proj, products.EPI_STORE_F32, "recurrence projections")
        decay = torch.empty((rows, hd), dtype=torch.float32, device=dev)
        ops.gla_decay(proj, 2 * hd + 2 * hp, self.a2_t, self.a2_b, decay, self.tau)
        # The recurrence writes the rows of live sequences only; the norm after it skips the others (rows of no sequence).
        o = torch.empty((rows, hp), dtype=torch.float32, device=dev)
        ops.linear_scan(proj, 0, 1, proj, hd, 1, proj, 2 * hd, decay, 0, True, None, 0, None, float(D) ** -0.5, mem.state, ctx.seq_rows,
                        ctx.seq_slot, o, ctx.seqs, H, D, P, write_state=mem.writes)
        y = torch.empty((rows, hp), dtype=x.dtype, device=dev)
        ops.gated_norm(o, proj, 2 * hd + hp, self.norm_weight, y, H, self.norm_eps, gate_first=False, factor=self.out_scale, row_slot=ctx.row_slot)
        products.linear(y, self.w_o, residual, products.EPI_ADD_F32, "output product")


@MIXERS.register("state_space_dual")
class StateSpaceDual(Mixer):
    def __init__(self, hidden_size: int, heads: int, value_dim: int, state_dim: int, groups: int, norm_groups: int, taps: int, norm_eps: float,
                 out_scale: float = 1.0):
        super().__init__(hidden_size=hidden_size, heads=heads, value_dim=value_dim, state_dim=state_dim, groups=groups, norm_groups=norm_groups,
                         taps=taps, norm_eps=norm_eps, out_scale=out_scale)
        self.hidden_size, self.heads, self.value_dim, self.state_dim = int(hidden_size), int(heads), int(value_dim), int(state_dim)
        self.groups, self.norm_groups, self.taps = int(groups), int(norm_groups), int(taps)
        self.norm_eps, self.out_scale = float(norm_eps), float(out_scale)
        if self.heads % self.groups:
            raise ValueError(f"{heads} heads are not a multiple of {groups} groups")
        if (self.heads * self.value_dim) % self.norm_groups:
            raise ValueError(f"an inner width of {heads * value_dim} does not split into {norm_groups} equal parts")
        if not 0 < self.state_dim <= 256:
            raise ValueError(f"a state of {state_dim} channels is outside what the recurrence kernel takes (1 to 256)")
        if not 1 <= self.taps <= ops.SSD_MAX_TAPS:
            raise ValueError(f"a convolution of {taps} taps is outside what the kernel takes (1 to {ops.SSD_MAX_TAPS})")
        self.inner = self.heads * self.value_dim
        self.channels = self.inner + 2 * self.groups * self.state_dim

    def tensors(self) -> Dict[str, TensorSpec]:
        e, h = self.hidden_size, self.heads
        return {
            "in": TensorSpec((2 * self.inner + 2 * self.groups * self.state_dim + h, e)),
            "conv": TensorSpec((self.channels, self.taps), role="vector"), "conv.b": TensorSpec((self.channels,), role="vector", init="zeros"),
            "dt_bias": TensorSpec((h,), role="vector", init="zeros"), "A_log": TensorSpec((h,), role="vector", init="zeros"),
            "D": TensorSpec((h,), role="vector", init="ones"), "norm": TensorSpec((self.inner,), role="vector", init="ones"),
            "o": TensorSpec((e, self.inner)),
        }

    def state_need(self) -> Optional[StateNeed]:
        return StateNeed((self.heads, self.value_dim, self.state_dim), torch.float32)     # value channel by value channel

    def more_state_needs(self) -> Dict[str, StateNeed]:
        # The convolution's last inputs; one row more than needed when taps is 1, so that the tensor is never empty.
        return {"conv": StateNeed((max(self.taps - 1, 1), self.channels), torch.float32)}

    def load(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        super().load(tensors, rt)
        self.w_in, self.w_o = tensors["in"].contiguous(), tensors["o"].contiguous()
        self.conv_t = tensors["conv"].t().contiguous()        # [taps, channels]
        self.conv_b, self.dt_bias, self.a_log, self.skip, self.norm_weight = (tensors[n].contiguous() for n in ("conv.b", "dt_bias", "A_log", "D", "norm"))

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx: StepContext, mem: RunMemory) -> None:
        tail = mem.states.get("mixer.conv")
        if mem.state is None or tail is None:
            raise RuntimeError("the state-space mixer was given no state: the cache does not serve this run")
        rows, H, P, N, G = x.shape[0], self.heads, self.value_dim, self.state_dim, self.groups
        inner, C, dev = self.inner, self.channels, x.device
        proj = torch.empty((rows, self.w_in.shape[0]), dtype=torch.float32, device=dev)
        products.linear(x, self.w_in, proj, products.EPI_STORE_F32, "recurrence projections")
        # Set-up and recurrence walk sequences: rows of no sequence are neither written nor read, and the norm at the end skips them.
        xbc = torch.empty((rows, C), dtype=torch.float32, device=dev)
        dtda = torch.empty((rows, 2 * H), dtype=torch.float32, device=dev)
        ops.ssd_prepare(proj, inner, inner + C, self.conv_t, self.conv_b, self.dt_bias, self.a_log, tail, ctx.seq_rows, ctx.seq_slot, xbc, dtda,
                        ctx.seqs, ctx.max_new, write_tail=mem.writes)
        o = torch.empty((rows, inner), dtype=torch.float32, device=dev)
        ops.linear_scan(xbc, inner + G * N, H // G, xbc, inner, H // G, xbc, 0, dtda, H, False, dtda, 0, self.skip, 1.0, mem.state, ctx.seq_rows,
                        ctx.seq_slot, o, ctx.seqs, H, N, P, write_state=mem.writes)
        y = torch.empty((rows, inner), dtype=x.dtype, device=dev)
        ops.gated_norm(o, proj, 0, self.norm_weight, y, self.norm_groups, self.norm_eps, gate_first=True, factor=self.out_scale, row_slot=ctx.row_slot)
        products.linear(y, self.w_o, residual, products.EPI_ADD_F32, "output product")
