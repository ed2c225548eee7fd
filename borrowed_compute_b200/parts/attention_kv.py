"""Grouped-query attention whose keys and values have widths of their own, with the
variations a configuration may ask for as parameters:

- biases on the q, k and v projections;
- an RMS norm of q and of k before rotation, each with a plain weight: over the whole
  projection (``qk_norm="whole"``: all heads at once, before they are split into heads) or
  over every head by itself with one weight of ``head_dim`` values that the heads share
  (``qk_norm="head"``);
- rotary positions on the first ``rotary_dims`` dimensions of each head only (dimension i
  paired with i + rotary_dims / 2, or 2i with 2i + 1 if the position encoding pairs
  neighbours; the rest pass unchanged);
- a score scale given by the configuration;
- a sliding ``window`` and/or a ``chunk`` mask: position i sees j <= i only if both lie in
  the same chunk of ``chunk`` positions, counted from the sequence's position 0;
- a ``sink``: one added to the softmax's denominator, as if every row also saw a position
  of score 0 that has no value, so that a row's weights may add up to less than one;
- ``out_scale``, a factor on the mixer's result (a mixer that runs beside another).

The fused projection keeps its float accumulators; biases, norm statistics and the rotation
are float; q, the cached k and v and the attention's output take the activation type.  The
cache lets go of whole chunks behind the newest one.
"""

from __future__ import annotations

from typing import Any, Dict, Mapping, Optional

import torch

from .. import ops
from . import products
from .base import MIXERS, POSITION_ENCODINGS, CacheNeed, Mixer, RunMemory, Runtime, StepContext, TensorSpec


force_rows = False      # tests: take the one-warp-a-row kernel (the checked twin) for bfloat16 too
force_tiles = False     # tests: keep prompts off the tcgen05 kernel (the mma.sync tiles serve every width)


@MIXERS.register("gqa_attention_kv")
class GroupedQueryAttentionKV(Mixer):
    def __init__(self, hidden_size: int, heads: int, kv_heads: int, head_dim: int, value_dim: int, position: Mapping[str, Any],
                 scale: Optional[float] = None, window: int = 0, chunk: int = 0, bias: bool = False, qk_norm_eps: Optional[float] = None,
                 qk_norm: str = "whole", sink: bool = False, out_scale: float = 1.0):
        super().__init__(hidden_size=hidden_size, heads=heads, kv_heads=kv_heads, head_dim=head_dim, value_dim=value_dim, position=position,
                         scale=scale, window=window, chunk=chunk, bias=bias, qk_norm_eps=qk_norm_eps, qk_norm=qk_norm, sink=sink,
                         out_scale=out_scale)
        if qk_norm not in ("whole", "head"):
            raise ValueError(f"qk_norm {qk_norm!r} is neither 'whole' nor 'head'")
        if qk_norm == "head" and bias:
            raise ValueError("the norm of single heads takes no biases")
        self.per_head, self.sink, self.out_scale = qk_norm == "head", bool(sink), float(out_scale)
        if heads % kv_heads:
            raise ValueError(f"{heads} heads are not a multiple of {kv_heads} kv heads")
        if not 0 < head_dim <= 256 or not 0 < value_dim <= 256:
            raise ValueError(f"head size {head_dim} or value size {value_dim} is refused by the attention kernels (1 to 256)")
        self.hidden_size, self.heads, self.kv_heads = int(hidden_size), int(heads), int(kv_heads)
        self.head_dim, self.value_dim = int(head_dim), int(value_dim)
        self.window, self.chunk, self.bias = int(window), int(chunk), bool(bias)
        self.scale = float(scale) if scale is not None else 1.0 / float(head_dim) ** 0.5
        self.qk_norm_eps = None if qk_norm_eps is None else float(qk_norm_eps)
        pos = dict(position)
        self.position = POSITION_ENCODINGS.get(pos.pop("kind"))(**pos)
        self.rotary_dims = int(getattr(self.position, "head_dim", 0))
        if self.rotary_dims > self.head_dim:
            raise ValueError(f"{self.rotary_dims} rotated dimensions do not fit a head of {self.head_dim}")

    def tensors(self) -> Dict[str, TensorSpec]:
        q, kv, v, e = self.heads * self.head_dim, self.kv_heads * self.head_dim, self.kv_heads * self.value_dim, self.hidden_size
        out = {"q": TensorSpec((q, e)), "k": TensorSpec((kv, e)), "v": TensorSpec((v, e)), "o": TensorSpec((e, self.heads * self.value_dim))}
        if self.bias:
            out.update({"q.b": TensorSpec((q,), role="vector", init="zeros"), "k.b": TensorSpec((kv,), role="vector", init="zeros"),
                        "v.b": TensorSpec((v,), role="vector", init="zeros")})
        if self.qk_norm_eps is not None:
            nq, nk = (self.head_dim, self.head_dim) if self.per_head else (q, kv)
            out.update({"q.norm": TensorSpec((nq,), role="vector", init="ones"), "k.norm": TensorSpec((nk,), role="vector", init="ones")})
        return out

    def cache_need(self) -> Optional[CacheNeed]:
        return CacheNeed.keys_values(self.kv_heads, self.head_dim, self.window, value_dim=self.value_dim, chunk=self.chunk)

    def load(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        super().load(tensors, rt)
        self.w_qkv = torch.cat([tensors["q"], tensors["k"], tensors["v"]], dim=0).contiguous()
        self.w_o = tensors["o"].contiguous()
        self.b_qkv = torch.cat([tensors["q.b"], tensors["k.b"], tensors["v.b"]]).contiguous() if self.bias else None
        self.q_norm = tensors["q.norm"].contiguous() if self.qk_norm_eps is not None else None
        self.k_norm = tensors["k.norm"].contiguous() if self.qk_norm_eps is not None else None
        self.position.load({}, rt)

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx: StepContext, mem: RunMemory) -> None:
        rows = x.shape[0]
        H, G, D, DV = self.heads, self.kv_heads, self.head_dim, self.value_dim
        qkv = torch.empty((rows, self.w_qkv.shape[0]), dtype=torch.float32, device=x.device)
        products.linear(x, self.w_qkv, qkv, products.EPI_STORE_F32, "qkv product")
        table = self.position.rotary()
        q = torch.empty((rows, H * D), dtype=x.dtype, device=x.device)
        if self.per_head or (table is not None and table.pairing == 1):
            if self.bias or (self.qk_norm_eps is not None and not self.per_head):
                raise RuntimeError("rotation of neighbouring dimensions comes with the norm of single heads (or none) and no biases")
            ops.qkv_prepare_heads(qkv, self.q_norm, self.k_norm, None if table is None else table.cos_sin, ctx.row_pos, ctx.row_slot,
                                  mem.page_table, q, mem.k_pages, mem.v_pages, H, G, D, DV, self.rotary_dims if table is not None else 0,
                                  0 if table is None else table.pairing, self.qk_norm_eps or 0.0, write_cache=mem.writes)
        else:
            ops.qkv_prepare(qkv, self.b_qkv, self.q_norm, self.k_norm, None if table is None else table.cos_sin, ctx.row_pos, ctx.row_slot,
                            mem.page_table, q, mem.k_pages, mem.v_pages, H, G, D, DV, self.rotary_dims if table is not None else 0,
                            self.qk_norm_eps or 0.0, write_cache=mem.writes)
        att = torch.empty((rows, H * DV), dtype=x.dtype, device=x.device)
        self.attend(q, att, ctx, mem)
        products.linear(att, self.w_o, residual, products.EPI_ADD_F32, "output product")

    def attend(self, q: torch.Tensor, out: torch.Tensor, ctx: StepContext, mem: RunMemory) -> None:
        H, G, D, DV = self.heads, self.kv_heads, self.head_dim, self.value_dim
        if not force_rows and not force_tiles and not ctx.decode and q.dtype == torch.bfloat16 \
                and ops.attention_prefill_tc_accepts(H, G, D, q, H * D, DV):
            # Prompts with heads of 64 or 128 and values no wider: tcgen05 tiles, scores and output in tensor memory.
            ops.attention_prefill(q, H * D, mem.k_pages, mem.v_pages, mem.page_table, ctx.seq_rows, ctx.seq_slot, ctx.seq_start, out,
                                  ctx.seqs, ctx.max_new, H, G, D, window=self.window, scale=self.scale, use_tc=True, chunk=self.chunk,
                                  value_dim=DV, sink=self.sink, out_scale=self.out_scale)
            return
        if not force_rows and not force_tiles and ctx.decode and D == DV and self.chunk == 0 and ops.attention_decode_accepts(H, G, D, q.dtype):
            # Single rows over keys and values of one width, no chunk mask: the kernel that splits a row's positions over blocks.
            ops.attention_decode(q, H * D, mem.k_pages, mem.v_pages, mem.page_table, ctx.row_pos, ctx.row_slot, out, H, G, D, window=self.window,
                                 scale=self.scale, reach=ctx.max_total, sink=self.sink, out_scale=self.out_scale)
            return
        if not force_rows and ops.attention_tiles_accepts(H, G, D, DV, q.dtype):
            # Tensor-core tiles, for prompts and for single rows alike: the heads of a kv head share every page read.
            ops.attention_tiles(q, H * D, mem.k_pages, mem.v_pages, mem.page_table, ctx.seq_rows, ctx.seq_slot, ctx.seq_start, out,
                                ctx.seqs, ctx.max_new, H, G, D, DV, window=self.window, chunk=self.chunk, scale=self.scale, sink=self.sink,
                                out_scale=self.out_scale)
            return
        ops.attention_rows(q, H * D, mem.k_pages, mem.v_pages, mem.page_table, ctx.row_pos, ctx.row_slot, out, H, G, D,
                           window=self.window, scale=self.scale, value_dim=DV, chunk=self.chunk, sink=self.sink, out_scale=self.out_scale)
