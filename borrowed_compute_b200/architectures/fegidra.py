"""The Fegidra decoder as a layout of parts.

Every layer is a parallel block, x += mixer(conv(norm1 x)) + feed_forward(norm2 x), whose
mixer is named layer by layer: the generalized delta rule (a recurrent mixer with a float
state a head) or grouped-query attention with biases, a norm of q and of k over the whole
projection, rotation of part of each head, values narrower than keys and a chunk mask.  The
feed-forward is dense with the PolyNorm activation, or absent.  The model keeps no table of
positions and has no limit of its own on a sequence's length; the engine's does.

Tensor names: ``embed``, ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.canon1``, ``l<i>.mix.*``,
``l<i>.mlp.*``, ``final.norm``, ``head``; matrices are [out, in].
"""

from __future__ import annotations

from ..config.fegidra import AttentionMixerConfig, FegidraConfig, complete_from_shapes
from ..parts.base import LayerSpec, ModelSpec, PartSpec, RunSpec
from .registry import register_architecture

# The design fixes no longest sequence; this bounds the rotary table an engine would build if asked for everything.
NO_LIMIT = 1 << 20


def fegidra_model_spec(cfg: FegidraConfig) -> ModelSpec:
    layers, tolerated = [], []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        parts = {"norm1": PartSpec("rmsnorm", {"size": cfg.width, "eps": cfg.norm_eps, "tensor": "norm1"}, p)}
        if cfg.taps > 0:
            parts["conv"] = PartSpec("causal_conv_residual", {"width": cfg.width, "taps": cfg.taps, "tensor": "canon1"}, p)
        m = layer.mixer
        if isinstance(m, AttentionMixerConfig):
            position = {"kind": "none"} if m.rot_dims == 0 else \
                {"kind": "rotary", "head_dim": m.rot_dims, "theta": m.rot_base, "pairing": "half", "max_positions": NO_LIMIT}
            parts["mixer"] = PartSpec("gqa_attention_kv", {
                "hidden_size": cfg.width, "heads": m.heads, "kv_heads": m.kv_heads, "head_dim": m.dim, "value_dim": m.vdim,
                "position": position, "scale": m.scale, "chunk": m.chunk, "bias": True, "qk_norm_eps": cfg.norm_eps}, p + "mix.")
        else:
            parts["mixer"] = PartSpec("generalized_delta", {
                "hidden_size": cfg.width, "heads": m.heads, "head_dim": m.dim, "decay_rank": m.decay_rank, "norm_eps": cfg.norm_eps}, p + "mix.")
        if layer.ff > 0:
            parts["norm2"] = PartSpec("rmsnorm", {"size": cfg.width, "eps": cfg.norm_eps, "tensor": "norm2"}, p)
            parts["feed_forward"] = PartSpec("polynorm_mlp", {"hidden_size": cfg.width, "intermediate_size": layer.ff, "eps": cfg.norm_eps}, p + "mlp.")
        else:
            tolerated.append((p + "norm2", (cfg.width,)))      # the norm of the branch this layer leaves out
        layers.append(LayerSpec("parallel", parts))
    return ModelSpec(
        hidden_size=cfg.width,
        vocab_size=cfg.vocab,
        max_positions=NO_LIMIT,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "tensor": "embed"}, ""),
        layers=tuple(layers),
        schedule=tuple(RunSpec(i) for i in range(len(layers))),
        final_norm=PartSpec("rmsnorm", {"size": cfg.width, "eps": cfg.norm_eps, "tensor": "norm"}, "final."),
        head=PartSpec("linear_head", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "tensor": "head"}, ""),
        tolerated=tuple(tolerated),
    )


register_architecture("Fegidra", FegidraConfig.from_dict, fegidra_model_spec, complete=complete_from_shapes)
