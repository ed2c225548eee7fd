"""The Pozirax decoder as a layout of parts.

Every layer is a parallel block with one norm, x += mixer(h) + feed_forward(h) with h = norm1(x).  The mixer is
named layer by layer: gated linear attention (a recurrent mixer with a decay per key channel), or two mixers side
by side, sliding-window attention (a norm of every head of q and k, rotation of neighbouring dimensions, a sink in the
softmax) beside a state-space mixer of the dual form, each with a factor.  The feed-forward routes every row to a few
of many small gated experts (sigmoid scores as weights on the experts' input) and adds a shared expert, or is
absent.  The embedding's rows are scaled; the scores pass a soft cap.  A stretch of layers may run several times with
the same weights, each pass with a cache and state of its own; before each pass the stream is mixed with the
embedding's output and a vector of the pass is added.

Tensor names: ``embed``, ``loop.in``, ``loop.step``, ``l<i>.norm1``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm``,
``head``; matrices are [out, in].
"""

from __future__ import annotations

from ..config.pozirax import GlaMixerConfig, PoziraxConfig, complete_from_shapes
from ..parts.base import LayerSpec, ModelSpec, PartSpec, RunSpec
from .registry import register_architecture

# The design fixes no longest sequence; this bounds the rotary table an engine would build if asked for everything.
NO_LIMIT = 1 << 20


def pozirax_model_spec(cfg: PoziraxConfig) -> ModelSpec:
    E, eps = cfg.width, cfg.norm_eps
    layers = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        parts = {"norm1": PartSpec("rmsnorm", {"size": E, "eps": eps, "tensor": "norm1"}, p)}
        m = layer.mixer
        if isinstance(m, GlaMixerConfig):
            parts["mixer"] = PartSpec("gated_linear_attention", {
                "hidden_size": E, "heads": m.heads, "head_dim": m.dim, "value_dim": m.vdim, "decay_rank": m.rank, "tau": m.tau,
                "norm_eps": eps}, p + "mix.")
        else:
            a, s = m.left, m.right
            position = {"kind": "none"} if a.rot_dims == 0 else \
                {"kind": "rotary", "head_dim": a.rot_dims, "theta": a.rot_base, "pairing": "adjacent", "max_positions": NO_LIMIT}
            left = {"kind": "gqa_attention_kv", "hidden_size": E, "heads": a.heads, "kv_heads": a.kv_heads, "head_dim": a.dim,
                    "value_dim": a.vdim, "position": position, "scale": a.scale, "window": a.window, "qk_norm_eps": eps, "qk_norm": "head",
                    "sink": True, "out_scale": m.left_scale}
            right = {"kind": "state_space_dual", "hidden_size": E, "heads": s.heads, "value_dim": s.vdim, "state_dim": s.state,
                     "groups": s.groups, "norm_groups": s.norm_groups, "taps": s.taps, "norm_eps": eps, "out_scale": m.right_scale}
            parts["mixer"] = PartSpec("side_by_side", {"left": left, "right": right}, p + "mix.")
        if layer.mlp is not None:
            f = layer.mlp
            parts["feed_forward"] = PartSpec("routed_experts", {
                "hidden_size": E, "experts": f.experts, "top": f.top, "intermediate_size": f.ff, "shared_size": f.shared_ff,
                "score": "sigmoid", "renormalize": False, "weight_on": "input"}, p + "mlp.")
        layers.append(LayerSpec("parallel", parts))
    # The order of the runs: layers ahead of the stretch once, the stretch `times` times, the rest once.
    n = len(layers)
    schedule, junctions = [], ()
    if cfg.loop is None:
        schedule = [RunSpec(i) for i in range(n)]
    else:
        lp = cfg.loop
        junctions = (PartSpec("mix_with_embedding", {"hidden_size": E, "passes": lp.times, "matrix": "in", "steps": "step"}, "loop."),)
        schedule = [RunSpec(i) for i in range(lp.start)]
        for t in range(lp.times):
            schedule += [RunSpec(i, enter=(0, t) if i == lp.start else None) for i in range(lp.start, lp.stop)]
        schedule += [RunSpec(i) for i in range(lp.stop, n)]
    return ModelSpec(
        hidden_size=E,
        vocab_size=cfg.vocab,
        max_positions=NO_LIMIT,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": E, "tensor": "embed", "scale": cfg.embedding_scale}, ""),
        layers=tuple(layers),
        schedule=tuple(schedule),
        final_norm=PartSpec("rmsnorm", {"size": E, "eps": eps, "tensor": "norm"}, "final."),
        head=PartSpec("linear_head", {"vocab_size": cfg.vocab, "hidden_size": E, "tensor": "head", "softcap": cfg.logit_softcap}, ""),
        junctions=junctions,
    )


register_architecture("Pozirax", PoziraxConfig.from_dict, pozirax_model_spec, complete=complete_from_shapes)
