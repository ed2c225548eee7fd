"""Typed configuration of the Pozirax decoder, read from its config.json.

The file gives the model's sizes (``vocab``, ``width``), its constants (``norm.eps``,
``embedding.scale``, ``logit_softcap``), a list ``layers`` whose entries differ (each names
its mixer by ``type``, the mixer's sizes in ``mixer`` and its feed-forward in ``mlp``, or
null for none) and, optionally, ``loop``: a stretch of layers that runs several times.  The
one size the file does not give, the inner width of a gated-linear-attention mixer's decay
projection, is the shape of a tensor and is filled in from the model folder
(``complete_from_shapes``); a configuration written by hand states it as ``mixer.rank``.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple

from .errors import ConfigError
from .fegidra import _num

MIXER_TYPES = ("gla", "parallel")


@dataclass(frozen=True)
class GlaMixerConfig:
    heads: int
    dim: int
    vdim: int
    tau: float
    rank: int


@dataclass(frozen=True)
class WindowAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int           # 0: every earlier position
    rot_dims: int         # 0: no rotation
    rot_base: float


@dataclass(frozen=True)
class StateSpaceConfig:
    heads: int
    vdim: int
    state: int
    groups: int
    norm_groups: int
    taps: int


@dataclass(frozen=True)
class PairMixerConfig:
    left: WindowAttentionConfig
    right: StateSpaceConfig
    left_scale: float
    right_scale: float


@dataclass(frozen=True)
class ExpertsConfig:
    experts: int
    top: int
    ff: int
    shared_ff: int        # 0: no shared expert


@dataclass(frozen=True)
class PoziraxLayerConfig:
    type: str
    mixer: Any                       # GlaMixerConfig or PairMixerConfig
    mlp: Optional[ExpertsConfig]     # None: no feed-forward


@dataclass(frozen=True)
class LoopConfig:
    start: int
    stop: int
    times: int


def _attention(m: Any, where: str) -> WindowAttentionConfig:
    heads, dim = _num(m, "heads", where), _num(m, "dim", where)
    kv_heads = _num(m, "kv_heads", where, default=heads)
    if heads % kv_heads:
        raise ConfigError(f"config.json: '{where}.heads' ({heads}) is not a multiple of kv_heads ({kv_heads})")
    rot, mask = m.get("rot"), m.get("mask")
    rot_dims = _num(rot, "dims", where + ".rot") if rot is not None else 0
    if rot_dims % 2 or rot_dims > dim:
        raise ConfigError(f"config.json: '{where}.rot.dims' ({rot_dims}) must be even and at most dim ({dim})")
    return WindowAttentionConfig(
        heads=heads, kv_heads=kv_heads, dim=dim, vdim=_num(m, "vdim", where, default=dim),
        scale=_num(m, "scale", where, float, default=1.0 / float(dim) ** 0.5),
        window=_num(mask, "size", where + ".mask") if mask is not None else 0,
        rot_dims=rot_dims, rot_base=_num(rot, "base", where + ".rot", float) if rot is not None else 10000.0)


def _state_space(m: Any, where: str) -> StateSpaceConfig:
    heads, groups = _num(m, "heads", where), _num(m, "groups", where, default=1)
    vdim, parts = _num(m, "vdim", where), _num(m, "norm_groups", where, default=1)
    if heads % groups:
        raise ConfigError(f"config.json: '{where}.heads' ({heads}) is not a multiple of groups ({groups})")
    if (heads * vdim) % parts:
        raise ConfigError(f"config.json: '{where}.norm_groups' ({parts}) does not divide heads * vdim ({heads * vdim})")
    return StateSpaceConfig(heads=heads, vdim=vdim, state=_num(m, "state", where), groups=groups, norm_groups=parts, taps=_num(m, "conv", where))


def _experts(mlp: Any, where: str) -> ExpertsConfig:
    if not isinstance(mlp, Mapping) or mlp.get("kind") != "moe":
        raise ConfigError(f"config.json: '{where}.kind' {mlp.get('kind') if isinstance(mlp, Mapping) else mlp!r} is not supported (only 'moe')")
    experts, top = _num(mlp.get("router"), "experts", where + ".router"), _num(mlp.get("router"), "top", where + ".router")
    if top > experts:
        raise ConfigError(f"config.json: '{where}.router.top' ({top}) is more than the {experts} experts")
    shared = mlp.get("shared")
    return ExpertsConfig(experts=experts, top=top, ff=_num(mlp.get("expert"), "ff", where + ".expert"),
                         shared_ff=_num(shared, "ff", where + ".shared") if shared is not None else 0)


@dataclass(frozen=True)
class PoziraxConfig:
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    logit_softcap: float             # 0: scores as they are
    layers: Tuple[PoziraxLayerConfig, ...]
    loop: Optional[LoopConfig]

    @staticmethod
    def from_dict(d: Mapping[str, Any]) -> "PoziraxConfig":
        top = "config.json"
        vocab, width = _num(d, "vocab", top), _num(d, "width", top)
        if d.get("norm") is None:
            raise ConfigError("config.json: required key 'norm.eps' is missing")
        eps = _num(d["norm"], "eps", "norm", float)
        scale = _num(d["embedding"], "scale", "embedding", float) if d.get("embedding") is not None else 1.0
        softcap = _num(d, "logit_softcap", top, float) if d.get("logit_softcap") is not None else 0.0
        raw = d.get("layers")
        if not isinstance(raw, (list, tuple)) or not raw:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, entry in enumerate(raw):
            where = f"layers[{i}]"
            if not isinstance(entry, Mapping) or entry.get("type") not in MIXER_TYPES:
                raise ConfigError(f"config.json: '{where}.type' must be one of {list(MIXER_TYPES)}, got {entry.get('type') if isinstance(entry, Mapping) else entry!r}")
            m, mw = entry.get("mixer"), where + ".mixer"
            if not isinstance(m, Mapping):
                raise ConfigError(f"config.json: '{mw}' must be an object")
            if entry["type"] == "gla":
                dim = _num(m, "dim", mw)
                mixer: Any = GlaMixerConfig(heads=_num(m, "heads", mw), dim=dim, vdim=_num(m, "vdim", mw, default=dim),
                                            tau=_num(m, "tau", mw, float), rank=_num(m, "rank", mw))
            else:
                if not isinstance(m.get("left"), Mapping) or not isinstance(m.get("right"), Mapping):
                    raise ConfigError(f"config.json: '{mw}' needs the objects 'left' and 'right'")
                mixer = PairMixerConfig(left=_attention(m["left"], mw + ".left"), right=_state_space(m["right"], mw + ".right"),
                                        left_scale=_num(m, "left_scale", mw, float, default=1.0, positive=False),
                                        right_scale=_num(m, "right_scale", mw, float, default=1.0, positive=False))
            mlp = entry.get("mlp")
            layers.append(PoziraxLayerConfig(entry["type"], mixer, None if mlp is None else _experts(mlp, where + ".mlp")))
        loop = None
        if d.get("loop") is not None:
            lp = d["loop"]
            start = _num(lp, "start", "loop", positive=False)
            loop = LoopConfig(start=start, stop=_num(lp, "stop", "loop"), times=_num(lp, "times", "loop"))
            if not 0 <= loop.start < loop.stop <= len(layers):
                raise ConfigError(f"config.json: 'loop' runs layers {loop.start} to {loop.stop - 1}, the model has {len(layers)}")
        return PoziraxConfig(vocab=vocab, width=width, norm_eps=eps, embedding_scale=scale, logit_softcap=softcap, layers=tuple(layers), loop=loop)


def complete_from_shapes(config: Mapping[str, Any], shapes: Mapping[str, Tuple[int, ...]]) -> Dict[str, Any]:
    """config.json with the sizes that only tensor shapes give filled in: a gated-linear-attention mixer's
    ``rank`` is the number of rows of its inner decay projection ``l<i>.mix.a1``."""
    out = copy.deepcopy(dict(config))
    layers = out.get("layers")
    if not isinstance(layers, list):
        return out
    for i, entry in enumerate(layers):
        if isinstance(entry, dict) and entry.get("type") == "gla" and isinstance(entry.get("mixer"), dict) and "rank" not in entry["mixer"]:
            shape = shapes.get(f"l{i}.mix.a1")
            if shape is not None and len(shape) == 2:
                entry["mixer"]["rank"] = int(shape[0])
    return out
