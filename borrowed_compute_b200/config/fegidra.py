"""Typed configuration of the Fegidra decoder, read from its config.json.

The file gives the model's sizes (``vocab``, ``width``), two constants (``norm.eps``,
``canon.taps``) and a list ``layers`` whose entries differ: each names its mixer (``type``),
the mixer's sizes (``mixer``) and its feed-forward (``mlp``, or null for none).  The one size
the file does not give, the inner width of a delta-rule mixer's decay projection, is the
shape of a tensor and is filled in from the model folder (``complete_from_shapes``); a
configuration written by hand states it as ``mixer.decay_rank``.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple

from .errors import ConfigError

MIXER_TYPES = ("general_delta", "attention")


def _num(d: Mapping[str, Any], key: str, where: str, kind=int, default=None, positive: bool = True):
    if not isinstance(d, Mapping):
        raise ConfigError(f"config.json: '{where}' must be an object")
    if key not in d or d[key] is None:
        if default is not None:
            return default
        raise ConfigError(f"config.json: required key '{where}.{key}' is missing")
    v = d[key]
    if isinstance(v, bool) or not isinstance(v, (int, float) if kind is float else int):
        raise ConfigError(f"config.json: '{where}.{key}' must be {'a number' if kind is float else 'an integer'}, got {v!r}")
    if positive and not v > 0:
        raise ConfigError(f"config.json: '{where}.{key}' must be positive, got {v!r}")
    return kind(v)


@dataclass(frozen=True)
class DeltaMixerConfig:
    heads: int
    dim: int
    decay_rank: int


@dataclass(frozen=True)
class AttentionMixerConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    chunk: int            # 0: no chunk mask
    rot_dims: int         # 0: no rotation
    rot_base: float


@dataclass(frozen=True)
class FegidraLayerConfig:
    type: str
    mixer: Any                      # DeltaMixerConfig or AttentionMixerConfig
    ff: int                         # 0: no feed-forward


@dataclass(frozen=True)
class FegidraConfig:
    vocab: int
    width: int
    norm_eps: float
    taps: int                       # 0: no input convolution
    layers: Tuple[FegidraLayerConfig, ...]

    @staticmethod
    def from_dict(d: Mapping[str, Any]) -> "FegidraConfig":
        top = "config.json"
        vocab, width = _num(d, "vocab", top), _num(d, "width", top)
        eps = _num(d.get("norm"), "eps", "norm", float) if d.get("norm") is not None else None
        if eps is None:
            raise ConfigError("config.json: required key 'norm.eps' is missing")
        taps = _num(d["canon"], "taps", "canon") if d.get("canon") is not None else 0
        raw = d.get("layers")
        if not isinstance(raw, (list, tuple)) or not raw:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, entry in enumerate(raw):
            where = f"layers[{i}]"
            if not isinstance(entry, Mapping) or entry.get("type") not in MIXER_TYPES:
                raise ConfigError(f"config.json: '{where}.type' must be one of {list(MIXER_TYPES)}, got {entry.get('type') if isinstance(entry, Mapping) else entry!r}")
            m = entry.get("mixer")
            mw = where + ".mixer"
            if entry["type"] == "general_delta":
                mixer = DeltaMixerConfig(heads=_num(m, "heads", mw), dim=_num(m, "dim", mw), decay_rank=_num(m, "decay_rank", mw))
            else:
                heads, dim = _num(m, "heads", mw), _num(m, "dim", mw)
                kv_heads = _num(m, "kv_heads", mw, default=heads)
                if heads % kv_heads:
                    raise ConfigError(f"config.json: '{mw}.heads' ({heads}) is not a multiple of kv_heads ({kv_heads})")
                rot, mask = m.get("rot"), m.get("mask")
                rot_dims = _num(rot, "dims", mw + ".rot") if rot is not None else 0
                if rot_dims % 2 or rot_dims > dim:
                    raise ConfigError(f"config.json: '{mw}.rot.dims' ({rot_dims}) must be even and at most dim ({dim})")
                mixer = AttentionMixerConfig(
                    heads=heads, kv_heads=kv_heads, dim=dim, vdim=_num(m, "vdim", mw, default=dim),
                    scale=_num(m, "scale", mw, float, default=1.0 / float(dim) ** 0.5),
                    chunk=_num(mask, "size", mw + ".mask") if mask is not None else 0,
                    rot_dims=rot_dims, rot_base=_num(rot, "base", mw + ".rot", float) if rot is not None else 10000.0)
            mlp = entry.get("mlp")
            ff = 0
            if mlp is not None:
                if not isinstance(mlp, Mapping) or mlp.get("kind", "dense") != "dense":
                    raise ConfigError(f"config.json: '{where}.mlp.kind' {mlp.get('kind') if isinstance(mlp, Mapping) else mlp!r} is not supported (only 'dense')")
                ff = _num(mlp, "ff", where + ".mlp")
            layers.append(FegidraLayerConfig(entry["type"], mixer, ff))
        return FegidraConfig(vocab=vocab, width=width, norm_eps=eps, taps=taps, layers=tuple(layers))


def complete_from_shapes(config: Mapping[str, Any], shapes: Mapping[str, Tuple[int, ...]]) -> Dict[str, Any]:
    """config.json with the sizes that only tensor shapes give filled in: a delta-rule mixer's
    ``decay_rank`` is the number of rows of its inner decay projection ``l<i>.mix.w1``."""
    out = copy.deepcopy(dict(config))
    layers = out.get("layers")
    if not isinstance(layers, list):
        return out
    for i, entry in enumerate(layers):
        if isinstance(entry, dict) and entry.get("type") == "general_delta" and isinstance(entry.get("mixer"), dict) \
                and "decay_rank" not in entry["mixer"]:
            shape = shapes.get(f"l{i}.mix.w1")
            if shape is not None and len(shape) == 2:
                entry["mixer"]["decay_rank"] = int(shape[0])
    return out
