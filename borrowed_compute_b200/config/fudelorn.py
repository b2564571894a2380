"""Typed configuration of the Fudelorn decoder, read from its config.json.

The file gives the model's sizes (``vocab``, ``width``), ``norm.eps`` and a list ``layers`` whose entries differ: each
names its mixer by ``type`` (``latent_attention``: a latent of keys and values, a rotated key part the heads share,
every earlier position visible; ``latent_attention_2``: no positions, a sliding window), the mixer's sizes in ``mixer``
and its feed-forward in ``mlp`` (``kind`` ``dense`` or ``moe``, or null for none).  A mixer with ``kv_from`` reads the
cache of the layer it names instead of keeping one.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple

from .errors import ConfigError
from .fegidra import _num

MIXER_TYPES = ("latent_attention", "latent_attention_2")


@dataclass(frozen=True)
class StretchConfig:
    """How rotary frequencies are stretched for long contexts (None: not at all)."""
    factor: float
    original: float
    fast: float
    slow: float


@dataclass(frozen=True)
class LatentMixerConfig:
    heads: int
    dim: int              # plain query/key dimensions a head
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    rot_dim: int          # rotated query/key dimensions a head (0: none); the rotated key part is shared by the heads
    rot_base: float
    stretch: Optional[StretchConfig]
    window: int           # 0: every earlier position
    kv_from: Optional[int]


@dataclass(frozen=True)
class DenseConfig:
    ff: int


@dataclass(frozen=True)
class TableExpertsConfig:
    experts: int
    top: int
    ff: int
    shared_ff: int        # 0: no shared expert


@dataclass(frozen=True)
class FudelornLayerConfig:
    type: str
    mixer: LatentMixerConfig
    mlp: Any              # DenseConfig, TableExpertsConfig or None


def _mixer(kind: str, m: Any, where: str) -> LatentMixerConfig:
    heads, dim = _num(m, "heads", where), _num(m, "dim", where)
    rot_dim = _num(m, "rot_dim", where, default=0, positive=False)
    rot, mask = m.get("rot"), m.get("mask")
    if kind == "latent_attention_2" and (rot_dim or rot is not None):
        raise ConfigError(f"config.json: '{where}' is of a type without positions and may not rotate")
    if kind == "latent_attention_2" and mask is None:
        raise ConfigError(f"config.json: required key '{where}.mask' is missing")
    base, stretch = 10000.0, None
    if rot_dim:
        if rot_dim < 0 or rot_dim % 2:
            raise ConfigError(f"config.json: '{where}.rot_dim' ({rot_dim}) must be even")
        if rot is None:
            raise ConfigError(f"config.json: required key '{where}.rot' is missing")
        if _num(rot, "dims", where + ".rot") != rot_dim:
            raise ConfigError(f"config.json: '{where}.rot.dims' must equal rot_dim ({rot_dim}): the whole rotated part turns")
        base = _num(rot, "base", where + ".rot", float)
        sc = rot.get("scaling")
        if sc is not None:
            w = where + ".rot.scaling"
            stretch = StretchConfig(factor=_num(sc, "factor", w, float), original=_num(sc, "original", w, float), fast=_num(sc, "fast", w, float),
                                    slow=_num(sc, "slow", w, float))
    kv_from = m.get("kv_from")
    if kv_from is not None and (isinstance(kv_from, bool) or not isinstance(kv_from, int) or kv_from < 0):
        raise ConfigError(f"config.json: '{where}.kv_from' must name a layer, got {kv_from!r}")
    return LatentMixerConfig(
        heads=heads, dim=dim, vdim=_num(m, "vdim", where, default=dim), q_rank=_num(m, "q_rank", where), kv_rank=_num(m, "kv_rank", where),
        scale=_num(m, "scale", where, float, default=1.0 / float(dim + rot_dim) ** 0.5), rot_dim=rot_dim, rot_base=base, stretch=stretch,
        window=_num(mask, "size", where + ".mask") if mask is not None else 0, kv_from=kv_from)


def _mlp(mlp: Any, where: str):
    if mlp is None:
        return None
    if not isinstance(mlp, Mapping) or mlp.get("kind") not in ("dense", "moe"):
        raise ConfigError(f"config.json: '{where}.kind' must be 'dense' or 'moe', got {mlp.get('kind') if isinstance(mlp, Mapping) else mlp!r}")
    if mlp["kind"] == "dense":
        return DenseConfig(ff=_num(mlp, "ff", where))
    experts, top = _num(mlp.get("router"), "experts", where + ".router"), _num(mlp.get("router"), "top", where + ".router")
    if top > experts:
        raise ConfigError(f"config.json: '{where}.router.top' ({top}) is more than the {experts} experts")
    shared = mlp.get("shared")
    return TableExpertsConfig(experts=experts, top=top, ff=_num(mlp.get("expert"), "ff", where + ".expert"),
                              shared_ff=_num(shared, "ff", where + ".shared") if shared is not None else 0)


@dataclass(frozen=True)
class FudelornConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[FudelornLayerConfig, ...]

    @staticmethod
    def from_dict(d: Mapping[str, Any]) -> "FudelornConfig":
        vocab, width = _num(d, "vocab", ""), _num(d, "width", "")
        if d.get("norm") is None:
            raise ConfigError("config.json: required key 'norm.eps' is missing")
        eps = _num(d.get("norm"), "eps", "norm", float)
        raw = d.get("layers")
        if not isinstance(raw, (list, tuple)) or not raw:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, entry in enumerate(raw):
            where = f"layers[{i}]"
            if not isinstance(entry, Mapping) or entry.get("type") not in MIXER_TYPES:
                raise ConfigError(f"config.json: '{where}.type' must be one of {list(MIXER_TYPES)}, got "
                                  f"{entry.get('type') if isinstance(entry, Mapping) else entry!r}")
            if not isinstance(entry.get("mixer"), Mapping):
                raise ConfigError(f"config.json: '{where}.mixer' must be an object")
            mixer = _mixer(entry["type"], entry["mixer"], where + ".mixer")
            if mixer.kv_from is not None:
                j = mixer.kv_from
                if j >= i or layers[j].mixer.kv_from is not None:
                    raise ConfigError(f"config.json: '{where}.mixer.kv_from' ({j}) must name an earlier layer that keeps a cache of its own")
                o = layers[j].mixer
                if (o.kv_rank, o.rot_dim, o.rot_base, o.stretch) != (mixer.kv_rank, mixer.rot_dim, mixer.rot_base, mixer.stretch):
                    raise ConfigError(f"config.json: '{where}.mixer' reads layer {j}'s cache, so its kv_rank, rot_dim and rotation must equal that layer's")
                if o.window and (mixer.window == 0 or mixer.window > o.window):
                    raise ConfigError(f"config.json: '{where}.mixer' sees further back than layer {j}, whose cache it reads, keeps")
            layers.append(FudelornLayerConfig(type=entry["type"], mixer=mixer, mlp=_mlp(entry.get("mlp"), where + ".mlp")))
        return FudelornConfig(vocab=vocab, width=width, norm_eps=eps, layers=tuple(layers))
