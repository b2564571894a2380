"""Typed configuration of the Logirax decoder, read from its config.json.

The file gives the model's sizes (``vocab``, ``width``), ``norm.eps``, ``embedding.scale``, ``logit_scale`` and a list
``layers`` whose entries differ: each names its mixer by ``type`` (``attention``: grouped-query attention whose heads' scores
are mixed, with a sliding window that keeps a sequence's first positions; ``latent_attention``: a latent of keys and values, a
rotated key part the heads share, a learned sink in the softmax), the mixer's sizes in ``mixer`` and its feed-forward in
``mlp`` (``kind`` ``dense`` with a ``limit``, or ``moe`` with ``router``, ``expert`` and ``shared``, or null for none).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from .errors import ConfigError
from .fegidra import _num

MIXER_TYPES = ("attention", "latent_attention")


@dataclass(frozen=True)
class TalkingMixerConfig:
    heads: int
    kv_heads: int
    dim: int
    scale: float
    softcap: float        # 0: scores are not bounded
    window: int           # 0: every earlier position
    keep_first: int       # positions at a sequence's start that stay visible behind the window
    rot_dims: int         # rotated dimensions of a head (0: none)
    rot_base: float


@dataclass(frozen=True)
class SinkLatentMixerConfig:
    heads: int
    dim: int              # plain query/key dimensions a head
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    rot_dim: int          # rotated query/key dimensions a head (0: none); the rotated key part is shared by the heads
    rot_base: float


@dataclass(frozen=True)
class ClippedDenseConfig:
    ff: int
    limit: float


@dataclass(frozen=True)
class RoutedExpertsConfig:
    experts: int
    top: int
    ff: int
    weight_scale: float
    shared_ff: int        # 0: no shared expert


@dataclass(frozen=True)
class LogiraxLayerConfig:
    type: str
    mixer: Any            # TalkingMixerConfig or SinkLatentMixerConfig
    mlp: Any              # ClippedDenseConfig, RoutedExpertsConfig or None


def _rotation(m: Mapping[str, Any], where: str) -> Tuple[int, float]:
    rot = m.get("rot")
    if rot is None:
        return 0, 10000.0
    dims = _num(rot, "dims", where + ".rot", positive=False)
    if dims < 0 or dims % 2:
        raise ConfigError(f"config.json: '{where}.rot.dims' ({dims}) must be even and not negative")
    return dims, _num(rot, "base", where + ".rot", float, default=10000.0)


def _talking(m: Any, where: str) -> TalkingMixerConfig:
    heads, dim = _num(m, "heads", where), _num(m, "dim", where)
    kv_heads = _num(m, "kv_heads", where, default=heads)
    if heads % kv_heads:
        raise ConfigError(f"config.json: '{where}.heads' ({heads}) must be a multiple of kv_heads ({kv_heads})")
    if _num(m, "vdim", where, default=dim) != dim:
        raise ConfigError(f"config.json: '{where}.vdim' must equal dim ({dim}): the values of this mixer are its keys")
    dims, base = _rotation(m, where)
    if dims > dim:
        raise ConfigError(f"config.json: '{where}.rot.dims' ({dims}) is more than the head's {dim} dimensions")
    mask = m.get("mask")
    window = _num(mask, "size", where + ".mask") if mask is not None else 0
    keep = _num(mask, "keep_first", where + ".mask", default=0, positive=False) if mask is not None else 0
    if keep < 0:
        raise ConfigError(f"config.json: '{where}.mask.keep_first' must not be negative, got {keep}")
    cap = _num(m, "softcap", where, float, default=0.0, positive=False)
    if cap < 0:
        raise ConfigError(f"config.json: '{where}.softcap' must not be negative, got {cap}")
    return TalkingMixerConfig(heads=heads, kv_heads=kv_heads, dim=dim, scale=_num(m, "scale", where, float, default=1.0 / float(dim) ** 0.5),
                              softcap=cap, window=window, keep_first=keep, rot_dims=dims, rot_base=base)


def _latent(m: Any, where: str) -> SinkLatentMixerConfig:
    heads, dim = _num(m, "heads", where), _num(m, "dim", where)
    rot_dim = _num(m, "rot_dim", where, default=0, positive=False)
    dims, base = _rotation(m, where)
    if rot_dim < 0 or rot_dim % 2:
        raise ConfigError(f"config.json: '{where}.rot_dim' ({rot_dim}) must be even and not negative")
    if dims != rot_dim:
        raise ConfigError(f"config.json: '{where}.rot.dims' ({dims}) must equal rot_dim ({rot_dim}): the whole rotated part turns")
    return SinkLatentMixerConfig(heads=heads, dim=dim, vdim=_num(m, "vdim", where, default=dim), q_rank=_num(m, "q_rank", where),
                                 kv_rank=_num(m, "kv_rank", where), scale=_num(m, "scale", where, float, default=1.0 / float(dim + rot_dim) ** 0.5),
                                 rot_dim=rot_dim, rot_base=base)


def _mlp(mlp: Any, where: str):
    if mlp is None:
        return None
    if not isinstance(mlp, Mapping) or mlp.get("kind") not in ("dense", "moe"):
        raise ConfigError(f"config.json: '{where}.kind' must be 'dense' or 'moe', got {mlp.get('kind') if isinstance(mlp, Mapping) else mlp!r}")
    if mlp["kind"] == "dense":
        return ClippedDenseConfig(ff=_num(mlp, "ff", where), limit=_num(mlp, "limit", where, float))
    router = mlp.get("router")
    experts, top = _num(router, "experts", where + ".router"), _num(router, "top", where + ".router")
    if top > experts:
        raise ConfigError(f"config.json: '{where}.router.top' ({top}) is more than the {experts} experts")
    shared = mlp.get("shared")
    return RoutedExpertsConfig(experts=experts, top=top, ff=_num(mlp.get("expert"), "ff", where + ".expert"),
                               weight_scale=_num(router, "scale", where + ".router", float, default=1.0),
                               shared_ff=_num(shared, "ff", where + ".shared") if shared is not None else 0)


@dataclass(frozen=True)
class LogiraxConfig:
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    logit_scale: float
    layers: Tuple[LogiraxLayerConfig, ...]

    @staticmethod
    def from_dict(d: Mapping[str, Any]) -> "LogiraxConfig":
        vocab, width = _num(d, "vocab", ""), _num(d, "width", "")
        if d.get("norm") is None:
            raise ConfigError("config.json: required key 'norm.eps' is missing")
        eps = _num(d.get("norm"), "eps", "norm", float)
        emb = d.get("embedding")
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
            mixer = (_talking if entry["type"] == "attention" else _latent)(entry["mixer"], where + ".mixer")
            layers.append(LogiraxLayerConfig(type=entry["type"], mixer=mixer, mlp=_mlp(entry.get("mlp"), where + ".mlp")))
        return LogiraxConfig(vocab=vocab, width=width, norm_eps=eps,
                             embedding_scale=_num(emb, "scale", "embedding", float, default=1.0) if emb is not None else 1.0,
                             logit_scale=_num(d, "logit_scale", "", float, default=1.0), layers=tuple(layers))
