"""The Logirax decoder as a layout of parts.

Every layer is a sandwich block, x += norm1b(mixer(shift(norm1 x))); x += norm2b(ff(norm2 x)), whose norms store their weights
around zero (w = 1 + stored) and whose mixer reads its input after a token shift (every channel moves part of the way towards
its value at the position before).  The mixer is grouped-query attention whose heads' scores are mixed before the softmax,
whose values are its keys and whose window keeps the first positions, or latent attention with neighbouring rotated pairs and a
learned sink.  The feed-forward is dense with a clipped gate, or routed experts (sigmoid scores, the chosen ones' weights
divided by their sum and scaled) plus a shared expert, or absent.  Embedded rows are scaled; the head is the embedding table,
its scores scaled.

Tensor names: ``embed``, ``l<i>.norm1``, ``l<i>.norm1b``, ``l<i>.norm2``, ``l<i>.norm2b``, ``l<i>.shift``, ``l<i>.mix.*``,
``l<i>.mlp.*``, ``final.norm``; matrices are [out, in].
"""

from __future__ import annotations

from ..config.logirax import ClippedDenseConfig, LogiraxConfig, TalkingMixerConfig
from ..parts.base import LayerSpec, ModelSpec, PartSpec, RunSpec
from .registry import register_architecture

# The design fixes no longest sequence; this bounds the rotary table an engine would build if asked for everything.
NO_LIMIT = 1 << 20


def logirax_model_spec(cfg: LogiraxConfig) -> ModelSpec:
    E, eps = cfg.width, cfg.norm_eps

    def norm(name: str, prefix: str) -> PartSpec:
        return PartSpec("rmsnorm", {"size": E, "eps": eps, "tensor": name, "offset": 1.0}, prefix)

    layers, schedule = [], []
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}.", layer.mixer
        if isinstance(m, TalkingMixerConfig):
            position = {"kind": "none"} if not m.rot_dims else \
                {"kind": "rotary", "head_dim": m.rot_dims, "theta": m.rot_base, "pairing": "half", "max_positions": NO_LIMIT}
            mixer = PartSpec("talking_attention", {
                "hidden_size": E, "heads": m.heads, "kv_heads": m.kv_heads, "head_dim": m.dim, "norm_eps": eps, "position": position,
                "scale": m.scale, "softcap": m.softcap, "window": m.window, "keep_first": m.keep_first, "bias": True}, p + "mix.")
        else:
            position = {"kind": "none"} if not m.rot_dim else \
                {"kind": "rotary", "head_dim": m.rot_dim, "theta": m.rot_base, "pairing": "adjacent", "max_positions": NO_LIMIT}
            mixer = PartSpec("latent_attention", {
                "hidden_size": E, "heads": m.heads, "head_dim": m.dim, "value_dim": m.vdim, "q_rank": m.q_rank, "kv_rank": m.kv_rank,
                "norm_eps": eps, "rot_dim": m.rot_dim, "position": position, "scale": m.scale, "sink": True}, p + "mix.")
        parts = {"norm1": norm("norm1", p), "conv": PartSpec("token_shift", {"width": E, "tensor": "shift"}, p), "mixer": mixer,
                 "norm1b": norm("norm1b", p)}
        f = layer.mlp
        if f is not None:
            parts["norm2"], parts["norm2b"] = norm("norm2", p), norm("norm2b", p)
            if isinstance(f, ClippedDenseConfig):
                parts["feed_forward"] = PartSpec("clipped_glu", {"hidden_size": E, "intermediate_size": f.ff, "limit": f.limit}, p + "mlp.")
            else:
                parts["feed_forward"] = PartSpec("routed_experts", {
                    "hidden_size": E, "experts": f.experts, "top": f.top, "intermediate_size": f.ff, "shared_size": f.shared_ff,
                    "score": "sigmoid", "renormalize": True, "weight_on": "output", "weight_factor": f.weight_scale}, p + "mlp.")
        layers.append(LayerSpec("sandwich", parts))
        schedule.append(RunSpec(i))
    tolerated = tuple((f"l{i}.{n}", (E,)) for i, layer in enumerate(cfg.layers) if layer.mlp is None for n in ("norm2", "norm2b"))
    return ModelSpec(
        hidden_size=E,
        vocab_size=cfg.vocab,
        max_positions=NO_LIMIT,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": E, "tensor": "embed", "scale": cfg.embedding_scale}, ""),
        layers=tuple(layers),
        schedule=tuple(schedule),
        final_norm=norm("norm", "final."),
        head=PartSpec("linear_head", {"vocab_size": cfg.vocab, "hidden_size": E, "tied": True, "tensor": "head", "scale": cfg.logit_scale}, ""),
        tolerated=tolerated,
    )


register_architecture("Logirax", LogiraxConfig.from_dict, logirax_model_spec)
