"""The Fudelorn decoder as a layout of parts.

Every layer is a sandwich block, x += norm1b(mixer(norm1 x)); x += norm2b(ff(norm2 x)), whose mixer is latent attention:
with a rotated key part that the heads share and every earlier position visible, or without positions and with a sliding
window.  A mixer may read an earlier layer's cache instead of keeping one.  The feed-forward is dense with the square of
relu, or experts of that form named by a table from the token id, plus a shared expert with a gate; or absent.

Tensor names: ``embed``, ``l<i>.norm1``, ``l<i>.norm1b``, ``l<i>.norm2``, ``l<i>.norm2b``, ``l<i>.mix.*``, ``l<i>.mlp.*``,
``final.norm``, ``head``; matrices are [out, in].
"""

from __future__ import annotations

from ..config.fudelorn import DenseConfig, FudelornConfig
from ..parts.base import LayerSpec, ModelSpec, PartSpec, RunSpec
from .registry import register_architecture

# The design fixes no longest sequence; this bounds the rotary table an engine would build if asked for everything.
NO_LIMIT = 1 << 20


def fudelorn_model_spec(cfg: FudelornConfig) -> ModelSpec:
    E, eps = cfg.width, cfg.norm_eps
    layers, schedule = [], []
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}.", layer.mixer
        position = {"kind": "none"}
        if m.rot_dim:
            s = m.stretch
            position = {"kind": "rotary", "head_dim": m.rot_dim, "theta": m.rot_base, "pairing": "half", "max_positions": NO_LIMIT,
                        "scaling": None if s is None else {"type": "yarn", "factor": s.factor, "original": s.original, "fast": s.fast, "slow": s.slow}}
        parts = {
            "norm1": PartSpec("rmsnorm", {"size": E, "eps": eps, "tensor": "norm1"}, p),
            "norm1b": PartSpec("rmsnorm", {"size": E, "eps": eps, "tensor": "norm1b"}, p),
            "mixer": PartSpec("latent_attention", {
                "hidden_size": E, "heads": m.heads, "head_dim": m.dim, "value_dim": m.vdim, "q_rank": m.q_rank, "kv_rank": m.kv_rank,
                "norm_eps": eps, "rot_dim": m.rot_dim, "position": position, "scale": m.scale, "window": m.window,
                "own_kv": m.kv_from is None}, p + "mix."),
        }
        f = layer.mlp
        if f is not None:
            parts["norm2"] = PartSpec("rmsnorm", {"size": E, "eps": eps, "tensor": "norm2"}, p)
            parts["norm2b"] = PartSpec("rmsnorm", {"size": E, "eps": eps, "tensor": "norm2b"}, p)
            if isinstance(f, DenseConfig):
                parts["feed_forward"] = PartSpec("plain_mlp", {"hidden_size": E, "intermediate_size": f.ff, "activation": "relu2"}, p + "mlp.")
            else:
                parts["feed_forward"] = PartSpec("routed_experts", {
                    "hidden_size": E, "experts": f.experts, "top": f.top, "intermediate_size": f.ff, "shared_size": f.shared_ff,
                    "weight_on": "output", "router": "table", "expert": "relu2", "shared_gate": f.shared_ff > 0, "vocab_size": cfg.vocab}, p + "mlp.")
        layers.append(LayerSpec("sandwich", parts))
        schedule.append(RunSpec(i, memory_of=m.kv_from))
    return ModelSpec(
        hidden_size=E,
        vocab_size=cfg.vocab,
        max_positions=NO_LIMIT,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": E, "tensor": "embed"}, ""),
        layers=tuple(layers),
        schedule=tuple(schedule),
        final_norm=PartSpec("rmsnorm", {"size": E, "eps": eps, "tensor": "norm"}, "final."),
        head=PartSpec("linear_head", {"vocab_size": cfg.vocab, "hidden_size": E, "tensor": "head"}, ""),
    )


register_architecture("Fudelorn", FudelornConfig.from_dict, fudelorn_model_spec)
