"""Vezatar, as a description made of the library's parts.

A decoder whose layers norm each sublayer on both sides,
    x += norm_1b(mixer(norm_1(x)));  x += norm_2b(ff(norm_2(x)))          (a layer may have no ff)
with a latent-attention mixer (one cached latent per position, shared rotated key part, softmax sink, output gate;
a layer may read an earlier layer's cache instead of projecting a latent of its own) and, per layer, a dense
feed-forward with a clamped gate or a routed one with a shared expert.  Tensor names: embed, head, final.norm,
and per layer i: l<i>.norm1 / norm1b / norm2 / norm2b, l<i>.mix.<name>, l<i>.mlp.<name>.
"""

from __future__ import annotations

from ..config.vezatar import ARCHITECTURE, DENSE_GATE_ALPHA, MAX_POSITIONS, DenseMlpConfig, MoeMlpConfig, VezatarConfig
from ..registry import Architecture, register_architecture
from ..spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry


def describe_vezatar(cfg: VezatarConfig) -> ModelSpec:
    def norm(prefix: str) -> PartSpec:
        return PartSpec("rmsnorm", {"size": cfg.width, "eps": cfg.eps, "name": ""}, prefix)

    layers, schedule = [], []
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}.", layer.mixer
        position = PartSpec("rotary", {"rotary_dim": m.rot_dims, "theta": m.rot_base, "scaling": m.rot_scaling, "interleaved": True}) \
            if m.rot_dims else PartSpec("none")
        mixer = PartSpec(
            "latent_attention",
            {
                "hidden_size": cfg.width, "num_heads": m.heads, "dim": m.dim, "rot_dim": m.rot_dim, "vdim": m.vdim,
                "kv_rank": m.kv_rank, "scale": m.scale, "eps": cfg.eps, "sink": True, "gate": True,
                "own_kv": m.kv_from is None, "window": 0, "position": position,
            },
            p + "mix.",
        )
        norms = {"mixer": norm(p + "norm1"), "mixer_out": norm(p + "norm1b")}
        ff = None
        if isinstance(layer.mlp, DenseMlpConfig):
            ff = PartSpec(
                "gated_mlp",
                {
                    "hidden_size": cfg.width, "intermediate_size": layer.mlp.ff, "activation": "clamped_swish",
                    "limit": layer.mlp.limit, "alpha": DENSE_GATE_ALPHA, "names": {"gate": "gate", "up": "up", "down": "down"},
                },
                p + "mlp.",
            )
        elif isinstance(layer.mlp, MoeMlpConfig):
            ff = PartSpec(
                "routed_experts",
                {
                    "hidden_size": cfg.width, "n_experts": layer.mlp.experts, "top": layer.mlp.top, "expert_ff": layer.mlp.expert_ff,
                    "bias": True, "renormalize": False, "shared_ff": layer.mlp.shared_ff, "shared_gate": layer.mlp.shared_ff > 0,
                },
                p + "mlp.",
            )
        if ff is not None:
            norms.update({"feed_forward": norm(p + "norm2"), "feed_forward_out": norm(p + "norm2b")})
        layers.append(LayerSpec(block="sandwich", mixer=mixer, feed_forward=ff, norms=norms))
        schedule.append(ScheduleEntry(i, cache_from=m.kv_from))
    return ModelSpec(
        architecture=cfg.architecture,
        hidden_size=cfg.width,
        vocab_size=cfg.vocab,
        max_positions=MAX_POSITIONS,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "name": ""}, "embed"),
        layers=tuple(layers),
        schedule=tuple(schedule),
        final_norm=norm("final.norm"),
        head=PartSpec("linear_head", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "tied_to": None, "name": ""}, "head"),
        stored_dtype="bfloat16",
    )


register_architecture(Architecture(ARCHITECTURE, VezatarConfig.from_json, describe_vezatar), replace=True)
