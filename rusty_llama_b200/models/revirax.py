"""Revirax, as a description made of the library's parts.

A decoder whose layers norm each sublayer on both sides,
    x += norm_1b(mixer(norm_1(x)));  x += norm_2b(ff(norm_2(x)))          (a layer may have no ff)
with norm weights stored as their distance from one, a feed-forward W_down relu(W_up h)^2, and per layer one of three mixers:

  lightning   linear attention with a constant decay per head over silu'd q, k, v, the heads normed together, an output gate
  attention   grouped-query softmax attention: partly rotated heads (halves paired, frequencies rescaled by wavelength
              bands), its own score scale, a sink per head in the softmax's denominator
  parallel    two mixers on the same input, their results scaled and summed: a windowed softmax attention with biases,
              ramp-rescaled rotation with a magnitude, scores mixed across heads and an output gate; and a minimal gated
              recurrent unit

Tensor names: embed, head, final.norm, and per layer i: l<i>.norm1 / norm1b / norm2 / norm2b, l<i>.mix.<name>
(l<i>.mix.left.<name>, l<i>.mix.right.<name> in a parallel layer; a bias is its matrix's name + ".b"), l<i>.mlp.up / down.
"""

from __future__ import annotations

from ..config.revirax import (
    ARCHITECTURE, MAX_POSITIONS, LightningMixerConfig, ParallelMixerConfig, ReviraxConfig, SoftmaxMixerConfig,
)
from ..registry import Architecture, register_architecture
from ..spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

_ATTENTION_NAMES = {"q": "q", "k": "k", "v": "v", "o": "o", "gate": "g", "sink": "sink", "head_mix": "talk",
                    "q_bias": "q.b", "k_bias": "k.b", "v_bias": "v.b", "o_bias": "o.b"}


def _softmax_attention(m: SoftmaxMixerConfig, width: int, prefix: str, **options) -> PartSpec:
    position = PartSpec("rotary", {"rotary_dim": m.rot_dims, "theta": m.rot_base, "scaling": m.rot_scaling, "interleaved": False}) \
        if m.rot_dims else PartSpec("none")
    params = {
        "hidden_size": width, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim, "value_dim": m.vdim,
        "scale": m.scale, "window": m.window, "position": position, "names": _ATTENTION_NAMES,
    }
    params.update(options)
    return PartSpec("attention", params, prefix)


def describe_revirax(cfg: ReviraxConfig) -> ModelSpec:
    def norm(prefix: str) -> PartSpec:
        return PartSpec("rmsnorm", {"size": cfg.width, "eps": cfg.eps, "name": "", "offset": 1.0}, prefix)

    layers, schedule = [], []
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}.", layer.mixer
        if isinstance(m, LightningMixerConfig):
            mixer = PartSpec(
                "decay_linear_attention",
                {"hidden_size": cfg.width, "num_heads": m.heads, "dim": m.dim, "vdim": m.vdim, "decay": m.decay, "eps": cfg.eps,
                 "activation": "silu", "gate": True},
                p + "mix.",
            )
        elif isinstance(m, SoftmaxMixerConfig):
            mixer = _softmax_attention(m, cfg.width, p + "mix.", sink=True)
        elif isinstance(m, ParallelMixerConfig):
            left = _softmax_attention(m.left, cfg.width, "left.", bias=True, head_mix=True, gate=True)
            right = PartSpec("min_gru", {"hidden_size": cfg.width, "width": m.right_width, "bias": True}, "right.")
            mixer = PartSpec("parallel", {"branches": ((left, m.left_scale), (right, m.right_scale))}, p + "mix.")
        else:
            raise TypeError(f"layer {i}: {type(m).__name__} is not a mixer configuration of this architecture")
        norms = {"mixer": norm(p + "norm1"), "mixer_out": norm(p + "norm1b")}
        ff = None
        if layer.mlp is not None:
            ff = PartSpec(
                "mlp", {"hidden_size": cfg.width, "intermediate_size": layer.mlp.ff, "activation": "relu2", "names": {"up": "up", "down": "down"}},
                p + "mlp.",
            )
            norms.update({"feed_forward": norm(p + "norm2"), "feed_forward_out": norm(p + "norm2b")})
        layers.append(LayerSpec(block="sandwich", mixer=mixer, feed_forward=ff, norms=norms))
        schedule.append(ScheduleEntry(i))
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


register_architecture(Architecture(ARCHITECTURE, ReviraxConfig.from_json, describe_revirax), replace=True)
