"""The Simetar decoder, described as data and registered by name.

A layer: x += norm1(mixer(x)), then, where the layer has a feed-forward,
x += norm2(ff(x)); the sublayers read the stream itself and the layer norms (weight and
bias) sit on what they return. The model's last norm is a layer norm too; the head has a
table of its own. Tensor names: `embed`, `head`, `final.norm`, `final.norm.b`, and per
layer `l<i>.` + norm1, norm1.b, norm2, norm2.b, mix.*, mlp.*.
"""

from __future__ import annotations

import dataclasses

from ..config.registry import register_architecture
from ..config.simetar import BandScaling, SimetarConfig
from ..parts.spec import LayerSpec, ModelSpec, PartSpec


def describe_simetar(cfg: SimetarConfig) -> ModelSpec:
    width = cfg.width

    def norm(name: str) -> PartSpec:
        return PartSpec("layernorm", {"hidden_size": width, "eps": cfg.norm_eps}, {"weight": name, "bias": name + ".b"})

    layers = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        m = p + "mix."
        scaling = dataclasses.asdict(layer.scaling) if layer.scaling is not None else None
        if layer.type == "attention":
            bands = None
            if isinstance(layer.scaling, BandScaling):
                bands = {"factor": layer.scaling.factor, "low_freq_factor": layer.scaling.low,
                         "high_freq_factor": layer.scaling.high,
                         "original_max_position_embeddings": layer.scaling.original}
            position = PartSpec("rope_pairs", {"theta": layer.rot_base, "rotary_dim": layer.rot_dims, "llama3": bands})
            names = {"q": m + "q", "q_bias": m + "q.b", "k": m + "k", "k_bias": m + "k.b", "q_norm": m + "q.norm",
                     "k_norm": m + "k.norm", "gate": m + "g", "o": m + "o"}
            if layer.taps is not None:  # (a single tap is still stored: one factor per channel)
                names.update(q_conv=m + "q.conv", k_conv=m + "k.conv")
            mixer = PartSpec(
                "conv_attention",
                {"hidden_size": width, "n_heads": layer.heads, "n_kv_heads": layer.kv_heads, "head_dim": layer.dim,
                 "scale": layer.scale, "window": layer.window, "softcap": layer.softcap, "sink_logit": 0.0,
                 "taps": layer.taps or 1, "norm_eps": cfg.norm_eps, "position": position}, names)
        else:
            position = PartSpec("rope", {"theta": layer.rot_base, "head_dim": layer.rot_dims,
                                         "rotary_dim": layer.rot_dims, "ramp": scaling})
            mixer = PartSpec(
                "latent_attention",
                {"hidden_size": width, "n_heads": layer.heads, "head_dim": layer.dim, "value_dim": layer.value_dim,
                 "latent_rank": layer.latent_rank, "scale": layer.scale, "window": None, "eps": cfg.norm_eps,
                 "sink": False, "gate": "element", "rope_dim": layer.rot_dim, "position": position,
                 "cache_from": layer.kv_from},
                {"q": m + "q", "down": m + "dkv", "latent_norm": m + "dkv.norm", "up_k": m + "uk", "up_v": m + "uv",
                 "gate": m + "g", "o": m + "o"})
        norms = {"mixer": norm(p + "norm1")}
        feed_forward = None
        if layer.ff is not None:
            feed_forward = PartSpec(
                "gated_mlp", {"hidden_size": width, "intermediate_size": layer.ff, "activation": "gelu_tanh"},
                {"gate": p + "mlp.gate", "up": p + "mlp.up", "down": p + "mlp.down"})
            norms["feed_forward"] = norm(p + "norm2")
        layers.append(LayerSpec(block="post_norm", mixer=mixer, feed_forward=feed_forward, norms=norms))
    sizes = {"vocab_size": cfg.vocab, "hidden_size": width}
    return ModelSpec(
        hidden_size=width,
        vocab_size=cfg.vocab,
        embedding=PartSpec("table", dict(sizes), {"weight": "embed"}),
        layers=layers,
        order=list(range(len(layers))),
        final_norm=norm("final.norm"),
        head=PartSpec("linear", dict(sizes), {"weight": "head"}),
    )


register_architecture("Simetar", SimetarConfig.from_text, describe_simetar, model_types=("simetar",), replace=True)
