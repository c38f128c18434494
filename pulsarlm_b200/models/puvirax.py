"""The Puvirax decoder, described as data and registered by name.

A layer: x += mixer(norm1(x)), then, where the layer has a feed-forward, x += ff(norm2(x)),
both norms RMS norms with weights. The embedding is the token's row of `embed` plus a row of
`bigram` chosen by a hash of (token before, token); the model's last norm is `final.norm` and
the head is `embed` again, its logits scaled. Per layer `l<i>.`: norm1, norm2, mix.{q, k, v, o,
q.norm, k.norm, rel, vmix, g}, mlp.{up, down} or mlp.{router, correction, e<j>.up, e<j>.down,
shared.up, shared.down}.
"""

from __future__ import annotations

from ..config.puvirax import GROUP_TOP, PuviraxConfig
from ..config.registry import register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec

VALUE_STREAM = "first_values"   # the name under which the first mixing layer's values travel through a step


def describe_puvirax(cfg: PuviraxConfig) -> ModelSpec:
    width = cfg.width

    def norm(name: str) -> PartSpec:
        return PartSpec("rmsnorm", {"hidden_size": width, "eps": cfg.norm_eps}, {"weight": name})

    layers = []
    first_mixing = next((i for i, layer in enumerate(cfg.layers) if layer.v_mix), None)
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        m = p + "mix."
        names = {"q": m + "q", "k": m + "k", "v": m + "v", "o": m + "o"}
        params = {"hidden_size": width, "n_heads": layer.heads, "n_kv_heads": layer.kv_heads, "head_dim": layer.dim,
                  "value_dim": layer.value_dim, "scale": layer.scale, "window": layer.window, "norm_eps": cfg.norm_eps,
                  # (softmax weights enter the value product rounded once, as in the plain kernels: measured on this
                  # design, the second bfloat16 term changes the logits' error by less than the runs differ)
                  "split_weights": False, "position": PartSpec("none")}
        if layer.type == "attention":
            params["qk_norm"] = "unit_after"
            params["head_gate"] = True
            names["gate"] = m + "g"
            if layer.rot_base is not None and layer.rot_dims > 0:
                bands = None
                if layer.scaling is not None:
                    bands = {"factor": layer.scaling.factor, "low_freq_factor": layer.scaling.low,
                             "high_freq_factor": layer.scaling.high,
                             "original_max_position_embeddings": layer.scaling.original}
                # (the frequencies' exponent is 2i / rot.dims: the rotated part is a head of its own size)
                params["position"] = PartSpec("rope", {"theta": layer.rot_base, "head_dim": layer.rot_dims,
                                                       "rotary_dim": layer.rot_dims, "llama3": bands})
        else:
            params["qk_norm"] = "per_head" if layer.type == "attention_2" else "whole"
            params["bias_far"] = layer.bias_max
            params["bias_rows"] = layer.bias_rows
            names.update(q_norm=m + "q.norm", k_norm=m + "k.norm", distance_bias=m + "rel")
        names["value_mix"] = m + "vmix"   # (read by the layers that mix; the others may store one and ignore it)
        if layer.v_mix:
            params["value_stream"] = VALUE_STREAM
            params["value_mix"] = "source" if i == first_mixing else "mix"
        if layer.mlp is None:
            names["ignored"] = {p + "norm2": (width,)}  # (a layer without feed-forward may still store its norm)
        mixer = PartSpec("normed_attention", params, names)
        norms = {"mixer": norm(p + "norm1")}
        feed_forward = None
        if layer.mlp is not None:
            norms["feed_forward"] = norm(p + "norm2")
            f = p + "mlp."
            if layer.mlp.kind == "dense":
                feed_forward = PartSpec("mlp", {"hidden_size": width, "intermediate_size": layer.mlp.ff,
                                                "activation": "relu2", "bias": False},
                                        {"up": f + "up", "down": f + "down"})
            else:
                mlp = layer.mlp
                names = {"router": f + "router", "correction": f + "correction", "expert_up": f + "e{e}.up",
                         "expert_down": f + "e{e}.down"}
                if mlp.shared_ff is not None:
                    names.update(shared_up=f + "shared.up", shared_down=f + "shared.down")
                feed_forward = PartSpec(
                    "moe", {"hidden_size": width, "expert_size": mlp.ff, "n_experts": mlp.experts, "top": mlp.top,
                            "groups": mlp.groups, "keep_groups": mlp.keep_groups, "shared_size": mlp.shared_ff,
                            "scores": "sigmoid", "group_top": GROUP_TOP, "renormalise": False, "expert": "relu2"},
                    names)
        layers.append(LayerSpec(block="pre_norm", mixer=mixer, feed_forward=feed_forward, norms=norms))
    sizes = {"vocab_size": cfg.vocab, "hidden_size": width}
    if cfg.pairs is not None:
        embedding = PartSpec("pair_hash_table", {**sizes, "buckets": cfg.pairs.buckets, "mul_prev": cfg.pairs.mul_prev,
                                                 "mul_cur": cfg.pairs.mul_cur}, {"weight": "embed", "pairs": "bigram"})
    else:
        embedding = PartSpec("table", dict(sizes), {"weight": "embed"})
    return ModelSpec(
        hidden_size=width,
        vocab_size=cfg.vocab,
        embedding=embedding,
        layers=layers,
        order=list(range(len(layers))),
        final_norm=norm("final.norm"),
        head=PartSpec("linear", {**sizes, "scale": cfg.logit_scale}, {"weight": None}),
    )


register_architecture("Puvirax", PuviraxConfig.from_text, describe_puvirax, model_types=("puvirax",), replace=True)
