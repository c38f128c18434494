"""PuviraxConfig: the typed configuration of the Puvirax decoder.

Puvirax lists its layers one by one. Every layer is a pre-norm block (RMS norms) whose mixer
is grouped-query softmax attention in one of three forms:

* `attention`: rotate-half rotation of part of every head with frequencies scaled by
  wavelength bands, then q and k divided by their root mean square per head (no weights),
  causal, an output gate per head;
* `attention_2`: an RMS norm with weights on every head of q and k (one weight row shared by
  the heads), no rotation, a learned bias by distance and head on the scaled scores, a sliding
  window;
* `attention_3`: an RMS norm with weights over the whole q projection and over the whole k
  projection, no rotation, the same kind of bias, causal.

Key and value sizes may differ. A layer with `v_mix` blends its values with those the first
such layer made of the same token. The feed-forward is W_down relu(W_up h)^2, dense or as
routed experts (sigmoid scores, a correction only the choice sees, groups ranked by the sum
of their two best choice scores, weights not renormalised) beside a shared expert. The
embedding adds a row of a second table chosen by a hash of (token before, token); the head is
the embedding table, its logits times `logit_scale`.
"""

from __future__ import annotations

import dataclasses

from .base import ConfigError, read_field, require_positive

MIXERS = ("attention", "attention_2", "attention_3")
GROUP_TOP = 2   # a group of experts is ranked by the sum of this many of its largest choice scores


@dataclasses.dataclass(frozen=True)
class BandScaling:
    """Frequencies scaled by wavelength bands: `rot.scaling`."""

    factor: float
    low: float
    high: float
    original: float


@dataclasses.dataclass(frozen=True)
class PuviraxFeedForward:
    """`mlp` of a layer. kind "dense": `ff`. kind "moe": `ff` is an expert's size; `experts`, `top`,
    `groups` and `keep_groups` the router's; `shared_ff` the shared expert's size (None: none)."""

    kind: str
    ff: int
    experts: int = 0
    top: int = 0
    groups: int = 1
    keep_groups: int = 1
    shared_ff: int | None = None


@dataclasses.dataclass(frozen=True)
class PuviraxLayer:
    """One entry of config.json's `layers`. Fields a mixer kind does not have are None."""

    type: str
    heads: int
    kv_heads: int
    dim: int
    value_dim: int
    scale: float
    v_mix: bool
    window: int | None                  # None: every earlier token
    rot_base: float | None = None       # attention
    rot_dims: int = 0
    scaling: BandScaling | None = None
    bias_max: float | None = None       # attention_2, attention_3: the distance at which the bias table ends
    bias_rows: int | None = None        # rows of the bias table, where the configuration names them (optional
                                        # key `bias_rows`: else only the stored tensor gives them)
    mlp: PuviraxFeedForward | None = None


@dataclasses.dataclass(frozen=True)
class PairTable:
    """`embedding.bigram`: rows of the second table and the hash's two multipliers."""

    buckets: int
    mul_prev: int
    mul_cur: int


def _feed_forward(entry: dict, i: int) -> PuviraxFeedForward | None:
    mlp = entry.get("mlp")
    if mlp is None:
        return None
    if not isinstance(mlp, dict):
        raise ConfigError(f"config.json: layers[{i}].mlp must be an object or null")
    kind = read_field(mlp, "kind", str, "dense")
    if kind == "dense":
        ff = read_field(mlp, "ff", int)
        require_positive(f"layers[{i}].mlp.ff", ff)
        return PuviraxFeedForward("dense", ff)
    if kind != "moe":
        raise ConfigError(f"config.json: layers[{i}].mlp.kind {kind!r} is unsupported (supported: 'dense', 'moe')")
    ff = read_field(read_field(mlp, "expert", dict), "ff", int)
    router = read_field(mlp, "router", dict)
    experts, top = read_field(router, "experts", int), read_field(router, "top", int)
    for name, value in (("expert.ff", ff), ("router.experts", experts), ("router.top", top)):
        require_positive(f"layers[{i}].mlp.{name}", value)
    groups = router.get("groups")
    count = keep = 1
    if isinstance(groups, dict):
        count = read_field(groups, "count", int)
        keep = read_field(groups, "keep", int, count)
    elif groups is not None:
        raise ConfigError(f"config.json: layers[{i}].mlp.router.groups must be an object or null")
    if count <= 0 or experts % count or not 0 < keep <= count:
        raise ConfigError(f"config.json: layers[{i}].mlp.router: {experts} experts in {count} groups of which "
                          f"{keep} stay")
    if top > keep * (experts // count):
        raise ConfigError(f"config.json: layers[{i}].mlp.router: {top} experts cannot be chosen from {keep} groups "
                          f"of {experts // count}")
    shared = mlp.get("shared")
    shared_ff = None
    if isinstance(shared, dict):
        shared_ff = read_field(shared, "ff", int)
        require_positive(f"layers[{i}].mlp.shared.ff", shared_ff)
    elif shared is not None:
        raise ConfigError(f"config.json: layers[{i}].mlp.shared must be an object or null")
    return PuviraxFeedForward("moe", ff, experts, top, count, keep, shared_ff)


def _rot(mixer: dict, i: int, dim: int):
    rot = mixer.get("rot")
    if rot is None:
        return None, 0, None
    if not isinstance(rot, dict):
        raise ConfigError(f"config.json: layers[{i}].mixer.rot must be an object or null")
    base, dims = read_field(rot, "base", float), read_field(rot, "dims", int)
    if dims < 0 or dims % 2 or dims > dim:
        raise ConfigError(f"config.json: layers[{i}].mixer.rot.dims must be even, not negative and at most dim "
                          f"({dim}), got {dims}")
    s = rot.get("scaling")
    scaling = None
    if isinstance(s, dict):
        scaling = BandScaling(read_field(s, "factor", float), read_field(s, "low", float),
                              read_field(s, "high", float), read_field(s, "original", float))
    elif s is not None:
        raise ConfigError(f"config.json: layers[{i}].mixer.rot.scaling must be an object or null")
    return base, dims, scaling


@dataclasses.dataclass(frozen=True)
class PuviraxConfig:
    architecture: str
    vocab: int
    width: int
    norm_eps: float
    logit_scale: float
    pairs: PairTable | None
    layers: tuple[PuviraxLayer, ...]

    @staticmethod
    def from_text(text: dict) -> "PuviraxConfig":
        layers_text = read_field(text, "layers", list)
        if not layers_text:
            raise ConfigError("config.json: 'layers' must list at least one layer")
        layers: list[PuviraxLayer] = []
        for i, entry in enumerate(layers_text):
            if not isinstance(entry, dict):
                raise ConfigError(f"config.json: layers[{i}] must be an object")
            kind = read_field(entry, "type", str)
            if kind not in MIXERS:
                raise ConfigError(f"config.json: layers[{i}].type {kind!r} is unknown (known: {', '.join(MIXERS)})")
            mixer = read_field(entry, "mixer", dict)
            heads, dim = read_field(mixer, "heads", int), read_field(mixer, "dim", int)
            kv_heads, vdim = read_field(mixer, "kv_heads", int, heads), read_field(mixer, "vdim", int, dim)
            for name, value in (("heads", heads), ("kv_heads", kv_heads), ("dim", dim), ("vdim", vdim)):
                require_positive(f"layers[{i}].mixer.{name}", value)
            if heads % kv_heads:
                raise ConfigError(f"config.json: layers[{i}].mixer: {heads} heads are not a multiple of "
                                  f"{kv_heads} kv_heads")
            mask = mixer.get("mask")
            window = read_field(mask, "size", int) if isinstance(mask, dict) else None
            if window is not None:
                require_positive(f"layers[{i}].mixer.mask.size", window)
            base = scaling = bias_max = bias_rows = None
            dims = 0
            if kind == "attention":
                base, dims, scaling = _rot(mixer, i, dim)
            else:
                bias_max = read_field(mixer, "bias_max", float)
                if bias_max <= 0.0:
                    raise ConfigError(f"config.json: layers[{i}].mixer.bias_max must be positive, got {bias_max}")
                bias_rows = read_field(mixer, "bias_rows", int, None)
                if bias_rows is not None:
                    require_positive(f"layers[{i}].mixer.bias_rows", bias_rows)
            layers.append(PuviraxLayer(kind, heads, kv_heads, dim, vdim, read_field(mixer, "scale", float),
                                       bool(mixer.get("v_mix", False)), window, base, dims, scaling, bias_max,
                                       bias_rows, _feed_forward(entry, i)))
        mixing = [layer for layer in layers if layer.v_mix]
        if any(layer.kv_heads * layer.value_dim != mixing[0].kv_heads * mixing[0].value_dim for layer in mixing):
            raise ConfigError("config.json: layers with v_mix must agree in kv_heads x vdim (they share a token's values)")
        pairs = None
        embedding = text.get("embedding")
        if isinstance(embedding, dict) and isinstance(embedding.get("bigram"), dict):
            b = embedding["bigram"]
            pairs = PairTable(read_field(b, "buckets", int), read_field(b, "mul_prev", int),
                              read_field(b, "mul_cur", int))
            require_positive("embedding.bigram.buckets", pairs.buckets)
        cfg = PuviraxConfig(
            architecture=str(text.get("architecture") or "Puvirax"),
            vocab=read_field(text, "vocab", int),
            width=read_field(text, "width", int),
            norm_eps=read_field(read_field(text, "norm", dict), "eps", float),
            logit_scale=read_field(text, "logit_scale", float, 1.0),
            pairs=pairs,
            layers=tuple(layers),
        )
        require_positive("vocab", cfg.vocab)
        require_positive("width", cfg.width)
        return cfg

    def to_text(self) -> dict:
        """A config.json that `from_text` reads back to an equal configuration."""
        layers = []
        for layer in self.layers:
            mixer: dict = {"heads": layer.heads, "kv_heads": layer.kv_heads, "dim": layer.dim, "vdim": layer.value_dim,
                           "scale": layer.scale, "v_mix": layer.v_mix}
            if layer.window is not None:
                mixer["mask"] = {"size": layer.window}
            if layer.rot_base is not None:
                mixer["rot"] = {"base": layer.rot_base, "dims": layer.rot_dims}
                if layer.scaling is not None:
                    mixer["rot"]["scaling"] = dataclasses.asdict(layer.scaling)
            if layer.bias_max is not None:
                mixer["bias_max"] = layer.bias_max
            if layer.bias_rows is not None:
                mixer["bias_rows"] = layer.bias_rows
            mlp = None
            if layer.mlp is not None and layer.mlp.kind == "dense":
                mlp = {"kind": "dense", "ff": layer.mlp.ff}
            elif layer.mlp is not None:
                m = layer.mlp
                mlp = {"kind": "moe", "expert": {"ff": m.ff},
                       "router": {"experts": m.experts, "top": m.top,
                                  "groups": {"count": m.groups, "keep": m.keep_groups}}}
                if m.shared_ff is not None:
                    mlp["shared"] = {"ff": m.shared_ff}
            layers.append({"type": layer.type, "mixer": mixer, "mlp": mlp})
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
               "norm": {"eps": self.norm_eps}, "logit_scale": self.logit_scale, "layers": layers}
        if self.pairs is not None:
            out["embedding"] = {"bigram": dataclasses.asdict(self.pairs)}
        return out
