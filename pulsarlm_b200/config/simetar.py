"""SimetarConfig: the typed configuration of the Simetar decoder.

Simetar lists its layers one by one. A layer's mixer is either grouped-query attention
whose values are its keys (biased q and k, a short convolution over time on both, a norm
over each whole projection, neighbouring pairs rotated with frequency bands, capped
scores, a sliding window, a softmax with one more in its denominator) or attention over
a cached latent with one rotated key part shared by all heads (rotate-half with a ramp
between scaled and unscaled frequencies), which may read another layer's cache. Both gate
their heads' outputs per element. Layer norms (weight and bias) sit on what a sublayer
returns; the sublayers read the residual stream itself.
"""

from __future__ import annotations

import dataclasses

from .base import ConfigError, read_field, require_positive

MIXERS = ("attention", "latent_attention")


@dataclasses.dataclass(frozen=True)
class BandScaling:
    """Frequencies scaled by wavelength bands: `rot.scaling` of an attention layer."""

    factor: float
    low: float
    high: float
    original: float


@dataclasses.dataclass(frozen=True)
class RampScaling:
    """Frequencies blended along a ramp over the pair index: `rot.scaling` of a latent layer."""

    factor: float
    original: float
    fast: float
    slow: float


@dataclasses.dataclass(frozen=True)
class SimetarLayer:
    """One entry of config.json's `layers`. Fields a mixer kind does not have are None."""

    type: str
    heads: int
    dim: int
    value_dim: int
    scale: float
    rot_base: float
    rot_dims: int
    scaling: BandScaling | RampScaling | None
    ff: int | None                  # None: the layer has no feed-forward
    kv_heads: int | None = None     # attention
    taps: int | None = None
    window: int | None = None       # None: every earlier token
    softcap: float | None = None
    rot_dim: int | None = None      # latent_attention: size of the shared rotated key part
    latent_rank: int | None = None
    kv_from: int | None = None      # the layer whose cached rows this layer reads


def _feed_forward(entry: dict, i: int) -> int | None:
    mlp = entry.get("mlp")
    if mlp is None:
        return None
    if not isinstance(mlp, dict):
        raise ConfigError(f"config.json: layers[{i}].mlp must be an object or null")
    kind = read_field(mlp, "kind", str, "dense")
    if kind != "dense":
        raise ConfigError(f"config.json: layers[{i}].mlp.kind {kind!r} is unsupported (supported: 'dense')")
    ff = read_field(mlp, "ff", int)
    require_positive(f"layers[{i}].mlp.ff", ff)
    return ff


def _rot(mixer: dict, i: int, ramp: bool):
    rot = read_field(mixer, "rot", dict)
    base, dims = read_field(rot, "base", float), read_field(rot, "dims", int)
    if dims < 0 or dims % 2:
        raise ConfigError(f"config.json: layers[{i}].mixer.rot.dims must be even and not negative, got {dims}")
    s = rot.get("scaling")
    scaling = None
    if isinstance(s, dict):
        if ramp:
            scaling = RampScaling(read_field(s, "factor", float), read_field(s, "original", float),
                                  read_field(s, "fast", float), read_field(s, "slow", float))
        else:
            scaling = BandScaling(read_field(s, "factor", float), read_field(s, "low", float),
                                  read_field(s, "high", float), read_field(s, "original", float))
    elif s is not None:
        raise ConfigError(f"config.json: layers[{i}].mixer.rot.scaling must be an object or null")
    return base, dims, scaling


@dataclasses.dataclass(frozen=True)
class SimetarConfig:
    architecture: str
    vocab: int
    width: int
    norm_eps: float
    layers: tuple[SimetarLayer, ...]

    @staticmethod
    def from_text(text: dict) -> "SimetarConfig":
        layers_text = read_field(text, "layers", list)
        if not layers_text:
            raise ConfigError("config.json: 'layers' must list at least one layer")
        layers: list[SimetarLayer] = []
        for i, entry in enumerate(layers_text):
            if not isinstance(entry, dict):
                raise ConfigError(f"config.json: layers[{i}] must be an object")
            kind = read_field(entry, "type", str)
            if kind not in MIXERS:
                raise ConfigError(f"config.json: layers[{i}].type {kind!r} is unknown (known: {', '.join(MIXERS)})")
            mixer = read_field(entry, "mixer", dict)
            ff = _feed_forward(entry, i)
            heads, dim, vdim = (read_field(mixer, k, int) for k in ("heads", "dim", "vdim"))
            for name, value in (("heads", heads), ("dim", dim), ("vdim", vdim)):
                require_positive(f"layers[{i}].mixer.{name}", value)
            scale = read_field(mixer, "scale", float)
            if kind == "attention":
                base, dims, scaling = _rot(mixer, i, ramp=False)
                kv_heads = read_field(mixer, "kv_heads", int, heads)
                require_positive(f"layers[{i}].mixer.kv_heads", kv_heads)
                if heads % kv_heads:
                    raise ConfigError(f"config.json: layers[{i}].mixer: {heads} heads are not a multiple of "
                                      f"{kv_heads} kv_heads")
                if vdim != dim:
                    raise ConfigError(f"config.json: layers[{i}].mixer: the values are the keys, so vdim ({vdim}) "
                                      f"must equal dim ({dim})")
                if dims > dim:
                    raise ConfigError(f"config.json: layers[{i}].mixer.rot.dims {dims} exceeds dim {dim}")
                mask = mixer.get("mask")
                window = read_field(mask, "size", int) if isinstance(mask, dict) else None
                if window is not None:
                    require_positive(f"layers[{i}].mixer.mask.size", window)
                taps = read_field(mixer, "conv", int, None)     # None: no convolution and no taps stored
                if taps is not None:
                    require_positive(f"layers[{i}].mixer.conv", taps)
                softcap = read_field(mixer, "softcap", float, None)
                if softcap is not None and softcap <= 0.0:
                    raise ConfigError(f"config.json: layers[{i}].mixer.softcap must be positive, got {softcap}")
                layers.append(SimetarLayer(kind, heads, dim, vdim, scale, base, dims, scaling, ff, kv_heads=kv_heads,
                                           taps=taps, window=window, softcap=softcap))
            else:
                base, dims, scaling = _rot(mixer, i, ramp=True)
                rot_dim, rank = read_field(mixer, "rot_dim", int), read_field(mixer, "kv_rank", int)
                require_positive(f"layers[{i}].mixer.kv_rank", rank)
                if rot_dim < 0 or rot_dim != dims:
                    raise ConfigError(f"config.json: layers[{i}].mixer: rot.dims ({dims}) must equal rot_dim "
                                      f"({rot_dim})")
                source = read_field(mixer, "kv_from", int, None)
                layer = SimetarLayer(kind, heads, dim, vdim, scale, base, dims, scaling, ff, rot_dim=rot_dim,
                                     latent_rank=rank, kv_from=source)
                if source is not None:
                    if not 0 <= source < i:
                        raise ConfigError(f"config.json: layers[{i}].mixer.kv_from must name an earlier layer, "
                                          f"got {source}")
                    owner = layers[source]
                    if owner.type != "latent_attention" or owner.kv_from is not None:
                        raise ConfigError(f"config.json: layers[{i}].mixer.kv_from names layer {source}, which "
                                          f"caches no latent of its own")
                    same = (owner.latent_rank, owner.rot_dim, owner.rot_base, owner.scaling) == (
                        rank, rot_dim, base, scaling)
                    if not same:
                        raise ConfigError(f"config.json: layers[{i}] reads the rows of layer {source}, whose "
                                          f"kv_rank, rot_dim or rotation differ from its own")
                layers.append(layer)
        norm = read_field(text, "norm", dict)
        cfg = SimetarConfig(
            architecture=str(text.get("architecture") or "Simetar"),
            vocab=read_field(text, "vocab", int),
            width=read_field(text, "width", int),
            norm_eps=read_field(norm, "eps", float),
            layers=tuple(layers),
        )
        require_positive("vocab", cfg.vocab)
        require_positive("width", cfg.width)
        return cfg

    def to_text(self) -> dict:
        """A config.json that `from_text` reads back to an equal configuration."""
        layers = []
        for layer in self.layers:
            rot: dict = {"base": layer.rot_base, "dims": layer.rot_dims}
            if layer.scaling is not None:
                rot["scaling"] = dataclasses.asdict(layer.scaling)
            mixer: dict = {"heads": layer.heads, "dim": layer.dim, "vdim": layer.value_dim, "scale": layer.scale,
                           "rot": rot}
            if layer.type == "attention":
                mixer.update(kv_heads=layer.kv_heads)
                if layer.taps is not None:
                    mixer["conv"] = layer.taps
                if layer.window is not None:
                    mixer["mask"] = {"size": layer.window}
                if layer.softcap is not None:
                    mixer["softcap"] = layer.softcap
            else:
                mixer.update(rot_dim=layer.rot_dim, kv_rank=layer.latent_rank)
                if layer.kv_from is not None:
                    mixer["kv_from"] = layer.kv_from
            layers.append({"type": layer.type, "mixer": mixer,
                           "mlp": None if layer.ff is None else {"kind": "dense", "ff": layer.ff}})
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "norm": {"eps": self.norm_eps}, "layers": layers}
