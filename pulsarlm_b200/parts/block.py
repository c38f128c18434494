"""Arrangements of norms, mixer and feed-forward around the residual stream.

A block's forward takes the fp32 residual stream `x` and the previous block's
not-yet-added output `delta`, and returns the same pair: the add is done inside
the next norm kernel (one pass over x instead of two).
"""

from __future__ import annotations

import torch

from . import native_layer
from ..kernels import ops
from .basic import NormedDelta, RMSNorm, ScaledPair, settle_pending
from .registry import BuildContext, build_part, register_part
from .spec import LayerSpec


@register_part("block", "pre_norm")
class PreNormBlock:
    """x += mixer(norm_mixer(x)); x += feed_forward(norm_ff(x))
    (pulsarlm-core/src/engine/model/llama.cpp:88-92). Norm names in the
    LayerSpec: "mixer" and "feed_forward". A LayerSpec whose feed_forward is None has
    the first line only."""

    def __init__(self, spec: LayerSpec, ctx: BuildContext):
        self.spec = spec
        self.mixer_norm = build_part("norm", spec.norms["mixer"], ctx)
        self.mixer = build_part("mixer", spec.mixer, ctx)
        self.ff_norm = self.feed_forward = None
        if spec.feed_forward is not None:
            self.ff_norm = build_part("norm", spec.norms["feed_forward"], ctx)
            self.feed_forward = build_part("feed_forward", spec.feed_forward, ctx)
        self._native: bool | None = None  # whether the parts are the ones the native layer call takes

    @classmethod
    def part_specs(cls, spec: LayerSpec):
        """(kind, PartSpec) of every part, so tensor needs can be listed without building."""
        out = [("norm", spec.norms["mixer"]), ("mixer", spec.mixer)]
        if spec.feed_forward is not None:
            out += [("norm", spec.norms["feed_forward"]), ("feed_forward", spec.feed_forward)]
        return out

    def parts(self):
        return [p for p in (self.mixer_norm, self.mixer, self.ff_norm, self.feed_forward) if p is not None]

    def forward(self, x: torch.Tensor, delta: torch.Tensor | None, batch) -> tuple[torch.Tensor, torch.Tensor]:
        # The standard parts in bfloat16: the whole layer from one native call (the same kernels
        # in the same order; see native_layer.py). Anything else: the parts' own calls below.
        if self._native is None:
            self._native = native_layer.eligible(self)
        if self._native:
            done = native_layer.forward(self, x, delta, batch)
            if done is not None:
                return done
        h = self.mixer_norm.forward(x, delta)
        mixed = self.mixer.forward(h, batch)
        if self.feed_forward is None:
            return x, mixed
        h = self.ff_norm.forward(x, mixed)
        return x, self.feed_forward.forward(h, batch)


@register_part("block", "sandwich_norm")
class SandwichNormBlock:
    """Every sublayer is normed before and after, and its normed output enters the
    residual stream scaled:

        x += m * norm_mixer_out(mixer(filter_mixer(norm_mixer(x))))
        x += m * norm_ff_out(feed_forward(filter_ff(norm_ff(x))))

    Norm names in the LayerSpec: "mixer", "mixer_out", "feed_forward", "feed_forward_out".
    `extras` of the LayerSpec: "residual_mult" (m, 1 when absent) and optional PartSpecs
    "mixer_filter" / "feed_forward_filter" of the "filter" registry (e.g. a short
    convolution over time), applied to the sublayer's input. A LayerSpec whose
    feed_forward is None has the first line only. The out-norm of a sublayer is not run
    on its own: its output travels as a NormedDelta and the next norm kernel norms it,
    adds it and norms the sum for the next sublayer in one pass."""

    def __init__(self, spec: LayerSpec, ctx: BuildContext):
        self.spec = spec
        extras = spec.extras or {}
        self.mult = float(extras.get("residual_mult", 1.0))
        self.mixer_norm = build_part("norm", spec.norms["mixer"], ctx)
        self.mixer_out_norm = build_part("norm", spec.norms["mixer_out"], ctx)
        self.mixer = build_part("mixer", spec.mixer, ctx)
        self.mixer_filter = build_part("filter", extras["mixer_filter"], ctx) if extras.get("mixer_filter") else None
        self.feed_forward = self.ff_norm = self.ff_out_norm = self.ff_filter = None
        if spec.feed_forward is not None:
            self.ff_norm = build_part("norm", spec.norms["feed_forward"], ctx)
            self.ff_out_norm = build_part("norm", spec.norms["feed_forward_out"], ctx)
            self.feed_forward = build_part("feed_forward", spec.feed_forward, ctx)
            if extras.get("feed_forward_filter"):
                self.ff_filter = build_part("filter", extras["feed_forward_filter"], ctx)

    @classmethod
    def part_specs(cls, spec: LayerSpec):
        extras = spec.extras or {}
        out = [("norm", spec.norms["mixer"]), ("norm", spec.norms["mixer_out"]), ("mixer", spec.mixer)]
        if extras.get("mixer_filter"):
            out.append(("filter", extras["mixer_filter"]))
        if spec.feed_forward is not None:
            out += [("norm", spec.norms["feed_forward"]), ("norm", spec.norms["feed_forward_out"]),
                    ("feed_forward", spec.feed_forward)]
            if extras.get("feed_forward_filter"):
                out.append(("filter", extras["feed_forward_filter"]))
        return out

    def parts(self):
        return [p for p in (self.mixer_norm, self.mixer_out_norm, self.mixer, self.mixer_filter, self.ff_norm,
                            self.ff_out_norm, self.feed_forward, self.ff_filter) if p is not None]

    def cache_holders(self):
        """The parts that keep something per request, the mixer first."""
        return [self.mixer] + [f for f in (self.mixer_filter, self.ff_filter) if f is not None]

    @staticmethod
    def _input(norm, filt, x, delta, batch):
        """A sublayer's input: the norm (with the pending output added first), then the filter.
        Where the filter can ride along in the norm's kernel (a step of single tokens), one launch."""
        if filt is None:
            return norm.forward(x, delta)
        ride = getattr(filt, "rides_along", None)
        conv = ride(batch) if ride is not None and isinstance(delta, NormedDelta) else None
        if conv is not None:
            return norm.forward(x, delta, conv=conv)
        return filt.forward(norm.forward(x, delta), batch)

    def forward(self, x: torch.Tensor, delta, batch):
        h = self._input(self.mixer_norm, self.mixer_filter, x, delta, batch)
        delta = self.mixer_out_norm.pending(self.mixer.forward(h, batch), self.mult)
        if self.feed_forward is None:
            return x, delta
        h = self._input(self.ff_norm, self.ff_filter, x, delta, batch)
        # A bias on the feed-forward's last projection is added by the kernel that norms its output.
        bias = getattr(self.feed_forward, "down_bias", None)
        if bias is not None:
            y = self.feed_forward.forward(h, batch, bias_taken=True)
        else:
            y = self.feed_forward.forward(h, batch)
        return x, self.ff_out_norm.pending(y, self.mult, bias)


@register_part("block", "post_norm")
class PostNormBlock:
    """The sublayers read the residual stream itself; the norm sits on what they return:

        x += norm_mixer(mixer(x))
        x += norm_ff(feed_forward(x))

    Norm names in the LayerSpec: "mixer" and "feed_forward"; a LayerSpec whose feed_forward
    is None has the first line only. The norms must know `pending(y)` (a sublayer's output
    that is normed on its way into the stream): the kernel that makes the next reader's
    input (the stream rounded to the engine's dtype) norms and adds the pending output in
    the same pass. In float32 the sublayers read the stream in place."""

    def __init__(self, spec: LayerSpec, ctx: BuildContext):
        self.spec = spec
        self.ctx = ctx
        self.mixer_norm = build_part("norm", spec.norms["mixer"], ctx)
        self.mixer = build_part("mixer", spec.mixer, ctx)
        self.feed_forward = self.ff_norm = None
        if spec.feed_forward is not None:
            self.ff_norm = build_part("norm", spec.norms["feed_forward"], ctx)
            self.feed_forward = build_part("feed_forward", spec.feed_forward, ctx)
        for norm in (self.mixer_norm, self.ff_norm):
            if norm is not None and not hasattr(norm, "pending"):
                raise ValueError(f"post_norm: the norm {norm.spec.kind!r} cannot be applied to a pending output")

    @classmethod
    def part_specs(cls, spec: LayerSpec):
        out = [("norm", spec.norms["mixer"]), ("mixer", spec.mixer)]
        if spec.feed_forward is not None:
            out += [("norm", spec.norms["feed_forward"]), ("feed_forward", spec.feed_forward)]
        return out

    def parts(self):
        return [p for p in (self.mixer_norm, self.mixer, self.ff_norm, self.feed_forward) if p is not None]

    def cache_holders(self):
        """The mixer and whatever else it keeps per request (`state_holders()`)."""
        return [self.mixer] + list(getattr(self.mixer, "state_holders", lambda: [])())

    def _read(self, x: torch.Tensor, delta) -> torch.Tensor:
        """A sublayer's input: the stream with whatever is pending added first."""
        if self.ctx.dtype == torch.float32:
            settle_pending(x, delta)
            return x
        return self.mixer_norm.stream(x, delta)

    def forward(self, x: torch.Tensor, delta, batch):
        delta = self.mixer_norm.pending(self.mixer.forward(self._read(x, delta), batch))
        if self.feed_forward is None:
            return x, delta
        return x, self.ff_norm.pending(self.feed_forward.forward(self._read(x, delta), batch))


@register_part("block", "parallel")
class ParallelBlock:
    """Both sublayers read the same stream, each through a norm of its own, and their
    outputs enter it together, each scaled per channel:

        x += scale_mixer * mixer(norm_mixer(x)) + scale_ff * feed_forward(norm_ff(x))

    Norm names in the LayerSpec: "mixer" and "feed_forward" (the latter only where the layer
    has a feed-forward). `extras`: "mixer_scale" / "feed_forward_scale", checkpoint names of
    the per-channel scales [hidden] (absent: unscaled). The sum is not formed here: the
    outputs travel as a ScaledPair and the next block's norm kernel scales them, adds them
    into the fp32 stream and writes both of its norms in one pass."""

    def __init__(self, spec: LayerSpec, ctx: BuildContext):
        self.spec = spec
        self.ctx = ctx
        extras = spec.extras or {}
        self.mixer_norm = build_part("norm", spec.norms["mixer"], ctx)
        self.mixer = build_part("mixer", spec.mixer, ctx)
        self.feed_forward = self.ff_norm = None
        if spec.feed_forward is not None:
            self.ff_norm = build_part("norm", spec.norms["feed_forward"], ctx)
            self.feed_forward = build_part("feed_forward", spec.feed_forward, ctx)
        self.scales = _LayerScales(extras.get("mixer_scale"),
                                   extras.get("feed_forward_scale") if spec.feed_forward is not None else None,
                                   int(spec.norms["mixer"].params["hidden_size"]))

    @classmethod
    def part_specs(cls, spec: LayerSpec):
        extras = spec.extras or {}
        out = [("norm", spec.norms["mixer"]), ("mixer", spec.mixer)]
        if spec.feed_forward is not None:
            out += [("norm", spec.norms["feed_forward"]), ("feed_forward", spec.feed_forward)]
        names = {"mixer": extras.get("mixer_scale"),
                 "feed_forward": extras.get("feed_forward_scale") if spec.feed_forward is not None else None}
        out.append(("block", _scales_spec(names, int(spec.norms["mixer"].params["hidden_size"]))))
        return out

    def parts(self):
        return [p for p in (self.mixer_norm, self.mixer, self.ff_norm, self.feed_forward, self.scales) if p is not None]

    def cache_holders(self):
        """The parts that keep something per request: the mixer, then what it names besides."""
        return [self.mixer] + list(getattr(self.mixer, "state_holders", lambda: [])())

    def _fused(self) -> bool:
        """Whether both norms are the plain RMS norm with one eps: one kernel then writes both."""
        return (type(self.mixer_norm) is RMSNorm and (self.ff_norm is None or (
            type(self.ff_norm) is RMSNorm and self.ff_norm.eps == self.mixer_norm.eps)))

    def forward(self, x: torch.Tensor, delta, batch):
        tokens, hidden = x.shape
        if self._fused() and (delta is None or isinstance(delta, ScaledPair)):
            dtype, device = self.ctx.dtype, x.device
            h1 = torch.empty((tokens, hidden), dtype=dtype, device=device)
            h2 = torch.empty((tokens, hidden), dtype=dtype, device=device) if self.ff_norm is not None else None
            d = delta or ScaledPair(None, None)
            ops.pair_residual_norm(x, d.y1, d.s1, d.y2, d.s2, d.also, self.mixer_norm.weight_f32(),
                                   self.ff_norm.weight_f32() if self.ff_norm is not None else None, h1, h2,
                                   self.mixer_norm.eps)
        else:
            h1 = self.mixer_norm.forward(x, delta)
            h2 = self.ff_norm.forward(x, None) if self.ff_norm is not None else None
        y1 = self.mixer.forward(h1, batch)
        y2 = self.feed_forward.forward(h2, batch) if self.feed_forward is not None else None
        return x, ScaledPair(y1, self.scales.mixer, y2, self.scales.feed_forward)


def _scales_spec(names: dict, hidden: int):
    from .spec import PartSpec
    return PartSpec("layer_scales", {"hidden_size": hidden}, dict(names))


@register_part("block", "layer_scales")
class _LayerScales:
    """The per-channel scales of a parallel block's two outputs (fp32 [hidden] each), as a
    part of its own so that the loader hears of the tensors. tensors: mixer, feed_forward
    (either may be None)."""

    def __init__(self, mixer_name, ff_name, hidden: int):
        self.names = {"mixer": mixer_name, "feed_forward": ff_name}
        self.hidden = hidden
        self.mixer: torch.Tensor | None = None
        self.feed_forward: torch.Tensor | None = None

    @classmethod
    def part_specs(cls, spec):
        return []

    @classmethod
    def tensor_needs(cls, spec):
        from .spec import TensorNeed
        hidden = int(spec.params["hidden_size"])
        return {name: TensorNeed((hidden,), role="vector") for name in spec.tensors.values() if name}

    def load(self, tensors) -> None:
        for role, name in self.names.items():
            if name:
                setattr(self, role, tensors[name].float().contiguous())
