"""Norm, position encoding, embedding, output head and the gated feed-forward.

Each takes its sizes and constants from its PartSpec and its tensors by the
names the spec gives; none knows the model around it.
"""

from __future__ import annotations

import dataclasses
import math

import torch

from ..kernels import ops
from .linear import activated_linear, gated_feed_forward, linear
from .registry import BuildContext, Part, register_part
from .spec import PartSpec, StateNeed, TensorNeed


@dataclasses.dataclass
class NormedDelta:
    """A sublayer's output that enters the residual stream normed and scaled:
    x += mult * rmsnorm(y + bias) * weight (weight fp32, eps the norm's). A block hands
    it on in the place of a plain delta; the next norm's kernel does the norm, the add
    and its own norm in one pass."""

    y: torch.Tensor
    weight: torch.Tensor
    eps: float
    mult: float = 1.0
    bias: torch.Tensor | None = None


@dataclasses.dataclass
class ScaledPair:
    """The outputs of two sublayers that read the same stream, each scaled per channel on
    its way in: x += s1 * y1 + s2 * y2 (+ also). y2 / s2 are None for a layer with one
    sublayer; s1 / s2 None means unscaled; `also` is an fp32 [T, H] row added too. A block
    hands it on in the place of a plain delta; the next norm's kernel does the adds and its
    own norm in one pass (ops.pair_residual_norm)."""

    y1: torch.Tensor
    s1: torch.Tensor | None
    y2: torch.Tensor | None = None
    s2: torch.Tensor | None = None
    also: torch.Tensor | None = None

    def with_also(self, rows: torch.Tensor) -> "ScaledPair":
        if self.also is not None:
            rows = self.also + rows
        return dataclasses.replace(self, also=rows)


@register_part("norm", "rmsnorm")
class RMSNorm(Part):
    """h = v * rsqrt(mean(v^2) + eps) * weight over the fp32 residual stream, with
    the pending layer output added first (v = x + delta, x updated in place; a
    NormedDelta is normed and scaled on its way in, a ScaledPair scaled and added).
    params: hidden_size, eps, unit_offset (optional: the stored weight is kept around
    zero and the scale is 1 + weight, formed in fp32). tensors: weight [hidden_size].
    Formula: pulsarlm-core/src/kernels/rmsnorm.cu:29-49."""

    def __init__(self, spec: PartSpec, ctx: BuildContext):
        super().__init__(spec, ctx)
        self.hidden = int(self.param("hidden_size"))
        self.eps = float(self.param("eps"))
        self.unit_offset = bool(spec.params.get("unit_offset", False))
        self.weight: torch.Tensor | None = None

    @classmethod
    def tensor_needs(cls, spec: PartSpec) -> dict[str, TensorNeed]:
        role = "offset" if spec.params.get("unit_offset") else "vector"
        return {spec.tensors["weight"]: TensorNeed((int(spec.params["hidden_size"]),), role=role)}

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        self.weight = tensors[self.spec.tensors["weight"]].contiguous()
        self._weight_f32: torch.Tensor | None = None
        if self.unit_offset:
            self.weight = self._weight_f32 = (self.weight.float() + 1.0).contiguous()

    def weight_f32(self) -> torch.Tensor:
        if self._weight_f32 is None:
            self._weight_f32 = self.weight.float().contiguous()
        return self._weight_f32

    def forward(self, x: torch.Tensor, delta: "torch.Tensor | NormedDelta | None" = None,
                rows: torch.Tensor | None = None, conv: tuple | None = None) -> torch.Tensor:
        """conv: see ops.add_normed_rmsnorm (only with a NormedDelta; the caller checks that the
        step's entries bring one token each)."""
        n = rows.numel() if rows is not None else x.shape[0]
        out = torch.empty((n, self.hidden), dtype=self.ctx.dtype, device=x.device)
        if isinstance(delta, ScaledPair):
            if conv is not None:
                raise ValueError("rmsnorm: a filter cannot ride along with a pair of scaled outputs")
            ops.pair_residual_norm(x, delta.y1, delta.s1, delta.y2, delta.s2, delta.also, self.weight_f32(), None,
                                   out, None, self.eps, rows)
        elif isinstance(delta, NormedDelta):
            ops.add_normed_rmsnorm(x, delta.y, delta.weight, delta.mult, delta.eps, self.weight_f32(), self.eps, out,
                                   rows, delta.bias, conv)
        else:
            ops.add_rmsnorm(x, delta, self.weight, self.eps, out, rows)
        return out

    def pending(self, y: torch.Tensor, mult: float = 1.0, bias: torch.Tensor | None = None) -> NormedDelta:
        """`y` as a residual contribution normed by this norm: mult * rmsnorm(y + bias) * weight."""
        return NormedDelta(y, self.weight_f32(), self.eps, mult, bias)


@dataclasses.dataclass
class LayerNormedDelta:
    """A sublayer's output that enters the residual stream layer-normed:
    x += (y - mean(y)) / sqrt(var(y) + eps) * weight + bias (weight and bias fp32). A block
    hands it on in the place of a plain delta; the kernel that next reads the stream (the
    cast for the next sublayer, or the model's last norm) norms and adds it in the same pass."""

    y: torch.Tensor
    weight: torch.Tensor
    bias: torch.Tensor
    eps: float


def settle_pending(x: torch.Tensor, delta) -> None:
    """Adds whatever is pending into the fp32 stream `x` now, for a reader that cannot fold the
    add into its own kernel."""
    if delta is None:
        return
    if isinstance(delta, LayerNormedDelta):
        ops.add_layernorm(x, delta.y, delta.weight, delta.bias, delta.eps, None)
    elif isinstance(delta, NormedDelta):
        ops.add_normed_rmsnorm(x, delta.y, delta.weight, delta.mult, delta.eps, delta.weight, delta.eps, None, None,
                               delta.bias)
    elif isinstance(delta, torch.Tensor):
        x.add_(delta)
    else:
        raise TypeError(f"a pending {type(delta).__name__} can only be added by the norm kernel made for it")


@register_part("norm", "layernorm")
class LayerNorm(Part):
    """h = (v - mean(v)) / sqrt(var(v) + eps) * weight + bias over the fp32 residual stream,
    var the mean of the squared deviations, with whatever is pending added first (v = x +
    delta, x updated in place). `pending(y)` hands a sublayer's output on to be normed by this
    norm on its way into the stream. params: hidden_size, eps. tensors: weight, bias
    [hidden_size] (kept in float32)."""

    def __init__(self, spec: PartSpec, ctx: BuildContext):
        super().__init__(spec, ctx)
        self.hidden = int(self.param("hidden_size"))
        self.eps = float(self.param("eps"))
        self.weight: torch.Tensor | None = None
        self.bias: torch.Tensor | None = None

    @classmethod
    def tensor_needs(cls, spec: PartSpec) -> dict[str, TensorNeed]:
        hidden = int(spec.params["hidden_size"])
        return {spec.tensors["weight"]: TensorNeed((hidden,), role="vector"),
                spec.tensors["bias"]: TensorNeed((hidden,), role="offset")}

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        self.weight = tensors[self.spec.tensors["weight"]].float().contiguous()
        self.bias = tensors[self.spec.tensors["bias"]].float().contiguous()

    def forward(self, x: torch.Tensor, delta=None, rows: torch.Tensor | None = None) -> torch.Tensor:
        n = rows.numel() if rows is not None else x.shape[0]
        out = torch.empty((n, self.hidden), dtype=self.ctx.dtype, device=x.device)
        if isinstance(delta, LayerNormedDelta):
            ops.add_layernorm(x, delta.y, delta.weight, delta.bias, delta.eps, out, self.weight, self.bias, self.eps,
                              rows)
        else:
            settle_pending(x, delta)
            ops.add_layernorm(x, None, None, None, 0.0, out, self.weight, self.bias, self.eps, rows)
        return out

    def pending(self, y: torch.Tensor) -> LayerNormedDelta:
        return LayerNormedDelta(y, self.weight, self.bias, self.eps)

    def stream(self, x: torch.Tensor, delta=None) -> torch.Tensor:
        """The stream itself (not normed) in the engine's dtype, with whatever is pending added
        first: the input of a sublayer that reads the stream as it is."""
        out = torch.empty(x.shape, dtype=self.ctx.dtype, device=x.device)
        if isinstance(delta, LayerNormedDelta):
            ops.add_layernorm(x, delta.y, delta.weight, delta.bias, delta.eps, out)
        else:
            settle_pending(x, delta)
            ops.add_layernorm(x, None, None, None, 0.0, out)
        return out


def rope_inverse_frequencies(theta: float, head_dim: int, rotary_dim: int, llama3: dict | None) -> list[float]:
    """Radians per position for each rotated pair, in Python floats (fp64).

    f_j = theta^(-2j / head_dim); llama3 scaling by wavelength bands as in
    pulsarlm-core/src/kernels/rope.cpp:31-53.
    """
    out = []
    for pair in range(rotary_dim // 2):
        f = theta ** (-2.0 * pair / head_dim)
        if llama3 is not None:
            wavelength = 2.0 * math.pi / f
            original = float(llama3["original_max_position_embeddings"])
            low, high, factor = float(llama3["low_freq_factor"]), float(llama3["high_freq_factor"]), float(
                llama3["factor"])
            if wavelength < original / high:
                pass
            elif wavelength > original / low:
                f = f / factor
            elif high != low:
                smooth = (original / wavelength - low) / (high - low)
                f = (1.0 - smooth) * f / factor + smooth * f
        out.append(f)
    return out


def ramped_frequencies(theta: float, rotary_dim: int, ramp: dict) -> tuple[list[float], float]:
    """Radians per position for each rotated pair when scaled and unscaled frequencies are
    blended along a ramp over the pair index (the scaling known as YaRN), and the amplitude
    that multiplies cos and sin. With f_i = theta^(-2i / d) and index(t) = d ln(original /
    (2 pi t)) / (2 ln theta): lo = max(floor(index(fast)), 0), hi = min(ceil(index(slow)), d - 1),
    r_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1); the frequency is r_i f_i / factor +
    (1 - r_i) f_i and the amplitude 0.1 ln(factor) + 1. `ramp`: factor, original, fast, slow."""
    factor, original = float(ramp["factor"]), float(ramp["original"])

    def index(turns: float) -> float:
        return rotary_dim * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(theta))

    lo = max(math.floor(index(float(ramp["fast"]))), 0)
    hi = min(math.ceil(index(float(ramp["slow"]))), rotary_dim - 1)
    out = []
    for pair in range(rotary_dim // 2):
        f = theta ** (-2.0 * pair / rotary_dim)
        r = min(max((pair - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(f / factor * r + f * (1.0 - r))
    return out, 0.1 * math.log(factor) + 1.0


@register_part("position", "rope")
class Rope(Part):
    """Rotate-half rotary encoding. params: theta, head_dim, rotary_dim (even,
    <= head_dim; pairs are (j, j + rotary_dim / 2), dims past rotary_dim pass
    through), llama3 (None or the four scaling numbers), ramp (None or the four numbers of
    `ramped_frequencies`, which also sets `amplitude`, the number cos and sin are multiplied
    by; the frequencies' exponent is then 2j / rotary_dim). No tensors."""

    def __init__(self, spec: PartSpec, ctx: BuildContext):
        super().__init__(spec, ctx)
        self.head_dim = int(self.param("head_dim"))
        self.rotary_dim = int(self.param("rotary_dim"))
        self.amplitude = 1.0
        if self.rotary_dim % 2 or not 0 <= self.rotary_dim <= self.head_dim:
            raise ValueError(f"rope: rotary_dim {self.rotary_dim} must be even and at most head_dim {self.head_dim}")
        if spec.params.get("ramp"):
            if spec.params.get("llama3"):
                raise ValueError("rope: llama3 bands and a ramp exclude each other")
            freqs, self.amplitude = ramped_frequencies(float(self.param("theta")), self.rotary_dim, spec.params["ramp"])
        else:
            freqs = rope_inverse_frequencies(float(self.param("theta")), self.head_dim, self.rotary_dim,
                                             spec.params.get("llama3"))
        self.inv_freq = torch.tensor(freqs, dtype=torch.float64, device=ctx.device)

    def table(self) -> tuple[torch.Tensor | None, int]:
        return (self.inv_freq if self.rotary_dim > 0 else None), self.rotary_dim


@register_part("position", "rope_pairs")
class RopePairs(Part):
    """Rotary encoding over neighbouring pairs: within the first `rotary_dim` columns of a
    vector, (2i, 2i + 1) turns by the angle pos * f_i with f_i = theta^(-2i / rotary_dim) /
    factor (`factor`: linear position scaling, 1 when absent); the other columns pass through.
    params: theta, rotary_dim (even), factor (optional), llama3 (optional: the four numbers of
    the scaling by wavelength bands, see `rope_inverse_frequencies`). No tensors. `table()`
    gives the fp64 radians per position and the rotary width; the mixer's kernel decides what
    a vector is."""

    def __init__(self, spec: PartSpec, ctx: BuildContext):
        super().__init__(spec, ctx)
        self.rotary_dim = int(self.param("rotary_dim"))
        if self.rotary_dim % 2 or self.rotary_dim < 0:
            raise ValueError(f"rope_pairs: rotary_dim {self.rotary_dim} must be even and not negative")
        theta = float(self.param("theta"))
        factor = float(spec.params.get("factor") or 1.0)
        freqs = [f / factor for f in rope_inverse_frequencies(theta, max(self.rotary_dim, 1), self.rotary_dim,
                                                              spec.params.get("llama3"))]
        self.inv_freq = torch.tensor(freqs, dtype=torch.float64, device=ctx.device)

    def table(self) -> tuple[torch.Tensor | None, int]:
        return (self.inv_freq if self.rotary_dim > 0 else None), self.rotary_dim


@register_part("position", "none")
class NoPosition(Part):
    """No position encoding: q and k are used as projected."""

    def table(self) -> tuple[torch.Tensor | None, int]:
        return None, 0


@register_part("embedding", "table")
class Embedding(Part):
    """x[t] = weight[token[t]] * scale (pulsarlm-core/src/engine/model/llama.cpp:86 has
    no scale), written as fp32 into the residual stream. params: vocab_size,
    hidden_size, scale (optional, 1 when absent)."""

    def __init__(self, spec: PartSpec, ctx: BuildContext):
        super().__init__(spec, ctx)
        self.vocab = int(self.param("vocab_size"))
        self.hidden = int(self.param("hidden_size"))
        self.scale = float(spec.params.get("scale") or 1.0)
        self.weight: torch.Tensor | None = None

    @classmethod
    def tensor_needs(cls, spec: PartSpec) -> dict[str, TensorNeed]:
        return {spec.tensors["weight"]: TensorNeed((int(spec.params["vocab_size"]), int(spec.params["hidden_size"])))}

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        self.weight = tensors[self.spec.tensors["weight"]].contiguous()

    def forward(self, tokens: torch.Tensor, batch=None) -> torch.Tensor:
        """`batch`: the step (an embedding that adds learned positions or scales by a
        constant of the configuration reads batch.pos); this one uses its status word."""
        x = torch.empty((tokens.numel(), self.hidden), dtype=torch.float32, device=tokens.device)
        ops.embed(self.weight, tokens, x, batch.status if batch is not None else None, self.scale)
        return x


@register_part("embedding", "pair_hash_table")
class PairHashEmbedding(Part):
    """x[t] = weight[token[t]] + pairs[(before * mul_prev + token[t] * mul_cur) mod buckets] in fp32,
    where `before` is the token ahead of token[t] in its sequence; a sequence's first token
    takes the last row of `pairs` (row number `buckets`). The token before a step's first token
    is part of the request's state: one int32 per request slot, which the kernel reads for an
    entry's first row and moves on to the entry's last token. params: vocab_size, hidden_size,
    buckets, mul_prev, mul_cur. tensors: weight [vocab, hidden], pairs [buckets + 1, hidden]."""

    def __init__(self, spec: PartSpec, ctx: BuildContext):
        super().__init__(spec, ctx)
        self.vocab = int(self.param("vocab_size"))
        self.hidden = int(self.param("hidden_size"))
        self.buckets = int(self.param("buckets"))
        self.mul_prev = int(self.param("mul_prev"))
        self.mul_cur = int(self.param("mul_cur"))
        if self.buckets <= 0:
            raise ValueError(f"pair_hash_table: buckets must be positive, got {self.buckets}")
        self.weight: torch.Tensor | None = None
        self.pairs: torch.Tensor | None = None
        self.binding = None

    @classmethod
    def tensor_needs(cls, spec: PartSpec) -> dict[str, TensorNeed]:
        p = spec.params
        return {spec.tensors["weight"]: TensorNeed((int(p["vocab_size"]), int(p["hidden_size"]))),
                spec.tensors["pairs"]: TensorNeed((int(p["buckets"]) + 1, int(p["hidden_size"])))}

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        self.weight = tensors[self.spec.tensors["weight"]].contiguous()
        self.pairs = tensors[self.spec.tensors["pairs"]].contiguous()

    def cache_need(self) -> StateNeed:
        return StateNeed((1,), "int32")

    def bind_cache(self, binding) -> None:
        self.binding = binding

    def captures_state_steps(self) -> bool:
        return True  # (a step of single tokens reads and moves the slots on in one launch, nothing on the host)

    def forward(self, tokens: torch.Tensor, batch=None) -> torch.Tensor:
        if batch is None or self.binding is None:
            raise ValueError("pair_hash_table: the embedding needs the step (positions, entries, state slots)")
        x = torch.empty((tokens.numel(), self.hidden), dtype=torch.float32, device=tokens.device)
        ops.pair_embed(self.weight, self.pairs, tokens, batch.pos, batch.entry, batch.slots, self.binding.states.view(-1),
                       x, self.mul_prev, self.mul_cur, int(batch.n_decode) == tokens.numel(), batch.status)
        return x


@register_part("head", "linear")
class Head(Part):
    """logits = h W^T in fp32, times `scale` where given. params: vocab_size, hidden_size, scale
    (optional, 1 when absent). tensors: weight
    [vocab, hidden], or None for a head tied to the embedding table, which the
    model then hands over with `tie`. The reference ties when the weights hold
    no lm_head.weight (pulsarlm-core/src/engine/model/llama.cpp:31); here
    config.json's tie_word_embeddings decides, and the weights must agree."""

    def __init__(self, spec: PartSpec, ctx: BuildContext):
        super().__init__(spec, ctx)
        self.vocab = int(self.param("vocab_size"))
        self.hidden = int(self.param("hidden_size"))
        self.scale = float(spec.params.get("scale") or 1.0)
        self.weight: torch.Tensor | None = None

    @property
    def tied(self) -> bool:
        return self.spec.tensors.get("weight") is None

    @classmethod
    def tensor_needs(cls, spec: PartSpec) -> dict[str, TensorNeed]:
        name = spec.tensors.get("weight")
        shape = (int(spec.params["vocab_size"]), int(spec.params["hidden_size"]))
        if name is None:
            # A tied checkpoint may still store a copy of the table under the head's
            # name; it is allowed and not read.
            ignored = spec.tensors.get("ignored")
            return {ignored: TensorNeed(shape, role="ignored", optional=True)} if ignored else {}
        return {name: TensorNeed((int(spec.params["vocab_size"]), int(spec.params["hidden_size"])))}

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        if not self.tied:
            self.weight = tensors[self.spec.tensors["weight"]].contiguous()

    def tie(self, table: torch.Tensor) -> None:
        if tuple(table.shape) != (self.vocab, self.hidden):
            raise ValueError(f"head: cannot tie to a table of shape {tuple(table.shape)}")
        self.weight = table

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        logits = linear(h, self.weight, out_dtype=torch.float32)
        if self.scale != 1.0:
            logits.mul_(self.scale)
        return logits


@register_part("feed_forward", "gated_mlp")
class GatedMLP(Part):
    """(act(h Wg^T) * (h Wu^T)) Wd^T with act = SiLU
    (pulsarlm-core/src/engine/model/llama.cpp:91) or the tanh form of GELU. params:
    hidden_size, intermediate_size, activation ("silu", the default, or "gelu_tanh").
    tensors: gate, up [I, H], down [H, I].
    gate and up are stacked into one [2I, H] operand at load."""

    def __init__(self, spec: PartSpec, ctx: BuildContext):
        super().__init__(spec, ctx)
        self.hidden = int(self.param("hidden_size"))
        self.inter = int(self.param("intermediate_size"))
        self.activation = str(spec.params.get("activation") or "silu")
        if self.activation not in ("silu", "gelu_tanh"):
            raise ValueError(f"gated_mlp: unsupported activation {self.activation!r} (supported: 'silu', "
                             f"'gelu_tanh')")
        self.gate_up: torch.Tensor | None = None
        self.down: torch.Tensor | None = None

    @classmethod
    def tensor_needs(cls, spec: PartSpec) -> dict[str, TensorNeed]:
        h, i = int(spec.params["hidden_size"]), int(spec.params["intermediate_size"])
        t = spec.tensors
        return {t["gate"]: TensorNeed((i, h)), t["up"]: TensorNeed((i, h)), t["down"]: TensorNeed((h, i))}

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        t = self.spec.tensors
        self.gate_up = torch.cat([tensors[t["gate"]], tensors[t["up"]]], dim=0).contiguous()
        self.down = tensors[t["down"]].contiguous()

    def forward(self, h: torch.Tensor, batch) -> torch.Tensor:
        return gated_feed_forward(h, self.gate_up, self.down, self.activation)


@register_part("feed_forward", "mlp")
class PlainMLP(Part):
    """act(h Wu^T + bu) Wd^T + bd: an ungated feed-forward. params: hidden_size,
    intermediate_size, activation ("relu2": the square of relu), bias (whether both
    projections have one). tensors: up [I, H], down [H, I], up_bias [I], down_bias [H].
    The down projection's bias is added by `output_bias()`'s taker when the block
    takes it (a norm kernel that follows), else here."""

    def __init__(self, spec: PartSpec, ctx: BuildContext):
        super().__init__(spec, ctx)
        self.hidden = int(self.param("hidden_size"))
        self.inter = int(self.param("intermediate_size"))
        self.activation = str(spec.params.get("activation", "relu2"))
        if self.activation not in ("relu2",):
            raise ValueError(f"mlp: unsupported activation {self.activation!r} (supported: 'relu2')")
        self.has_bias = bool(spec.params.get("bias", False))
        self.up: torch.Tensor | None = None
        self.down: torch.Tensor | None = None
        self.up_bias: torch.Tensor | None = None
        self.down_bias: torch.Tensor | None = None

    @classmethod
    def tensor_needs(cls, spec: PartSpec) -> dict[str, TensorNeed]:
        h, i = int(spec.params["hidden_size"]), int(spec.params["intermediate_size"])
        t = spec.tensors
        needs = {t["up"]: TensorNeed((i, h)), t["down"]: TensorNeed((h, i))}
        if spec.params.get("bias"):
            needs[t["up_bias"]] = TensorNeed((i,), role="offset")
            needs[t["down_bias"]] = TensorNeed((h,), role="offset")
        return needs

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        t = self.spec.tensors
        self.up = tensors[t["up"]].contiguous()
        self.down = tensors[t["down"]].contiguous()
        if self.has_bias:
            self.up_bias = tensors[t["up_bias"]].to(self.ctx.dtype).contiguous()
            self.down_bias = tensors[t["down_bias"]].to(self.ctx.dtype).contiguous()

    def forward(self, h: torch.Tensor, batch, bias_taken: bool = False) -> torch.Tensor:
        """bias_taken: the caller adds `down_bias` itself (inside the kernel that reads the output)."""
        y = activated_linear(linear(h, self.up), self.up_bias, self.activation, self.down)
        if self.down_bias is not None and not bias_taken:
            ops.bias_act(y, self.down_bias, y, "none")
        return y
