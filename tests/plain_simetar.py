"""A plain, slow implementation of the Simetar decoder in float64 torch on the CPU, one
function per mechanism, written from the architecture's equations. It shares no code
with the engine: whole sequences at once, no cache, no pages, no state slots.

Notation: x [T, W] the residual stream, h a sublayer's input (the stream itself: this
design norms what a sublayer returns, not what it reads), weights by their checkpoint
names ([out, in], applied as W h). `forward(..., rounding=torch.bfloat16)` rounds where
a bfloat16 engine stores a tensor (projections, cached rows, sublayer outputs), so that
the comparison with such an engine sees its arithmetic and not its storage.
"""

from __future__ import annotations

import math

import torch


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def layer_norm(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, eps: float) -> torch.Tensor:
    centred = x - x.mean(-1, keepdim=True)
    return centred / torch.sqrt((centred * centred).mean(-1, keepdim=True) + eps) * weight + bias


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def causal_conv(u: torch.Tensor, taps: torch.Tensor) -> torch.Tensor:
    """u [T, C], taps [C, K]: y[t] = sum_j taps[:, j] * u[t - (K - 1) + j], zeros before the start."""
    n, k = u.shape[0], taps.shape[1]
    padded = torch.cat([torch.zeros(k - 1, u.shape[1], dtype=u.dtype), u], dim=0)
    return sum(padded[j:j + n] * taps[:, j] for j in range(k))


def banded_frequencies(rot: dict) -> torch.Tensor:
    """f_i = base^(-2i / dims), scaled by wavelength bands: short waves stay, long ones are
    divided by the factor, and those between are blended."""
    dims, base = rot["dims"], float(rot["base"])
    f = base ** (-2.0 * torch.arange(dims // 2, dtype=torch.float64) / dims)
    s = rot.get("scaling")
    if not s:
        return f
    factor, low, high, original = float(s["factor"]), float(s["low"]), float(s["high"]), float(s["original"])
    out = f.clone()
    for i in range(dims // 2):
        wave = 2.0 * math.pi / float(f[i])
        if wave < original / high:
            continue
        if wave > original / low:
            out[i] = f[i] / factor
        else:
            blend = (original / wave - low) / (high - low)
            out[i] = (1.0 - blend) * f[i] / factor + blend * f[i]
    return out


def ramped_frequencies(rot: dict) -> tuple[torch.Tensor, float]:
    """f_i = base^(-2i / dims) blended with f_i / factor along a ramp over the pair index, and
    the number that multiplies both cos and sin."""
    dims, base = rot["dims"], float(rot["base"])
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = base ** (-2.0 * i / dims)
    s = rot.get("scaling")
    if not s:
        return f, 1.0
    factor, original = float(s["factor"]), float(s["original"])

    def turns_to_index(turns: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(turns_to_index(float(s["fast"]))), 0)
    hi = min(math.ceil(turns_to_index(float(s["slow"]))), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_neighbours(x: torch.Tensor, positions: torch.Tensor, freqs: torch.Tensor) -> torch.Tensor:
    """x [T, heads, D]: columns (2i, 2i + 1) turn by positions * freqs[i]; columns past 2 len(freqs) stay."""
    dims = 2 * freqs.numel()
    angle = positions.double()[:, None, None] * freqs[None, None, :]
    c, s = angle.cos(), angle.sin()
    out = x.clone()
    even, odd = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = even * c - odd * s
    out[..., 1:dims:2] = odd * c + even * s
    return out


def rotate_halves(x: torch.Tensor, positions: torch.Tensor, freqs: torch.Tensor, amplitude: float) -> torch.Tensor:
    """x [T, heads, D]: columns (i, i + dims / 2) turn by positions * freqs[i], cos and sin times `amplitude`."""
    half = freqs.numel()
    angle = positions.double()[:, None, None] * freqs[None, None, :]
    c, s = angle.cos() * amplitude, angle.sin() * amplitude
    out = x.clone()
    first, second = x[..., :half], x[..., half:2 * half]
    out[..., :half] = first * c - second * s
    out[..., half:2 * half] = second * c + first * s
    return out


def visible(n: int, window: int | None) -> torch.Tensor:
    """[query, key] True where key <= query and, with a window, query - key < window."""
    i = torch.arange(n)
    back = i[:, None] - i[None, :]
    return (back >= 0) & (back < window if window else back >= 0)


def capped_attention_with_sink(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, see: torch.Tensor, scale: float,
                               cap: float | None) -> torch.Tensor:
    """One head: q [N, D], k [M, D], v [M, V], see [N, M]. Scores q . k * scale, squashed to
    cap * tanh(s / cap) when there is a cap; weights exp(s_j) / (1 + sum over the visible exp(s)):
    the 1 is a key with score 0 and no value, so a row's weights add up to less than 1."""
    scores = (q @ k.T) * scale
    if cap:
        scores = cap * torch.tanh(scores / cap)
    weights = torch.exp(scores).masked_fill(~see, 0.0)
    return (weights / (1.0 + weights.sum(-1, keepdim=True))) @ v


def _round(x: torch.Tensor, rounding) -> torch.Tensor:
    return x if rounding is None else x.to(rounding).double()


def conv_attention(mixer: dict, w: dict, p: str, h: torch.Tensor, eps: float, rounding=None) -> torch.Tensor:
    """Grouped-query attention whose values are its keys: q and k with biases, a short causal
    convolution on each, RMS norm over the whole of q and of k, neighbouring pairs rotated,
    capped scores, a window, a softmax with one more in its denominator, a gate per element."""
    heads, kv_heads, dim = mixer["heads"], mixer["kv_heads"], mixer["dim"]
    n = h.shape[0]
    q = _round(h @ w[p + "q"].T + w[p + "q.b"], rounding)
    k = _round(h @ w[p + "k"].T + w[p + "k.b"], rounding)
    gate = _round(h @ w[p + "g"].T, rounding)
    q = causal_conv(q, w[p + "q.conv"])
    k = causal_conv(k, w[p + "k.conv"])
    v = _round(k, rounding).view(n, kv_heads, dim)
    q = (rms(q, eps) * w[p + "q.norm"]).view(n, heads, dim)
    k = (rms(k, eps) * w[p + "k.norm"]).view(n, kv_heads, dim)
    positions = torch.arange(n)
    freqs = banded_frequencies(mixer["rot"])
    q = _round(rotate_neighbours(q, positions, freqs), rounding)
    k = _round(rotate_neighbours(k, positions, freqs), rounding)
    see = visible(n, (mixer.get("mask") or {}).get("size"))
    out = torch.zeros(n, heads, dim, dtype=torch.float64)
    for head in range(heads):
        g = head // (heads // kv_heads)
        out[:, head] = capped_attention_with_sink(q[:, head], k[:, g], v[:, g], see, mixer["scale"], mixer.get("softcap"))
    mixed = _round(_round(out.reshape(n, heads * dim), rounding) * torch.sigmoid(gate), rounding)
    return mixed @ w[p + "o"].T


def latent_rows(mixer: dict, w: dict, p: str, h: torch.Tensor, eps: float, rounding=None):
    """What a latent-attention layer caches per token: the normed latent [T, rank] and the
    rotated key part shared by all heads [T, rot_dim]."""
    rank = mixer["kv_rank"]
    z = _round(h @ w[p + "dkv"].T, rounding)
    latent = rms(z[:, :rank], eps) * w[p + "dkv.norm"]
    freqs, amplitude = ramped_frequencies(mixer["rot"])
    shared = rotate_halves(z[:, None, rank:], torch.arange(h.shape[0]), freqs, amplitude)[:, 0]
    return _round(latent, rounding), _round(shared, rounding)


def latent_attention(mixer: dict, w: dict, p: str, h: torch.Tensor, rows, rounding=None) -> torch.Tensor:
    """Causal attention over keys and values that are projections of a cached latent; every
    head's key is its own projection of the latent beside the one shared rotated part.
    `rows`: (latent, shared key part), the layer's own or another layer's."""
    heads, dim, rot_dim, vdim, rank = mixer["heads"], mixer["dim"], mixer["rot_dim"], mixer["vdim"], mixer["kv_rank"]
    n = h.shape[0]
    latent, shared = rows
    q = _round(h @ w[p + "q"].T, rounding).view(n, heads, dim + rot_dim)
    gate = _round(h @ w[p + "g"].T, rounding)
    freqs, amplitude = ramped_frequencies(mixer["rot"])
    q_turned = rotate_halves(q[..., dim:], torch.arange(n), freqs, amplitude)
    keys = (latent @ w[p + "uk"].T).view(n, heads, dim)
    values = (latent @ w[p + "uv"].T).view(n, heads, vdim)
    see = visible(n, None)
    out = torch.zeros(n, heads, vdim, dtype=torch.float64)
    for head in range(heads):
        scores = (q[:, head, :dim] @ keys[:, head].T + q_turned[:, head] @ shared.T) * mixer["scale"]
        out[:, head] = torch.softmax(scores.masked_fill(~see, float("-inf")), dim=-1) @ values[:, head]
    mixed = _round(_round(out.reshape(n, heads * vdim), rounding) * torch.sigmoid(gate), rounding)
    return mixed @ w[p + "o"].T


def gated_feed_forward(w: dict, p: str, h: torch.Tensor, rounding=None) -> torch.Tensor:
    gate, up = _round(h @ w[p + "gate"].T, rounding), _round(h @ w[p + "up"].T, rounding)
    return _round(gelu_tanh(gate) * up, rounding) @ w[p + "down"].T


def forward(config: dict, weights: dict, tokens, rounding=None, streams: list | None = None) -> torch.Tensor:
    """Logits [T, vocab] (float64) of one sequence. `weights`: name -> tensor (any float dtype).
    `streams`, when a list, receives the residual stream after every layer."""
    w = {k: v.double() for k, v in weights.items()}
    eps = float(config["norm"]["eps"])
    x = w["embed"][torch.as_tensor(list(tokens), dtype=torch.long)]
    cached: dict[int, tuple] = {}
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        mixer = layer["mixer"]
        h = _round(x, rounding)
        if layer["type"] == "attention":
            y = conv_attention(mixer, w, p + "mix.", h, eps, rounding)
        elif layer["type"] == "latent_attention":
            source = mixer.get("kv_from")
            if source is None:
                cached[i] = latent_rows(mixer, w, p + "mix.", h, eps, rounding)
                source = i
            y = latent_attention(mixer, w, p + "mix.", h, cached[source], rounding)
        else:
            raise ValueError(f"unknown layer type {layer['type']!r}")
        x = x + layer_norm(_round(y, rounding), w[p + "norm1"], w[p + "norm1.b"], eps)
        if layer.get("mlp") is not None:
            y = gated_feed_forward(w, p + "mlp.", _round(x, rounding), rounding)
            x = x + layer_norm(_round(y, rounding), w[p + "norm2"], w[p + "norm2.b"], eps)
        if streams is not None:
            streams.append(x.clone())
    return layer_norm(x, w["final.norm"], w["final.norm.b"], eps) @ w["head"].T


def relative_error(got: torch.Tensor, expected: torch.Tensor) -> float:
    """Largest |difference| over the largest |expected|."""
    return float((got.double() - expected.double()).abs().max() / expected.double().abs().max())
