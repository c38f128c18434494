"""A plain, slow implementation of the Puvirax decoder in float64 torch on the CPU, one
function per mechanism, written from the architecture's equations. It shares no code
with the engine: whole sequences at once, no cache, no pages, no state slots.

Notation: x [T, W] the residual stream, h a sublayer's input (the normed stream), weights
by their checkpoint names ([out, in], applied as W h). `forward(..., rounding=torch.bfloat16)`
rounds where a bfloat16 engine stores a tensor (projections, cached rows, sublayer outputs),
so that the comparison with such an engine sees its arithmetic and not its storage.
"""

from __future__ import annotations

import math

import torch


def relative_error_of(got: torch.Tensor, want: torch.Tensor) -> float:
    """Largest |difference| over largest |wanted|."""
    return float((got.double() - want.double()).abs().max() / want.double().abs().max().clamp(min=1e-30))


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def pair_embedding(tokens: list[int], table: torch.Tensor, pairs: torch.Tensor, cfg: dict,
                   before: int | None = None) -> torch.Tensor:
    """table[token] plus a row of `pairs` chosen by a hash of (token before, token); a sequence's
    first token takes the last row. `before`: the token ahead of tokens[0] (None: a sequence's start)."""
    b = cfg["embedding"]["bigram"]
    rows = []
    for t, tok in enumerate(tokens):
        prev = tokens[t - 1] if t > 0 else before
        rows.append(b["buckets"] if prev is None else (prev * b["mul_prev"] + tok * b["mul_cur"]) % b["buckets"])
    return table[torch.tensor(tokens)] + pairs[torch.tensor(rows)]


def banded_frequencies(rot: dict) -> torch.Tensor:
    """f_i = base^(-2i / dims); with scaling, short waves stay, long ones are divided by the
    factor, those between are blended."""
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


def rotate_halves(u: torch.Tensor, positions: torch.Tensor, rot: dict) -> torch.Tensor:
    """u [T, heads, dim]: column i of the first rot.dims columns is paired with column i + dims/2."""
    dims = rot["dims"]
    half = dims // 2
    angle = positions.to(torch.float64)[:, None] * banded_frequencies(rot)[None, :]
    cos, sin = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    a, b = u[..., :half], u[..., half:dims]
    return torch.cat([a * cos - b * sin, b * cos + a * sin, u[..., dims:]], dim=-1)


def distance_bucket(n: int, rows: int, far: float) -> int:
    """Distances below rows/2 have a row each; the others share the upper rows on a logarithmic scale
    that reaches the last row at `far`."""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


def distance_bias(table: torch.Tensor, far: float, n: int) -> torch.Tensor:
    """[n, n, heads]: table[bucket(i - j), h] for j <= i (zeros above the diagonal)."""
    rows = table.shape[0]
    by_distance = table[torch.tensor([distance_bucket(d, rows, far) for d in range(n)])]
    i = torch.arange(n)[:, None]
    j = torch.arange(n)[None, :]
    return by_distance[(i - j).clamp(min=0)] * (j <= i)[:, :, None]


def softmax_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, window: int | None,
                      bias: torch.Tensor | None) -> torch.Tensor:
    """q [T, H, D], k [T, G, D], v [T, G, Dv]; head h reads kv head h // (H / G); query i sees
    keys j <= i, with a window only those with i - j < window; bias [T, T, H] joins the scaled scores."""
    n, heads = q.shape[0], q.shape[1]
    per = heads // k.shape[1]
    i = torch.arange(n)[:, None]
    j = torch.arange(n)[None, :]
    seen = j <= i
    if window is not None:
        seen = seen & (i - j < window)
    out = torch.zeros(n, heads, v.shape[-1], dtype=torch.float64)
    for h in range(heads):
        s = (q[:, h] @ k[:, h // per].T) * scale
        if bias is not None:
            s = s + bias[:, :, h]
        s = s.masked_fill(~seen, float("-inf"))
        out[:, h] = torch.softmax(s, dim=-1) @ v[:, h // per]
    return out


def mixed_values(v: torch.Tensor, first: torch.Tensor | None, lam: float) -> torch.Tensor:
    return v if first is None else (1.0 - lam) * v + lam * first


def mixer(kind: str, h: torch.Tensor, w: dict, m: dict, eps: float, positions: torch.Tensor,
          first_values: torch.Tensor | None, rnd):
    """One of the three attention mixers; returns (output [T, W], this layer's values before mixing)."""
    n = h.shape[0]
    heads, kv, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q, k, v = rnd(h @ w["q"].T), rnd(h @ w["k"].T), rnd(h @ w["v"].T)
    window = m["mask"]["size"] if m.get("mask") else None
    bias = None
    if kind == "attention":
        q, k = q.view(n, heads, dim), k.view(n, kv, dim)
        if m.get("rot"):
            q, k = rotate_halves(q, positions, m["rot"]), rotate_halves(k, positions, m["rot"])
        q, k = rms(q, eps), rms(k, eps)
    elif kind == "attention_2":
        q = rms(q.view(n, heads, dim), eps) * w["q.norm"]
        k = rms(k.view(n, kv, dim), eps) * w["k.norm"]
    elif kind == "attention_3":
        q = (rms(q, eps) * w["q.norm"]).view(n, heads, dim)
        k = (rms(k, eps) * w["k.norm"]).view(n, kv, dim)
    else:
        raise ValueError(kind)
    if "rel" in w:
        bias = distance_bias(w["rel"], float(m["bias_max"]), n)
    own = v
    if m.get("v_mix"):
        v = mixed_values(v, first_values, float(w["vmix"]))
    q, k, v = rnd(q), rnd(k), rnd(v)
    a = softmax_attention(q, k, v.view(n, kv, vdim), float(m["scale"]), window, bias)
    if kind == "attention":
        gate = torch.sigmoid(rnd(h @ w["g"].T))
        a = a * gate[:, :, None]
    return rnd(rnd(a).reshape(n, heads * vdim) @ w["o"].T), own


def squared_relu_ff(h: torch.Tensor, up: torch.Tensor, down: torch.Tensor, rnd) -> torch.Tensor:
    z = rnd(h @ up.T)
    return rnd(rnd(torch.relu(z) ** 2) @ down.T)


def route(h: torch.Tensor, router: torch.Tensor, correction: torch.Tensor, r: dict) -> tuple[torch.Tensor, torch.Tensor]:
    """ids [T, top] and weights [T, top]: sigmoid scores; the choice sees score + correction, and only
    experts of the groups whose two best choice scores add up to most; the weights are the scores."""
    s = torch.sigmoid(h @ router.T)
    choice = s + correction
    experts, top = r["experts"], r["top"]
    groups = r.get("groups")
    if groups:
        size = experts // groups["count"]
        per_group = choice.view(-1, groups["count"], size)
        group_score = per_group.topk(min(2, size), dim=-1).values.sum(-1)
        kept = group_score.topk(groups["keep"], dim=-1).indices
        allowed = torch.zeros_like(group_score, dtype=torch.bool).scatter_(1, kept, True)
        choice = choice.masked_fill(~allowed.repeat_interleave(size, dim=1), float("-inf"))
    ids = choice.topk(top, dim=-1).indices
    return ids, s.gather(1, ids)


def routed_ff(h: torch.Tensor, w: dict, mlp: dict, rnd) -> torch.Tensor:
    ids, weights = route(h, w["router"], w["correction"], mlp["router"])
    out = torch.zeros(h.shape[0], w["e0.down"].shape[0], dtype=torch.float64)
    for t in range(h.shape[0]):
        for e, g in zip(ids[t].tolist(), weights[t].tolist()):
            out[t] += g * squared_relu_ff(h[t:t + 1], w[f"e{e}.up"], w[f"e{e}.down"], rnd)[0]
    if mlp.get("shared"):
        out = out + squared_relu_ff(h, w["shared.up"], w["shared.down"], rnd)
    return rnd(out)


def sub(weights: dict, prefix: str) -> dict:
    return {k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}


def forward(cfg: dict, weights: dict, tokens: list[int], rounding=None, streams: list | None = None) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence. weights: float64 tensors by checkpoint name.
    `streams`, if a list, receives the residual stream after every layer."""
    def rnd(t: torch.Tensor) -> torch.Tensor:
        return t.to(rounding).to(torch.float64) if rounding is not None else t

    eps = float(cfg["norm"]["eps"])
    positions = torch.arange(len(tokens))
    x = pair_embedding(tokens, weights["embed"], weights["bigram"], cfg)
    first_values = None
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = rnd(rms(x, eps) * weights[p + "norm1"])
        y, own = mixer(layer["type"], h, sub(weights, p + "mix."), layer["mixer"], eps, positions,
                       first_values if layer["mixer"].get("v_mix") else None, rnd)
        if layer["mixer"].get("v_mix") and first_values is None:
            first_values = own
        x = x + y
        mlp = layer.get("mlp")
        if mlp:
            h = rnd(rms(x, eps) * weights[p + "norm2"])
            w = sub(weights, p + "mlp.")
            x = x + (routed_ff(h, w, mlp, rnd) if mlp["kind"] == "moe" else squared_relu_ff(h, w["up"], w["down"], rnd))
        if streams is not None:
            streams.append(x.clone())
    h = rnd(rms(x, eps) * weights["final.norm"])
    return (h @ weights["embed"].T) * float(cfg["logit_scale"])
