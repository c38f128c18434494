"""Small Simetar configurations and random weights for the tests.

The configurations differ from each other in every size and constant: layer order (an
attention layer first, a latent layer first, two latent layers of which one reads the
other's rows, a reader directly after its owner and one two layers later), widths, head
counts (query heads per kv head 1, 2, 3 and 4), key sizes, rotary widths (all of a head,
part of it, none), bases and both kinds of frequency scaling (also absent), windows (one
layer without), taps (1 to 4), score caps (one layer without), scales, latent ranks,
value sizes above and below the key size, a layer without feed-forward. Weights are
drawn with torch and written with the `safetensors` package, so the engine's reader and
its names are checked against an independent file.
"""

from __future__ import annotations

import json
import os
import tempfile

import torch

import plain_simetar


def dense(ff):
    return {"kind": "dense", "ff": ff}


def attention_layer(heads, kv_heads, dim, window, rot_dims, taps, mlp, softcap=30.0, scale=None, base=10000.0,
                    bands=None):
    """bands: (factor, low, high, original) or None."""
    rot = {"base": base, "dims": rot_dims}
    if bands:
        rot["scaling"] = dict(zip(("factor", "low", "high", "original"), bands))
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "conv": taps,
             "scale": scale if scale is not None else dim ** -0.5, "rot": rot}
    if window is not None:
        mixer["mask"] = {"size": window}
    if softcap is not None:
        mixer["softcap"] = softcap
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


def latent_layer(heads, dim, rot_dim, vdim, rank, mlp, scale=None, base=10000.0, ramp=None, kv_from=None):
    """ramp: (factor, original, fast, slow) or None."""
    rot = {"base": base, "dims": rot_dim}
    if ramp:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), ramp))
    mixer = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank,
             "scale": scale if scale is not None else (dim + rot_dim) ** -0.5, "rot": rot}
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": mixer, "mlp": mlp}


_RAMP_A = (4.0, 64, 16.0, 1.0)
CONFIG_A = {
    "architecture": "Simetar", "vocab": 211, "width": 72, "norm": {"eps": 1e-5},
    "layers": [attention_layer(4, 2, 16, 21, 16, 3, dense(96), softcap=20.0, bands=(2.0, 1.0, 4.0, 64)),
               latent_layer(3, 16, 8, 24, 40, dense(96), ramp=_RAMP_A),
               attention_layer(4, 2, 16, 21, 16, 3, dense(96), softcap=20.0, bands=(2.0, 1.0, 4.0, 64)),
               latent_layer(3, 16, 8, 24, 40, dense(96), ramp=_RAMP_A, kv_from=1)],
}
CONFIG_B = {
    "architecture": "Simetar", "vocab": 97, "width": 40, "norm": {"eps": 1e-6},
    "layers": [latent_layer(2, 8, 4, 4, 24, None, scale=0.4, base=100.0),
               latent_layer(5, 12, 4, 16, 24, dense(56), scale=0.3, base=100.0, kv_from=0),
               attention_layer(3, 3, 8, None, 4, 2, dense(24), softcap=None, scale=0.5, base=500.0),
               attention_layer(6, 2, 12, 9, 0, 4, None, softcap=5.0, scale=0.3)],
}
_RAMP_C = (16.0, 32, 8.0, 2.0)
CONFIG_C = {
    "architecture": "Simetar", "vocab": 128, "width": 64, "norm": {"eps": 1e-6},
    "layers": [attention_layer(4, 1, 32, 40, 24, 1, dense(80), softcap=50.0, scale=0.2, bands=(8.0, 1.0, 2.0, 128)),
               latent_layer(4, 32, 16, 32, 48, dense(80), scale=0.15, ramp=_RAMP_C),
               attention_layer(2, 2, 16, 7, 16, 4, dense(48), softcap=2.0, base=50.0),
               latent_layer(2, 16, 16, 40, 48, dense(80), scale=0.2, ramp=_RAMP_C, kv_from=1)],
}
CONFIGS = {"A": (CONFIG_A, 16), "B": (CONFIG_B, 32), "C": (CONFIG_C, 16)}


def tensor_shapes(cfg: dict) -> dict[str, tuple[int, ...]]:
    w = cfg["width"]
    shapes = {"embed": (cfg["vocab"], w), "final.norm": (w,), "final.norm.b": (w,), "head": (cfg["vocab"], w)}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        shapes[p + "norm1"] = shapes[p + "norm1.b"] = (w,)
        heads, dim, vdim = m["heads"], m["dim"], m["vdim"]
        if layer["type"] == "attention":
            kv, taps = m["kv_heads"], m["conv"]
            for name, rows in (("q", heads * dim), ("k", kv * dim)):
                shapes[p + "mix." + name] = (rows, w)
                shapes[p + "mix." + name + ".b"] = shapes[p + "mix." + name + ".norm"] = (rows,)
                shapes[p + "mix." + name + ".conv"] = (rows, taps)
            shapes[p + "mix.g"] = (heads * vdim, w)
        else:
            rot, rank = m["rot_dim"], m["kv_rank"]
            shapes[p + "mix.q"] = (heads * (dim + rot), w)
            if m.get("kv_from") is None:
                shapes[p + "mix.dkv"] = (rank + rot, w)
                shapes[p + "mix.dkv.norm"] = (rank,)
            shapes[p + "mix.uk"], shapes[p + "mix.uv"] = (heads * dim, rank), (heads * vdim, rank)
            shapes[p + "mix.g"] = (heads * vdim, w)
        shapes[p + "mix.o"] = (w, heads * vdim)
        if layer["mlp"] is not None:
            shapes[p + "norm2"] = shapes[p + "norm2.b"] = (w,)
            shapes[p + "mlp.gate"] = shapes[p + "mlp.up"] = (layer["mlp"]["ff"], w)
            shapes[p + "mlp.down"] = (w, layer["mlp"]["ff"])
    return shapes


def random_weights(cfg: dict, seed: int, dtype: torch.dtype = torch.float32, sharp: float = 1.0) -> dict:
    """`sharp` multiplies every score (through the query norm's weight, or the query projection
    where there is no such norm): with 3 or 4 a softmax rests on a few keys anywhere in reach, so
    that one key too many or too few moves the logits by far more than a rounding. Matrices N(0, 1/sqrt(in)) (queries, keys and
    the latent's projections twice that, so that attention is far from uniform), norm weights 1 + 0.2 N (the norms on sublayer outputs 0.5 of
    that, so that the stream grows slowly), biases 0.3 N, convolution taps N(0, 0.6); rounded to
    `dtype`."""
    gen = torch.Generator().manual_seed(seed)
    out = {}
    shapes = tensor_shapes(cfg)
    for name, shape in shapes.items():
        leaf = name.split(".", 1)[1] if name[0] == "l" and "." in name else name
        if leaf.endswith(".b"):
            t = 0.3 * torch.randn(shape, generator=gen)
        elif leaf in ("norm1", "norm2"):
            t = 0.5 + 0.1 * torch.randn(shape, generator=gen)
        elif leaf.endswith("norm"):
            t = 1.0 + 0.2 * torch.randn(shape, generator=gen)
        elif leaf.endswith(".conv"):
            t = 0.6 * torch.randn(shape, generator=gen)
        elif name == "embed":
            t = torch.randn(shape, generator=gen)
        else:
            gain = 2.0 if leaf in ("mix.q", "mix.k", "mix.dkv", "mix.uk") else 1.0
            t = torch.randn(shape, generator=gen) * (gain / shape[1] ** 0.5)
        if leaf == "mix.q.norm" or (leaf == "mix.q" and name + ".norm" not in shapes):
            t = t * sharp
        out[name] = t.to(dtype)
    return out


def write_model_dir(folder: str, cfg: dict, weights: dict) -> str:
    from safetensors.torch import save_file

    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_file({k: v.contiguous() for k, v in weights.items()}, os.path.join(folder, "model.safetensors"))
    return folder


def random_tokens(cfg: dict, length: int, seed: int) -> list[int]:
    gen = torch.Generator().manual_seed(seed)
    return torch.randint(0, cfg["vocab"], (length,), generator=gen).tolist()


# Largest |difference| over largest |expected| of a row of logits, against the plain implementation
# in float64. The float32 engine is the sharp comparison. In bfloat16 the engine rounds activations
# at some ten places a layer; those runs hold most positions to the bar and none beyond a loose
# one, and what is off by a rounding is left to the float32 runs.
TOLERANCE = {"float32": 2e-4, "bfloat16": 6e-2}


def relative_error(got: torch.Tensor, want: torch.Tensor) -> float:
    return float((got.double() - want.double()).abs().max() / want.double().abs().max())


class TinySimetar:
    """A configuration with random weights rounded to the engine's dtype (so that the plain
    implementation, which runs in float64, and the engine start from identical numbers), its
    model folder, and the plain implementation's logits on demand."""

    def __init__(self, key: str, dtype: str, seed: int = 1, cfg: dict | None = None, weights: dict | None = None,
                 page: int = 16, sharp: float = 1.0):
        self.cfg, self.page = CONFIGS[key] if cfg is None else (cfg, page)
        self.dtype = dtype
        torch_dtype = torch.float32 if dtype == "float32" else torch.bfloat16
        self.weights = weights if weights is not None else random_weights(self.cfg, seed, torch_dtype, sharp)
        self.weights = {k: v.to(torch_dtype) for k, v in self.weights.items()}
        self.plain_weights = {k: v.double() for k, v in self.weights.items()}
        self._dir = tempfile.TemporaryDirectory()
        self.folder = write_model_dir(self._dir.name, self.cfg, self.weights)
        self._plain: dict[tuple, torch.Tensor] = {}

    def plain_logits(self, tokens) -> torch.Tensor:
        key = tuple(tokens)
        if key not in self._plain:
            self._plain[key] = plain_simetar.forward(self.cfg, self.plain_weights, list(tokens))
        return self._plain[key]

    def runner(self, n_pages: int, slots: int = 4, page: int | None = None):
        from pulsarlm_b200.cache.manager import CacheManager
        from pulsarlm_b200.engine.loading import load_model
        from pulsarlm_b200.engine.runner import ModelRunner

        model = load_model(self.folder, self.dtype, "cuda:0")
        cache = CacheManager(model.cache_needs(), page or self.page, n_pages, slots, model.ctx.dtype, "cuda:0")
        return ModelRunner(model, cache)

    def check(self, request_tokens: dict, got: dict, what: str) -> float:
        """Every returned row against the plain implementation's row at that position. float32:
        every position within the bar. bfloat16: every position within a loose bar and the
        median of a request's positions within half the bar."""
        worst = 0.0
        bar = TOLERANCE[self.dtype]
        loose = self.dtype == "bfloat16"
        for r, rows in got.items():
            ref = self.plain_logits(request_tokens[r])
            errors = []
            for position in sorted(rows):
                err = relative_error(rows[position], ref[position])
                errors.append(err)
                assert err < (0.25 if loose else bar), (
                    f"{what}: request {r!r} differs from the plain implementation at position "
                    f"{position} of {len(request_tokens[r])}: rel error {err:.3e} (bar {bar:.0e})")
            errors.sort()
            if loose:
                assert errors[len(errors) // 2] < bar / 2, f"{what}: request {r!r}: median error {errors[len(errors) // 2]:.3e}"
            worst = max(worst, errors[-1])
        return worst
