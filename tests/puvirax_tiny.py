"""Small Puvirax configurations and random weights for the tests.

The configurations differ from each other in every size and constant: layer order (each of the
three mixers first somewhere), widths, head counts (query heads per kv head 1, 2, 3, 4 and 8), key
sizes above and below the value size, rotary widths (part of a head, all of it, none), bases,
frequency scaling (also absent), windows, bias tables of different heights and reach, layers with
and without value mixing (the first mixing layer not always the first layer), dense and routed
feed-forwards (with and without groups, with and without a shared expert, one chosen expert and
several), a layer without feed-forward, logit scales (also 1). Weights are drawn with torch and
written with the `safetensors` package, so the engine's reader and its names are checked against an
independent file.
"""

from __future__ import annotations

import json
import os
import tempfile

import torch

import plain_puvirax


def dense(ff):
    return {"kind": "dense", "ff": ff}


def routed(ff, experts, top, groups=None, shared=None):
    """groups: (count, keep) or None."""
    mlp = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if groups:
        mlp["router"]["groups"] = {"count": groups[0], "keep": groups[1]}
    if shared:
        mlp["shared"] = {"ff": shared}
    return mlp


def rotary_layer(heads, kv_heads, dim, vdim, rot_dims, mlp, v_mix=True, scale=None, base=10000.0, bands=None):
    """bands: (factor, low, high, original) or None."""
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "v_mix": v_mix,
             "scale": scale if scale is not None else 2.0 * dim ** -0.5}
    if rot_dims is not None:
        mixer["rot"] = {"base": base, "dims": rot_dims}
        if bands:
            mixer["rot"]["scaling"] = dict(zip(("factor", "low", "high", "original"), bands))
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


def biased_layer(kind, heads, kv_heads, dim, vdim, rows, far, mlp, window=None, v_mix=True, scale=None):
    """kind "attention_2" (norm per head; with a window) or "attention_3" (norm over the projection). `rows` is
    not part of the configuration: it is the height of the layer's bias table, which only the tensor gives."""
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "v_mix": v_mix, "bias_max": far,
             "scale": scale if scale is not None else 2.0 * dim ** -0.5}
    if window is not None:
        mixer["mask"] = {"size": window}
    return {"type": kind, "mixer": mixer, "mlp": mlp, "_rows": rows}


def _config(vocab, width, eps, logit_scale, pairs, layers):
    """(config.json text, bias-table heights per layer)."""
    rows = [layer.pop("_rows", None) for layer in layers]
    return ({"architecture": "Puvirax", "vocab": vocab, "width": width, "norm": {"eps": eps},
             "logit_scale": logit_scale,
             "embedding": {"bigram": dict(zip(("buckets", "mul_prev", "mul_cur"), pairs))}, "layers": layers}, rows)


CONFIG_A = _config(211, 72, 1e-5, 1.5, (97, 31, 5), [
    biased_layer("attention_2", 4, 2, 16, 24, 12, 40, routed(24, 8, 2, (4, 2), 40), window=21),
    rotary_layer(4, 2, 24, 24, 8, dense(96), bands=(2.0, 1.0, 4.0, 64)),
    biased_layer("attention_3", 6, 2, 8, 24, 10, 64.0, None),
    rotary_layer(2, 2, 16, 24, 16, routed(16, 5, 1)),
])
CONFIG_B = _config(97, 40, 1e-6, 1.0, (13, 3, 11), [
    rotary_layer(3, 3, 8, 16, 4, dense(56), v_mix=False, scale=0.9, base=100.0),
    biased_layer("attention_3", 4, 1, 12, 8, 6, 9, routed(16, 6, 2, (3, 2)), scale=0.5),
    biased_layer("attention_2", 2, 1, 20, 8, 8, 30, dense(24), window=9),
    biased_layer("attention_2", 5, 5, 8, 4, 4, 5, None, window=3, v_mix=False),
])
CONFIG_C = _config(128, 64, 1e-6, 0.7, (251, 1, 2), [
    biased_layer("attention_3", 4, 1, 32, 32, 16, 100, dense(80), scale=0.25),
    rotary_layer(4, 2, 48, 64, 32, dense(48), v_mix=False, base=500.0, bands=(8.0, 1.0, 2.0, 128)),
    biased_layer("attention_2", 8, 1, 64, 32, 32, 64, routed(32, 8, 3, (2, 1), 48), window=40, scale=0.2),
    rotary_layer(2, 1, 128, 32, 64, dense(80), scale=0.15),
    rotary_layer(2, 1, 32, 32, None, dense(40)),
])
CONFIGS = {"A": (CONFIG_A, 16), "B": (CONFIG_B, 32), "C": (CONFIG_C, 16)}


def tensor_shapes(cfg: dict, rows: list) -> dict[str, tuple[int, ...]]:
    w = cfg["width"]
    shapes = {"embed": (cfg["vocab"], w), "bigram": (cfg["embedding"]["bigram"]["buckets"] + 1, w), "final.norm": (w,)}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        heads, kv, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        shapes[p + "norm1"] = (w,)
        shapes[p + "mix.q"], shapes[p + "mix.k"], shapes[p + "mix.v"] = (heads * dim, w), (kv * dim, w), (kv * vdim, w)
        shapes[p + "mix.o"] = (w, heads * vdim)
        if layer["type"] == "attention":
            shapes[p + "mix.g"] = (heads, w)
        else:
            whole = layer["type"] == "attention_3"
            shapes[p + "mix.q.norm"] = (heads * dim if whole else dim,)
            shapes[p + "mix.k.norm"] = (kv * dim if whole else dim,)
            shapes[p + "mix.rel"] = (rows[i], heads)
        if m.get("v_mix"):
            shapes[p + "mix.vmix"] = ()
        mlp = layer["mlp"]
        if mlp is None:
            continue
        shapes[p + "norm2"] = (w,)
        if mlp["kind"] == "dense":
            shapes[p + "mlp.up"], shapes[p + "mlp.down"] = (mlp["ff"], w), (w, mlp["ff"])
        else:
            for e in range(mlp["router"]["experts"]):
                shapes[p + f"mlp.e{e}.up"], shapes[p + f"mlp.e{e}.down"] = (mlp["expert"]["ff"], w), (w, mlp["expert"]["ff"])
            shapes[p + "mlp.router"], shapes[p + "mlp.correction"] = (mlp["router"]["experts"], w), (mlp["router"]["experts"],)
            if mlp.get("shared"):
                shapes[p + "mlp.shared.up"], shapes[p + "mlp.shared.down"] = (mlp["shared"]["ff"], w), (w, mlp["shared"]["ff"])
    return shapes


def random_weights(cfg: dict, rows: list, seed: int, dtype: torch.dtype = torch.float32, sharp: float = 1.0) -> dict:
    """`sharp` multiplies every score (through the query norm's weight, or the layer's scale where the norm
    has none: see TinyPuvirax): with 3 or more a softmax rests on a few keys anywhere in reach, so that one key too
    many or too few moves the logits by far more than a rounding. Matrices N(0, 1/sqrt(in)), norm weights 1 + 0.2 N
    (the stream's norms 0.5 + 0.1 N, so that the stream grows slowly), bias tables N(0, 1), mixing factors in
    (0.2, 0.8), router rows three times the usual size and corrections 0.3 N (so that choices are not close calls and
    the correction changes some); rounded to `dtype`."""
    gen = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg, rows).items():
        leaf = name.split(".", 1)[1] if name[0] == "l" and "." in name else name
        if leaf in ("norm1", "norm2"):
            t = 0.5 + 0.1 * torch.randn(shape, generator=gen)
        elif leaf.endswith("norm"):
            t = 1.0 + 0.2 * torch.randn(shape, generator=gen)
            if leaf == "mix.q.norm":
                t = t * sharp
        elif leaf == "mix.rel":
            t = torch.randn(shape, generator=gen)
        elif leaf == "mix.vmix":
            t = 0.2 + 0.6 * torch.rand(shape, generator=gen)
        elif leaf == "mlp.correction":
            t = 0.3 * torch.randn(shape, generator=gen)
        elif name in ("embed", "bigram"):
            t = torch.randn(shape, generator=gen)
        else:
            gain = 3.0 if leaf == "mlp.router" else 1.0
            t = torch.randn(shape, generator=gen) * (gain / shape[1] ** 0.5)
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


def sharpened(cfg: dict, sharp: float) -> dict:
    """The configuration with the scale of every layer whose q/k norm has no weights times `sharp`."""
    cfg = json.loads(json.dumps(cfg))
    for layer in cfg["layers"]:
        if layer["type"] == "attention":
            layer["mixer"]["scale"] *= sharp
    return cfg


class TinyPuvirax:
    """A configuration with random weights rounded to the engine's dtype (so that the plain
    implementation, which runs in float64, and the engine start from identical numbers), its
    model folder, and the plain implementation's logits on demand."""

    def __init__(self, key: str, dtype: str, seed: int = 1, cfg: dict | None = None, rows: list | None = None,
                 weights: dict | None = None, page: int = 16, sharp: float = 1.0):
        if cfg is None:
            (cfg, rows), page = CONFIGS[key]
        self.cfg, self.rows, self.page = sharpened(cfg, sharp), rows, page
        self.dtype = dtype
        torch_dtype = torch.float32 if dtype == "float32" else torch.bfloat16
        self.weights = weights if weights is not None else random_weights(self.cfg, rows, seed, torch_dtype, sharp)
        self.weights = {k: v.to(torch_dtype) for k, v in self.weights.items()}
        self.plain_weights = {k: v.double() for k, v in self.weights.items()}
        self._dir = tempfile.TemporaryDirectory()
        self.folder = write_model_dir(self._dir.name, self.cfg, self.weights)
        self._plain: dict[tuple, torch.Tensor] = {}

    def plain_logits(self, tokens) -> torch.Tensor:
        key = tuple(tokens)
        if key not in self._plain:
            self._plain[key] = plain_puvirax.forward(self.cfg, self.plain_weights, list(tokens))
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
        median of a request's positions within half the bar; where the model routes tokens to
        experts, one position a request may lie beyond the loose bar (a rounding can tip a router's
        close call, which moves a row by far more than a rounding; the float32 run of the same
        schedule holds every position)."""
        worst = 0.0
        bar = TOLERANCE[self.dtype]
        loose = self.dtype == "bfloat16"
        routed_layers = any((layer.get("mlp") or {}).get("kind") == "moe" for layer in self.cfg["layers"])
        for r, rows in got.items():
            ref = self.plain_logits(request_tokens[r])
            errors = []
            beyond = []
            for position in sorted(rows):
                err = relative_error(rows[position], ref[position])
                errors.append(err)
                if err >= (0.25 if loose else bar):
                    beyond.append((position, err))
            assert len(beyond) <= (1 if loose and routed_layers else 0), (
                f"{what}: request {r!r} differs from the plain implementation at positions "
                f"{beyond[:5]} of {len(request_tokens[r])} (rel error; bar {bar:.0e})")
            errors.sort()
            if loose:
                assert errors[len(errors) // 2] < bar / 2, f"{what}: request {r!r}: median error {errors[len(errors) // 2]:.3e}"
            worst = max(worst, errors[-1])
        return worst
