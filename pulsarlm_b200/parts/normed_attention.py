"""Grouped-query attention with normed queries and keys, key and value sizes of their own, an
optional bias by distance, values that may be mixed with an earlier layer's, and an optional
gate per head."""

from __future__ import annotations

import math

import torch

from ..kernels import ops
from .attention import Attention
from .linear import linear
from .registry import BuildContext, register_part
from .spec import KVCacheNeed, PartSpec, TensorNeed

QK_NORMS = ("none", "per_head", "whole", "unit_after")


def distance_bucket(distance: int, rows: int, far: float) -> int:
    """The row of a bias table of `rows` rows for a key `distance` tokens back: the first rows / 2
    distances have a row each; from there the rows are spaced evenly in the logarithm of the
    distance and the last one is reached at `far`."""
    half = rows // 2
    if distance < half:
        return distance
    if half == 0:
        return rows - 1
    if far <= half:
        return rows - 1
    step = math.log(distance / half) / math.log(far / half) * (rows - half)
    return min(rows - 1, half + int(math.floor(step)))


def bias_by_distance(table: torch.Tensor, far: float) -> torch.Tensor:
    """table [rows, heads] -> fp32 [heads, D] with column d = table[bucket(d)] for every distance up
    to the first that lands in the last row; greater distances read the last column (the kernels
    clamp the distance to D - 1). A head's entries lie side by side: the keys of a tile are
    neighbours in distance."""
    rows = table.shape[0]
    picks = []
    d = 0
    while True:
        b = distance_bucket(d, rows, far)
        picks.append(b)
        if b == rows - 1:
            break
        d += 1
    index = torch.tensor(picks, dtype=torch.long, device=table.device)
    return table.float()[index].t().contiguous()


@register_part("mixer", "normed_attention")
class NormedAttention(Attention):
    """q = Wq h [heads, dim], k = Wk h [kv_heads, dim], v = Wv h [kv_heads, vdim]; causal softmax
    attention of head h over kv head h // (heads / kv_heads) with scores (q . k) * scale, an
    optional sliding `window`, then the o projection over the concatenated heads [heads * vdim].

    `qk_norm`: how q and k are normed (RMS, eps `norm_eps`): "per_head" over each head's dim with
    the weights `q_norm` / `k_norm` [dim] shared by the heads; "whole" over the whole projection
    with weights [heads * dim] / [kv_heads * dim]; both before the position encoding;
    "unit_after": per head, no weights, after the position encoding; "none". `position`: a
    "position" PartSpec (rotate-half over part of every head, or none). `bias_far` with the tensor
    `distance_bias` [rows, heads]: a learned bias joins the scaled score of a key d tokens back, row
    `distance_bucket(d, rows, bias_far)` of the table (expanded to one row per distance at load).
    `value_mix` with `value_stream` (a name): the "source" layer leaves its values in the step under
    that name; a "mix" layer stores (1 - lambda) v + lambda v_source in its cache, lambda its scalar
    tensor `value_mix`. `head_gate`: every head's output is multiplied by sigmoid(Wg h)_h, `gate`
    [heads, hidden].

    q, k, v and the gate's logits come from one product. One kernel (csrc/norm_rope_mix.cu) then
    norms, rotates, mixes and writes q and the cache rows as rows of a common size (the larger of
    dim and vdim, rounded up to a multiple of 16, zeros past a row's own columns), so that the
    paged attention kernels, which know one row size, run them unchanged; the o projection's
    weights get zero columns to match, so nothing is compacted in between. A bias travels to the
    attention kernels as an extra, and a gate with it; a layer whose only extra would be the gate
    keeps the plain attention kernels in bfloat16 (tcgen05 for prompt portions at rows of 64 and
    128, work lists for many single tokens) and multiplies by the gate in a small kernel afterwards.

    params: hidden_size, n_heads, n_kv_heads, head_dim (dim), value_dim, scale, window, norm_eps,
    qk_norm, position, bias_far, bias_rows (optional), value_mix, value_stream, head_gate. tensors: q, k, v, o,
    q_norm, k_norm, distance_bias, value_mix, gate, and `ignored`: {name: shape} of tensors that a checkpoint may
    hold for the layer and nothing reads."""

    def __init__(self, spec: PartSpec, ctx: BuildContext):
        p = spec.params
        self.key_dim = int(p["head_dim"])
        self.value_dim = int(p.get("value_dim") or self.key_dim)
        self.row = -(-max(self.key_dim, self.value_dim) // 16) * 16
        scale = float(p["scale"]) if p.get("scale") is not None else 1.0 / math.sqrt(self.key_dim)
        inner = PartSpec(spec.kind, {**p, "head_dim": self.row, "scale": scale}, spec.tensors)
        super().__init__(inner, ctx)
        self.spec = spec
        if p.get("cache_from") is not None or p.get("softcap") or p.get("sink_logit") is not None:
            raise ValueError("normed_attention: cache_from, softcap and sinks are not supported")
        self.qk_norm = str(p.get("qk_norm") or "none")
        if self.qk_norm not in QK_NORMS:
            raise ValueError(f"normed_attention: unknown qk_norm {self.qk_norm!r} (known: {', '.join(QK_NORMS)})")
        self.norm_eps = float(p.get("norm_eps") or 0.0)
        self.bias_far = float(p["bias_far"]) if p.get("bias_far") is not None else None
        self.gated = bool(p.get("head_gate", False))
        self.head_gate = self.gated   # (whether the gate rides along inside the attention kernels: see bind_cache)
        self.value_mix = p.get("value_mix")
        self.value_stream = p.get("value_stream")
        if self.value_mix not in (None, "source", "mix") or (self.value_mix and not self.value_stream):
            raise ValueError("normed_attention: value_mix is 'source' or 'mix' and needs a value_stream name")
        self.lam = 0.0
        self.q_weight: torch.Tensor | None = None
        self.k_weight: torch.Tensor | None = None

    @classmethod
    def tensor_needs(cls, spec: PartSpec) -> dict[str, TensorNeed]:
        p, t = spec.params, spec.tensors
        h, nh, nkv, hd = (int(p[k]) for k in ("hidden_size", "n_heads", "n_kv_heads", "head_dim"))
        vd = int(p.get("value_dim") or hd)
        needs = {t["q"]: TensorNeed((nh * hd, h)), t["k"]: TensorNeed((nkv * hd, h)), t["v"]: TensorNeed((nkv * vd, h)),
                 t["o"]: TensorNeed((h, nh * vd))}
        norm = str(p.get("qk_norm") or "none")
        if norm in ("per_head", "whole"):
            needs[t["q_norm"]] = TensorNeed((hd if norm == "per_head" else nh * hd,), role="vector")
            needs[t["k_norm"]] = TensorNeed((hd if norm == "per_head" else nkv * hd,), role="vector")
        if p.get("bias_far") is not None:
            # (the table's rows are a size of the stored tensor; a configuration may name them, for random weights)
            needs[t["distance_bias"]] = TensorNeed((int(p.get("bias_rows") or -1), nh), role="offset")
        if p.get("head_gate"):
            needs[t["gate"]] = TensorNeed((nh, h))
        if p.get("value_mix") == "mix":
            needs[t["value_mix"]] = TensorNeed((), role="offset")
        elif t.get("value_mix"):
            # (the layer whose values the others mix in may store a factor too, and so may a layer that mixes
            # nothing: neither uses it)
            needs[t["value_mix"]] = TensorNeed((), role="ignored", optional=True)
        for name, shape in (t.get("ignored") or {}).items():
            # (tensors a checkpoint may hold for this layer that nothing reads)
            needs[name] = TensorNeed(tuple(shape), role="ignored", optional=True)
        return needs

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        t = self.spec.tensors
        nh, vd, row = self.n_heads, self.value_dim, self.row
        stacked = [tensors[t["q"]], tensors[t["k"]], tensors[t["v"]]]
        if self.gated:
            stacked.append(tensors[t["gate"]])
        width = sum(w.shape[0] for w in stacked)
        if self.ctx.dtype == torch.bfloat16 and width % 8:
            # (rows of the product's output start on 16 bytes: the kernels that read slices of it rely on that)
            stacked.append(torch.zeros((8 - width % 8, self.hidden), dtype=stacked[0].dtype, device=stacked[0].device))
        self.qkv = torch.cat(stacked, dim=0).contiguous()
        o = tensors[t["o"]]
        if row != vd:
            padded = torch.zeros((self.hidden, nh, row), dtype=o.dtype, device=o.device)
            padded[:, :, :vd] = o.view(self.hidden, nh, vd)
            o = padded.view(self.hidden, nh * row)
        self.o = o.contiguous()
        if self.qk_norm in ("per_head", "whole"):
            self.q_weight = tensors[t["q_norm"]].float().contiguous()
            self.k_weight = tensors[t["k_norm"]].float().contiguous()
        if self.bias_far is not None:
            self.distance_bias = bias_by_distance(tensors[t["distance_bias"]], self.bias_far)
        if self.value_mix == "mix":
            self.lam = float(tensors[t["value_mix"]].float().item())

    def cache_need(self) -> KVCacheNeed:
        return KVCacheNeed(self.n_kv, self.row, self.window, self.n_heads)

    def cache_read_need(self) -> KVCacheNeed:
        return self.cache_need()

    def bind_cache(self, binding) -> None:
        super().bind_cache(binding)
        # With the cache's page size known: a gate that would be the layer's only extra stays out of the attention
        # kernels where the plain tensor-core kernels take the shape (they are the faster builds).
        if self.gated and self.distance_bias is None and self.bias_far is None and self.ctx.dtype == torch.bfloat16:
            self._decode_kernel = self._prefill_kernel = None
            self.head_gate = not all(self._kernels(self.ctx.dtype))

    def _folds_rope(self, tokens, batch, inv_freq, rotary) -> bool:
        return False  # (norms, rotation and mixing are a kernel of their own)

    def native_choice(self, tokens, batch, row_stride):
        return None

    def forward(self, h: torch.Tensor, batch) -> torch.Tensor:
        tokens = h.shape[0]
        nh, nkv, hd, vd, row = self.n_heads, self.n_kv, self.key_dim, self.value_dim, self.row
        cache = self.cache
        table = batch.tables[cache.group]
        proj = linear(h, self.qkv)
        q_end, k_end, v_end = nh * hd, (nh + nkv) * hd, (nh + nkv) * hd + nkv * vd
        q = proj[:, :q_end].view(tokens, nh, hd)
        k = proj[:, q_end:k_end].view(tokens, nkv, hd)
        v = proj[:, k_end:v_end].view(tokens, nkv, vd)
        gate = proj[:, v_end:v_end + nh] if self.gated else None
        first, first_stride = None, None
        if self.value_mix == "source":
            # (with the row stride of the product they are columns of: a view of one token forgets it)
            batch.extras[("values", self.value_stream)] = (proj[:, k_end:v_end], proj.stride(0))
        elif self.value_mix == "mix":
            first, first_stride = batch.extras.get(("values", self.value_stream), (None, None))
            if first is None:
                raise RuntimeError(f"normed_attention: no layer before this one left values under {self.value_stream!r}")
            if first.shape[1] != nkv * vd:
                raise ValueError(f"normed_attention: the values under {self.value_stream!r} are {first.shape[1]} wide, "
                                 f"this layer's {nkv * vd}")
            first = first.view(tokens, nkv, vd)  # (a token's values as one row: the heads' split is each layer's own)
        q_rows = torch.empty((tokens, nh, row), dtype=h.dtype, device=h.device)
        inv_freq, rotary = self.position.table()
        ops.norm_rope_mix_write(q, k, v, first, self.lam, q_rows, batch.pos, batch.entry, table, cache.k_pool,
                                cache.v_pool, cache.page_size, inv_freq, rotary, self.qk_norm, self.q_weight,
                                self.k_weight, self.norm_eps, batch.status, proj.stride(0), first_stride)
        out = torch.empty((tokens, nh, row), dtype=h.dtype, device=h.device)
        self.attend(q_rows, out, table, batch, gate=gate if self.head_gate else None)
        if self.gated and not self.head_gate:
            ops.sigmoid_gate_heads(out, gate)
        return linear(out.view(tokens, nh * row), self.o)
