"""Attention over a cached low-rank latent: one row per token serves every head as key and value."""

from __future__ import annotations

import os

import numpy as np
import torch

from ..kernels import ops
from .attention import KVBinding, decode_splits
from .linear import linear
from .registry import BuildContext, Part, build_part, register_part
from .spec import KVCacheNeed, PartSpec, TensorNeed


# (1: every token attends on the CUDA-core kernel, for comparison)
CUDA_CORES_ONLY = os.environ.get("PULSARLM_B200_LATENT_CUDA_CORES", "0") == "1"


def per_head_linear(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor) -> None:
    """out[:, h, :] = x[:, h, :] @ weight[h]^T for x [T, H, K], weight [H, N, K], out [T, H, N]
    (a view whose last axis is contiguous). bfloat16: one batched library product that
    writes the strided output in place; float32: the package's own fp32 product per head."""
    heads = x.shape[1]
    if x.dtype == torch.float32:
        for h in range(heads):
            ops.gemm_f32(x[:, h], weight[h], out[:, h])
        return
    torch.bmm(x.transpose(0, 1), weight.transpose(1, 2), out=out.transpose(0, 1))


@register_part("mixer", "latent_attention")
class LatentAttention(Part):
    """Causal attention whose keys and values are projections of a shared latent:

        q = Wq h                       [heads, dim]
        c = rmsnorm(Wd h) * n          [rank]: the only thing cached per token
        k_h = Wuk_h c, v_h = Wuv_h c   per head
        p = softmax over {(q_h . k_h) * scale of the keys in reach} and one sink term exp(s_h)
        out = Wo concat_h(sigmoid(Wg h)_h * sum_j p_j v_h,j)

    Keys and values are never formed: with q'_h = Wuk_h^T q_h the scores are q'_h . c_j, and
    the weighted sum of the latents goes through Wuv_h afterwards, so attention runs over
    the paged latents with one shared "kv head" of size rank.

    With `rope_dim` = r > 0 every head's query has r more columns after its head_dim, the
    down projection r more rows after the latent's, and those rows (not normed) are one
    rotated key part shared by all heads: the score becomes q_h . k_h + rot(q_h^r) . rot(k^r),
    the cached row [c | rot(k^r)] of size rank + r, and the query row [q'_h | rot(q_h^r)];
    the weighted sum's first rank columns go through Wuv_h. The rotation is the "position"
    PartSpec's (`rope`: halves paired; `rope_pairs`: neighbours; its `amplitude` multiplies
    cos and sin). Without rope_dim there is no position encoding.

    params: hidden_size, n_heads, head_dim (of q and k, without the rotated part), value_dim,
    latent_rank, scale, window (None: every earlier token; n: the token itself and the n - 1
    before it), eps (of the latent's norm), sink (whether the softmax has the sink term), gate
    (False; True or "head": one logit per head; "element": one per output channel), rope_dim
    and position (optional), cache_from (optional: index of the layer whose cached rows this
    layer reads; it then has no down projection and no latent norm, and writes nothing).
    tensors: q [nh*(hd+r), H], down [rank+r, H], latent_norm [rank], up_k [nh*hd, rank],
    up_v [nh*vd, rank], sink [nh], gate [nh, H] or [nh*vd, H], o [H, nh*vd]."""

    def __init__(self, spec: PartSpec, ctx: BuildContext):
        super().__init__(spec, ctx)
        p = spec.params
        self.hidden = int(self.param("hidden_size"))
        self.n_heads = int(self.param("n_heads"))
        self.head_dim = int(self.param("head_dim"))
        self.value_dim = int(self.param("value_dim"))
        self.rank = int(self.param("latent_rank"))
        self.scale = float(self.param("scale"))
        self.window = int(p["window"]) if p.get("window") else None
        self.eps = float(self.param("eps"))
        self.has_sink = bool(p.get("sink", False))
        self.gate_kind = {True: "head", False: None, None: None}.get(p.get("gate"), p.get("gate"))
        if self.gate_kind not in (None, "head", "element"):
            raise ValueError(f"latent_attention: unknown gate {self.gate_kind!r} (known: 'head', 'element')")
        self.has_gate = self.gate_kind is not None
        self.rope_dim = int(p.get("rope_dim") or 0)
        self.row = self.rank + self.rope_dim          # what a token caches
        self.cache_from = p.get("cache_from")
        self.position = build_part("position", p["position"], ctx) if self.rope_dim else None
        self.interleaved = bool(self.rope_dim) and p["position"].kind == "rope_pairs"
        self.stacked: torch.Tensor | None = None
        self.up_k = self.up_v = self.o = self.latent_norm = self.sink = None
        self.cache: KVBinding | None = None
        self._tensor_cores: tuple[bool, bool] | None = None

    @classmethod
    def tensor_needs(cls, spec: PartSpec) -> dict[str, TensorNeed]:
        p, t = spec.params, spec.tensors
        h, nh, hd, vd, rank = (int(p[k]) for k in ("hidden_size", "n_heads", "head_dim", "value_dim", "latent_rank"))
        rot = int(p.get("rope_dim") or 0)
        needs = {t["q"]: TensorNeed((nh * (hd + rot), h)), t["up_k"]: TensorNeed((nh * hd, rank)),
                 t["up_v"]: TensorNeed((nh * vd, rank)), t["o"]: TensorNeed((h, nh * vd))}
        if p.get("cache_from") is None:
            needs[t["down"]] = TensorNeed((rank + rot, h))
            needs[t["latent_norm"]] = TensorNeed((rank,), role="vector")
        if p.get("sink"):
            needs[t["sink"]] = TensorNeed((nh,), role="offset")
        if p.get("gate"):
            needs[t["gate"]] = TensorNeed((nh * vd if p["gate"] == "element" else nh, h))
        return needs

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        t = self.spec.tensors
        nh, hd, vd, rank = self.n_heads, self.head_dim, self.value_dim, self.rank
        parts = [tensors[t["q"]]] + ([tensors[t["down"]]] if self.cache_from is None else []) + (
            [tensors[t["gate"]]] if self.has_gate else [])
        self.stacked = torch.cat(parts, dim=0).contiguous()      # q, latent, gate logits from one product
        # q'_h = Wuk_h^T q_h as a product with rows [rank] over dim: the transposed blocks.
        self.up_k = tensors[t["up_k"]].view(nh, hd, rank).transpose(1, 2).contiguous()   # [nh, rank, hd]
        self.up_v = tensors[t["up_v"]].view(nh, vd, rank).contiguous()                   # [nh, vd, rank]
        self.o = tensors[t["o"]].contiguous()
        self.latent_norm = tensors[t["latent_norm"]].float().contiguous() if self.cache_from is None else None
        self.sink = tensors[t["sink"]].float().contiguous() if self.has_sink else None

    def cache_need(self) -> KVCacheNeed | None:
        if self.cache_from is not None:
            return None
        return KVCacheNeed(1, self.row, self.window, self.n_heads, planes=1)

    def cache_read_need(self) -> KVCacheNeed:
        """How this layer reads cached rows, its own or those of the layer `cache_from` names."""
        return KVCacheNeed(1, self.row, self.window, self.n_heads, planes=1)

    def bind_cache(self, binding: KVBinding) -> None:
        self.cache = binding

    def forward(self, h: torch.Tensor, batch) -> torch.Tensor:
        tokens = h.shape[0]
        nh, hd, vd, rank, rot, row = self.n_heads, self.head_dim, self.value_dim, self.rank, self.rope_dim, self.row
        cache = self.cache
        table = batch.tables[cache.group]
        proj = linear(h, self.stacked)
        q = proj[:, : nh * (hd + rot)].view(tokens, nh, hd + rot)
        at = nh * (hd + rot)
        z = None
        if self.cache_from is None:
            z = proj[:, at: at + row]
            at += row
        gate = proj[:, at:] if self.has_gate else None
        q_latent = torch.empty((tokens, nh, row), dtype=h.dtype, device=h.device)
        per_head_linear(q[:, :, :hd], self.up_k, q_latent[:, :, :rank])
        if rot:
            inv_freq, _ = self.position.table()
            ops.latent_rope_write(q, q_latent, z, self.latent_norm, self.eps, rank, rot, inv_freq, self.interleaved,
                                  float(getattr(self.position, "amplitude", 1.0)), batch.pos, batch.entry, table,
                                  cache.k_pool, cache.page_size, batch.status)
        elif z is not None:
            ops.norm_write_paged(z, self.latent_norm, self.eps, batch.pos, batch.entry, table, cache.k_pool,
                                 cache.page_size, batch.status)
        mixed = torch.empty((tokens, nh, row), dtype=h.dtype, device=h.device)
        self.attend(q_latent, mixed, table, batch, gate if self.gate_kind == "head" else None)
        out = torch.empty((tokens, nh, vd), dtype=h.dtype, device=h.device)
        per_head_linear(mixed[:, :, :rank], self.up_v, out)
        flat = out.view(tokens, nh * vd)
        if self.gate_kind == "element":
            ops.sigmoid_gate(flat, gate)
        return linear(flat, self.o)

    # ------------------------------------------------------------------ planning a step
    def _kernels(self) -> tuple[bool, bool]:
        """Whether the tensor-core kernels for single tokens and for prompt portions take this
        layer's shape: all heads share the one latent row, so they are one group of n_heads
        query heads over a "kv head" of size rank."""
        if self._tensor_cores is None:
            dtype = self.ctx.dtype
            self._tensor_cores = (False, False) if CUDA_CORES_ONLY else (
                ops.attention_decode_supports(self.row, self.n_heads, self.cache.page_size, dtype),
                ops.attention_prefill_supports(self.row, self.cache.page_size, dtype))
        return self._tensor_cores

    def slow_path_note(self) -> str | None:
        if self.cache is None or self.ctx.dtype != torch.bfloat16 or all(self._kernels()):
            return None
        return (f"latent attention with rows of {self.row} and {self.n_heads} heads runs on the CUDA-core attention "
                f"kernel (the tensor-core kernels take ranks 32 to 128 in steps of 16, up to 16 heads and pages that "
                f"are multiples of 16 tokens); expect it several times slower")

    def plan_key(self):
        if self.cache is None:
            return None
        return ("latent attention", self.cache.page_size, self.row, self.n_heads, self.window, self.ctx.dtype)

    def plan_step(self, step) -> dict:
        """The tile list of the prompt-portion kernel (int32 [tiles, 4] rows of {first token
        row, rows, position of the first row, block-table row}, the tiles that read the most
        keys first) and the most keys a single token reads."""
        decode_kernel, prefill_kernel = self._kernels()
        plan: dict = {"tiles": None, "max_context": 0}
        if decode_kernel and step.n_decode:
            plan["max_context"] = step.context_bound if step.fixed_shape else max(step.context_lens[: step.n_decode])
        if not prefill_kernel or step.n_decode == step.n_entries:
            return plan
        rows = ops.attention_prefill_tile_rows()
        tiles = []
        for e in range(step.n_decode, step.n_entries):
            n, at = step.query_lens[e], step.first_rows[e]
            start = step.context_lens[e] - n
            tiles += [(at + r, min(rows, n - r), start + r, e) for r in range(0, n, rows)]
        tiles.sort(key=lambda t: -(min(t[2] + t[1], self.window + t[1]) if self.window else t[2] + t[1]))
        plan["tiles"] = np.array(tiles, dtype=np.int32).reshape(len(tiles), 4)
        return plan

    def attend(self, q: torch.Tensor, out: torch.Tensor, table: torch.Tensor, batch, gate) -> None:
        """out[t, h] = gate * sum_j p_j c_j over the latents in reach of token t. In bfloat16 the
        batch's leading single tokens go to the split-key tensor-core kernel and prompt
        portions to the tiled one, both with the sink and the gate in their last step and the
        softmax weights kept in two bfloat16 terms; float32, and shapes those kernels do not
        take, attend on the CUDA-core kernel."""
        cache = self.cache
        tokens = q.shape[0]
        plan = batch.plans.get(self.plan_key()) or {}
        decode_kernel, prefill_kernel = self._kernels()
        n_decode = min(int(batch.n_decode), tokens) if decode_kernel else 0
        if n_decode > 0:
            max_context = plan.get("max_context") or max(batch.host_context_lens[:n_decode])
            if self.window:
                max_context = min(max_context, self.window + 16)
            splits = decode_splits(n_decode, max_context, q.device, self.row, self.n_heads)
            scratch = None
            if splits > 1:
                scratch = torch.empty(ops.attention_decode_scratch_floats(n_decode, self.n_heads, self.row, splits),
                                      dtype=torch.float32, device=q.device)
            extras = ops.attention_extras(q[:n_decode], self.sink, gate[:n_decode] if gate is not None else None, True)
            ops.attention_decode(q[:n_decode], cache.k_pool, cache.v_pool, table, batch.pos[:n_decode],
                                 batch.entry[:n_decode], out[:n_decode], cache.page_size, self.window, self.scale,
                                 splits, scratch, batch.status, extras=extras)
        if n_decode == tokens:
            return
        tiles = plan.get("tiles")
        if prefill_kernel and tiles is not None and n_decode == int(batch.n_decode):
            # (the tile list covers exactly the tokens after the leading single tokens)
            ops.attention_prefill(q, cache.k_pool, cache.v_pool, table, tiles, out, cache.page_size, self.window,
                                  self.scale, batch.status, extras=ops.attention_extras(q, self.sink, gate, True))
            return
        ops.attention_simt(q[n_decode:], cache.k_pool, cache.v_pool, table, batch.pos[n_decode:],
                           batch.entry[n_decode:], out[n_decode:], cache.page_size, self.window, self.scale,
                           batch.status, sinks=self.sink, gate=gate[n_decode:] if gate is not None else None)
