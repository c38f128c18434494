"""Grouped-query attention whose values are its keys, with a short convolution over time on
the projected queries and keys and one norm over each whole projection."""

from __future__ import annotations

import torch

from ..kernels import ops
from .attention import Attention
from .gated_delta import FilterState
from .linear import linear
from .registry import BuildContext, register_part
from .spec import KVCacheNeed, PartSpec, TensorNeed


@register_part("mixer", "conv_attention")
class ConvAttention(Attention):
    """With h the mixer's input:

        u_q = Wq h + bq, u_k = Wk h + bk                    (biases optional)
        y[t] = sum_j c[:, j] * u[t - (taps - 1) + j]         per channel of q and of k, zeros before the start
        q^ = y_q / rms(y_q) * nq over ALL q channels at once, k^ likewise over all k channels
        q, k = rotate(q^), rotate(k^) per head (the "position" PartSpec; `rope_pairs` turns
               neighbouring pairs, `rope` halves), v = y_k: the filtered key before norm and rotation
        a_h = softmax attention of q_h over k_g, v_g (g = h // (heads / kv_heads)) with the base
              class's scale, window, score cap and sink term
        out = Wo (a * sigmoid(Wg h))                         (the gate per element, optional)

    The cache holds the rotated normed keys and, as values, the filtered keys. The last taps - 1
    projected rows of a request (before bias and convolution) are a state slot of its own
    (`state_holders`). Everything the base class knows about attending (kernels by shape, window,
    plans) applies unchanged; what lies between the projection and the cache is one kernel
    (csrc/conv_norm_rope.cu) that also moves the state slot on in steps of single tokens.

    params: hidden_size, n_heads, n_kv_heads, head_dim, taps (1 without the conv tensors: no
    convolution; 1 with them: one factor per channel), norm_eps (with
    the q_norm / k_norm tensors), scale, window, softcap, sink_logit, position. tensors: q [nh*hd,
    H], k [nkv*hd, H], o [H, nh*hd]; optional q_bias [nh*hd], k_bias [nkv*hd], q_conv [nh*hd,
    taps], k_conv [nkv*hd, taps], q_norm [nh*hd], k_norm [nkv*hd], gate [nh*hd, H]."""

    def __init__(self, spec: PartSpec, ctx: BuildContext):
        super().__init__(spec, ctx)
        if self.cache_from is not None or self.qk_norm_eps:
            raise ValueError("conv_attention: cache_from and per-head q/k norms are not supported")
        self.taps = int(spec.params.get("taps") or 1)
        if not 1 <= self.taps <= 16:
            raise ValueError(f"conv_attention: taps must be 1 to 16, got {self.taps}")
        self.norm_eps = float(spec.params.get("norm_eps") or 0.0)
        self.channels = (self.n_heads + self.n_kv) * self.head_dim
        self.filter_state = FilterState(self.taps, self.channels)
        self.interleaved = self.spec.params["position"].kind == "rope_pairs"
        self.bias = self.conv = self.gate_rows = None

    @classmethod
    def tensor_needs(cls, spec: PartSpec) -> dict[str, TensorNeed]:
        p, t = spec.params, spec.tensors
        h, nh, nkv, hd = (int(p[k]) for k in ("hidden_size", "n_heads", "n_kv_heads", "head_dim"))
        taps = int(p.get("taps") or 1)
        needs = {t["q"]: TensorNeed((nh * hd, h)), t["k"]: TensorNeed((nkv * hd, h)), t["o"]: TensorNeed((h, nh * hd))}
        for name, rows in (("q", nh * hd), ("k", nkv * hd)):
            if t.get(name + "_bias"):
                needs[t[name + "_bias"]] = TensorNeed((rows,), role="offset")
            if t.get(name + "_norm"):
                needs[t[name + "_norm"]] = TensorNeed((rows,), role="vector")
            if t.get(name + "_conv"):
                needs[t[name + "_conv"]] = TensorNeed((rows, taps))
        if t.get("gate"):
            needs[t["gate"]] = TensorNeed((nh * hd, h))
        return needs

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        t = self.spec.tensors
        stacked = [tensors[t["q"]], tensors[t["k"]]] + ([tensors[t["gate"]]] if t.get("gate") else [])
        self.qkv = torch.cat(stacked, dim=0).contiguous()      # q, k and the gate logits from one product
        self.gate_rows = bool(t.get("gate"))
        self.o = tensors[t["o"]].contiguous()

        def both(kind: str) -> torch.Tensor | None:
            names = (t.get("q_" + kind), t.get("k_" + kind))
            if not any(names):
                return None
            if kind == "conv" and not all(names):
                raise ValueError("conv_attention: q_conv and k_conv come together")
            nh, nkv, hd = self.n_heads, self.n_kv, self.head_dim
            parts = [tensors[n].float() if n else torch.zeros(rows, device=self.ctx.device)
                     for n, rows in zip(names, (nh * hd, nkv * hd))]
            return torch.cat(parts, dim=0).contiguous()

        self.bias = both("bias")
        self.conv = both("conv")
        if self.conv is None and self.taps > 1:
            raise ValueError("conv_attention: more than one tap needs the q_conv / k_conv tensors")
        self.q_norm = tensors[t["q_norm"]].float().contiguous() if t.get("q_norm") else None
        self.k_norm = tensors[t["k_norm"]].float().contiguous() if t.get("k_norm") else None

    def cache_need(self) -> KVCacheNeed:
        return KVCacheNeed(self.n_kv, self.head_dim, self.window, self.n_heads)

    def state_holders(self) -> list:
        """What else keeps something per request for this mixer: the convolutions' inputs."""
        return [self.filter_state]

    def captures_state_steps(self) -> bool:
        return True

    def _folds_rope(self, tokens, batch, inv_freq, rotary) -> bool:
        return False  # (convolution, norms and rotation are a kernel of their own)

    def native_choice(self, tokens, batch, row_stride):
        return None

    def forward(self, h: torch.Tensor, batch) -> torch.Tensor:
        tokens = h.shape[0]
        nh, nkv, hd, c = self.n_heads, self.n_kv, self.head_dim, self.channels
        cache = self.cache
        table = batch.tables[cache.group]
        proj = linear(h, self.qkv)                             # [T, c (+ nh * hd)]
        q = torch.empty((tokens, nh, hd), dtype=h.dtype, device=h.device)
        inv_freq, rotary = self.position.table()
        states = self.filter_state.states(h)
        single = int(batch.n_decode) == tokens                 # every entry brings one token
        ops.conv_norm_rope_write(proj[:, :c], self.bias, self.conv, states, batch.slots, single, self.q_norm,
                                 self.k_norm, self.norm_eps, inv_freq, rotary, self.interleaved,
                                 float(getattr(self.position, "amplitude", 1.0)), batch.pos, batch.entry, table,
                                 q.view(tokens, nh * hd), cache.k_pool, cache.v_pool, cache.page_size, nh, nkv, hd,
                                 batch.status)
        if self.taps > 1 and not single:
            ops.short_conv_state_strided(proj[:, :c], batch.entry, batch.slots, states)
        out = torch.empty((tokens, nh, hd), dtype=h.dtype, device=h.device)
        self.attend(q, out, table, batch)
        flat = out.view(tokens, nh * hd)
        if self.gate_rows:
            ops.sigmoid_gate(flat, proj[:, c:])
        return linear(flat, self.o)
