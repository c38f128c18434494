"""A routed feed-forward: many small feed-forwards (gated, or plain with the square of relu)
of which each token uses a few, chosen by a router, beside an optional one that every token uses."""

from __future__ import annotations

import os

import torch

from ..kernels import ops
from .linear import activated_linear, gated_feed_forward, linear
from .registry import BuildContext, Part, register_part
from .spec import PartSpec, TensorNeed

# From this many tokens a bfloat16 step sorts its (token, expert) pairs by expert and runs the
# experts as grouped matrix products; below, every pair streams its expert's weights.
GROUPED_MIN_TOKENS = int(os.environ.get("PULSARLM_B200_MOE_GROUPED_MIN_TOKENS", "48"))


@register_part("feed_forward", "moe")
class RoutedExperts(Part):
    """Router (fp32): z = Wr h, s = softmax(z) over all experts, choice scores c = s +
    correction; experts form `groups` equal groups of neighbours, a group's score is its
    largest choice score and only experts of the `keep_groups` best groups can be chosen; the
    `top` largest choice scores are chosen and weigh in with s / (sum of the chosen s + 1e-20).
    Expert e: W_down,e (silu(W_gate,e h) * (W_up,e h)), no biases. The output is the weighted
    sum of the chosen experts' outputs plus, where `shared_size` is given, a shared expert of
    the same form that every token uses.

    Steps of few tokens (and the float32 engine) run the chosen experts pair by pair
    (csrc/moe.cu: every (token, expert) pair streams its expert's weights, sums in fp32,
    nothing depends on the rest of the batch). Longer bfloat16 steps sort the pairs by expert
    on the device and run each projection as one grouped matrix product over the sorted rows.
    No step asks the host which experts were chosen, so steps of single tokens can be
    captured.

    Variants, all parameters: `scores` = "sigmoid" makes s the sigmoid of every logit alone
    (default "softmax"); `group_top` = n makes a group's score the sum of its n largest choice
    scores (default 1); `renormalise` = False leaves the chosen scores as the weights (default
    True); `expert` = "relu2" makes every expert, and the shared one, W_down relu(W_up h)^2 without
    a gate (default "gated_silu"; such experts have no `expert_gate` / `shared_gate` tensors).

    params: hidden_size, expert_size, n_experts, top, groups (default 1), keep_groups
    (default groups), shared_size (optional), scores, group_top, renormalise, expert. tensors: router [E, H], correction [E]
    (optional), experts: a name pattern with `{e}` for gate / up / down
    (`expert_gate`, `expert_up` [F, H], `expert_down` [H, F]), shared_gate, shared_up [Fs, H],
    shared_down [H, Fs]."""

    def __init__(self, spec: PartSpec, ctx: BuildContext):
        super().__init__(spec, ctx)
        p = spec.params
        self.hidden = int(self.param("hidden_size"))
        self.ff = int(self.param("expert_size"))
        self.n_experts = int(self.param("n_experts"))
        self.top = int(self.param("top"))
        self.groups = int(p.get("groups") or 1)
        self.keep = int(p.get("keep_groups") or self.groups)
        self.shared_size = int(p["shared_size"]) if p.get("shared_size") else 0
        self.sigmoid_scores = {"softmax": False, "sigmoid": True}[str(p.get("scores") or "softmax")]
        self.group_top = int(p.get("group_top") or 1)
        self.renormalise = bool(p.get("renormalise", True))
        self.gated = {"gated_silu": True, "relu2": False}[str(p.get("expert") or "gated_silu")]
        if self.n_experts % self.groups or not 0 < self.keep <= self.groups:
            raise ValueError(f"moe: {self.n_experts} experts in {self.groups} groups of which {self.keep} stay")
        if not 0 < self.top <= self.keep * (self.n_experts // self.groups):
            raise ValueError(f"moe: {self.top} experts cannot be chosen from {self.keep} groups of "
                             f"{self.n_experts // self.groups}")
        self.router = self.correction = None
        self.gate_up = self.down = None            # [E, 2F, H] ([E, F, H] without a gate), [E, H, F]
        self.gate_up_t = self.down_t = None        # the same with rows and columns swapped, for the grouped products
        self.shared_gate_up = self.shared_down = None

    @classmethod
    def tensor_needs(cls, spec: PartSpec) -> dict[str, TensorNeed]:
        p, t = spec.params, spec.tensors
        h, f, e = int(p["hidden_size"]), int(p["expert_size"]), int(p["n_experts"])
        gated = str(p.get("expert") or "gated_silu") == "gated_silu"
        needs = {t["router"]: TensorNeed((e, h))}
        if t.get("correction"):
            needs[t["correction"]] = TensorNeed((e,), role="offset")
        for i in range(e):
            if gated:
                needs[t["expert_gate"].format(e=i)] = TensorNeed((f, h))
            needs[t["expert_up"].format(e=i)] = TensorNeed((f, h))
            needs[t["expert_down"].format(e=i)] = TensorNeed((h, f))
        if p.get("shared_size"):
            fs = int(p["shared_size"])
            if gated:
                needs[t["shared_gate"]] = TensorNeed((fs, h))
            needs[t["shared_up"]] = TensorNeed((fs, h))
            needs[t["shared_down"]] = TensorNeed((h, fs))
        return needs

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        t = self.spec.tensors
        self.router = tensors[t["router"]].float().contiguous()
        self.correction = tensors[t["correction"]].float().contiguous() if t.get("correction") else None
        experts = range(self.n_experts)
        if self.gated:
            self.gate_up = torch.stack([torch.cat([tensors[t["expert_gate"].format(e=i)],
                                                   tensors[t["expert_up"].format(e=i)]], dim=0)
                                        for i in experts]).contiguous()
        else:
            self.gate_up = torch.stack([tensors[t["expert_up"].format(e=i)] for i in experts]).contiguous()
        self.down = torch.stack([tensors[t["expert_down"].format(e=i)] for i in experts]).contiguous()
        if self.shared_size:
            self.shared_gate_up = (torch.cat([tensors[t["shared_gate"]], tensors[t["shared_up"]]], dim=0).contiguous()
                                   if self.gated else tensors[t["shared_up"]].contiguous())
            self.shared_down = tensors[t["shared_down"]].contiguous()

    def _grouped(self, h: torch.Tensor) -> bool:
        return (h.dtype == torch.bfloat16 and h.shape[0] >= GROUPED_MIN_TOKENS and self.hidden % 8 == 0
                and self.ff % 8 == 0 and hasattr(torch.nn.functional, "grouped_mm"))

    def forward(self, h: torch.Tensor, batch) -> torch.Tensor:
        tokens = h.shape[0]
        ids, weights = ops.moe_route(h, self.router, self.correction, self.top, self.groups, self.keep,
                                     self.sigmoid_scores, self.group_top, self.renormalise)
        shared = None
        if self.shared_size and self.gated:
            shared = gated_feed_forward(h, self.shared_gate_up, self.shared_down)
        elif self.shared_size:
            shared = activated_linear(linear(h, self.shared_gate_up), None, "relu2", self.shared_down)
        out = torch.empty((tokens, self.hidden), dtype=h.dtype, device=h.device)
        if self._grouped(h):
            # Pairs in expert order; each projection one grouped product over the sorted rows (the
            # library's: operands [rows, K] and [E, K, N] with the experts' last rows as offsets).
            ends, row_of_pair, pair_of_row = ops.moe_sort(ids, self.n_experts)
            x = ops.moe_gather(h, pair_of_row, self.top)
            gate_up = torch.nn.functional.grouped_mm(x, self.gate_up.transpose(1, 2), offs=ends)
            act = torch.empty((x.shape[0], self.ff), dtype=h.dtype, device=h.device)
            if self.gated:
                ops.swiglu(gate_up, act)
            else:
                ops.bias_act(gate_up, None, act, "relu2")
            y = torch.nn.functional.grouped_mm(act, self.down.transpose(1, 2), offs=ends)
            ops.moe_combine(y, row_of_pair, weights, shared, out)
            return out
        act = torch.empty((tokens * self.top, self.ff), dtype=h.dtype, device=h.device)
        if self.gated:
            ops.moe_gate_up(h, self.gate_up, ids, act)
        else:
            ops.moe_up(h, self.gate_up, ids, act)
        ops.moe_down(act, self.down, ids, weights, shared, out)
        return out
