"""The Puvirax decoder in the engine against the plain implementation (plain_puvirax.py):
each mechanism's kernel alone, then whole models under every kind of schedule."""

from __future__ import annotations

import json

import pytest
import torch

import harness
import plain_puvirax as plain
import puvirax_tiny as pt

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _ops():
    from pulsarlm_b200.kernels import ops

    ops.require_device()
    return ops


def _i32(values):
    return torch.tensor(values, dtype=torch.int32, device=DEV)


def _bar(dtype) -> float:
    return 1e-5 if dtype == torch.float32 else 1e-2


def _paged(lengths, page, gen):
    """A block table over pages handed out in a scrambled order."""
    n_pages = sum(-(-n // page) for n in lengths) + 2
    order = torch.randperm(n_pages, generator=gen).tolist()
    table = torch.full((len(lengths), max(-(-n // page) for n in lengths)), -1, dtype=torch.int32)
    for e, n in enumerate(lengths):
        for j in range(-(-n // page)):
            table[e, j] = order.pop()
    return n_pages, table


# --------------------------------------------------------------------------- mechanisms alone

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_pair_embedding_reads_the_token_before_from_the_step_or_the_slot(dtype):
    """Three requests in slots 2, 0 and 3: portions whose first row needs the last token of the step before,
    single tokens, a request's very first token (the table's last row), a slot that is taken again."""
    ops = _ops()
    gen = torch.Generator().manual_seed(5)
    vocab, width, buckets = 50, 24, 13
    cfg = {"embedding": {"bigram": {"buckets": buckets, "mul_prev": 7, "mul_cur": 3}}}
    table = torch.randn(vocab, width, generator=gen).to(dtype)
    pairs = torch.randn(buckets + 1, width, generator=gen).to(dtype)
    state = torch.full((5,), 49, dtype=torch.int32, device=DEV)   # (what an earlier owner of a slot left behind)
    seqs = {0: torch.randint(0, vocab, (9,), generator=gen).tolist(), 1: torch.randint(0, vocab, (6,), generator=gen).tolist(),
            2: torch.randint(0, vocab, (4,), generator=gen).tolist()}
    slot_of = {0: 2, 1: 0, 2: 3}
    want = {r: plain.pair_embedding(s, table.double(), pairs.double(), cfg) for r, s in seqs.items()}
    fed = {r: 0 for r in seqs}
    # (entries of one token lead a step)
    for step in ([(0, 4), (1, 2)], [(2, 1), (0, 1), (1, 3)], [(0, 1), (1, 1), (2, 1)], [(2, 2), (0, 3)]):
        tokens, pos, entry, slots, rows = [], [], [], [], []
        for e, (r, n) in enumerate(step):
            tokens += seqs[r][fed[r]: fed[r] + n]
            pos += list(range(fed[r], fed[r] + n))
            entry += [e] * n
            slots.append(slot_of[r])
            rows.append((r, fed[r], n))
            fed[r] += n
        out = torch.empty(len(tokens), width, dtype=torch.float32, device=DEV)
        ops.pair_embed(table.to(DEV), pairs.to(DEV), _i32(tokens), _i32(pos), _i32(entry), _i32(slots), state, out, 7, 3,
                       all(n == 1 for _, n in step))
        at = 0
        for r, start, n in rows:
            assert plain.relative_error_of(out[at: at + n].cpu(), want[r][start: start + n]) < 1e-6, (step, r)
            at += n
    assert [int(state[slot_of[r]]) for r in seqs] == [seqs[r][fed[r] - 1] for r in seqs]


@pytest.mark.parametrize("mode,heads,kv,dim,vdim,rotary", [
    ("unit_after", 4, 2, 24, 16, 8), ("unit_after", 3, 3, 8, 16, 8), ("unit_after", 2, 1, 40, 40, 0),
    ("per_head", 4, 2, 16, 24, 0), ("per_head", 5, 1, 72, 8, 0), ("whole", 6, 2, 8, 24, 0), ("whole", 2, 2, 20, 4, 0),
    ("none", 2, 1, 16, 16, 16)])
@pytest.mark.parametrize("mix", [False, True])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norms_rotation_and_value_mixing_on_the_way_to_the_cache(mode, heads, kv, dim, vdim, rotary, mix, dtype):
    """q, k, v as slices of one projection; a short step (few heads a block) and a long one (a token a block);
    rows of the common size with zeros past their own columns; pages in a scrambled order."""
    ops = _ops()
    gen = torch.Generator().manual_seed(heads * 100 + dim)
    eps, lam, page = 1e-5, 0.3, 8
    row = -(-max(dim, vdim) // 16) * 16
    rot = {"base": 100.0, "dims": rotary, "scaling": {"factor": 2.0, "low": 1.0, "high": 3.0, "original": 32}}
    inv_freq = plain.banded_frequencies(rot).to(DEV) if rotary else None
    for lengths, starts, spare in (([5, 3], [9, 0], 3), ([70, 33], [3, 20], 3), ([300, 40], [7, 0], 8), ([260], [0], 5)):
        tokens = sum(lengths)
        width = heads * dim + kv * dim + kv * vdim
        proj = (torch.randn(tokens, width + spare, generator=gen) * 2).to(dtype)
        q = proj[:, : heads * dim].view(tokens, heads, dim)
        k = proj[:, heads * dim: (heads + kv) * dim].view(tokens, kv, dim)
        v = proj[:, (heads + kv) * dim: width].view(tokens, kv, vdim)
        first = torch.randn(tokens, kv, vdim, generator=gen).to(dtype) if mix else None
        wq = 1.0 + 0.3 * torch.randn(heads * dim if mode == "whole" else dim, generator=gen)
        wk = 1.0 + 0.3 * torch.randn(kv * dim if mode == "whole" else dim, generator=gen)
        pos = torch.cat([torch.arange(s, s + n) for s, n in zip(starts, lengths)])
        entry = torch.cat([torch.full((n,), e) for e, n in enumerate(lengths)])
        qd, kd = q.double(), k.double()
        if mode == "per_head":
            qd, kd = plain.rms(qd, eps) * wq.double(), plain.rms(kd, eps) * wk.double()
        elif mode == "whole":
            qd = (plain.rms(qd.reshape(tokens, -1), eps) * wq.double()).view(tokens, heads, dim)
            kd = (plain.rms(kd.reshape(tokens, -1), eps) * wk.double()).view(tokens, kv, dim)
        if rotary:
            qd, kd = plain.rotate_halves(qd, pos, rot), plain.rotate_halves(kd, pos, rot)
        if mode == "unit_after":
            qd, kd = plain.rms(qd, eps), plain.rms(kd, eps)
        vd = plain.mixed_values(v.double(), first.double() if mix else None, lam)
        n_pages, table = _paged([s + n for s, n in zip(starts, lengths)], page, gen)
        dev = proj.to(DEV)
        weights = (wq.to(DEV), wk.to(DEV)) if mode in ("per_head", "whole") else (None, None)

        def run(lo, hi):
            """Tokens [lo, hi) of the step as a launch of their own, into fresh pools."""
            k_pool = torch.full((n_pages, kv, page, row), 7.0, dtype=dtype, device=DEV)
            v_pool = torch.full_like(k_pool, 7.0)
            q_out = torch.full((hi - lo, heads, row), 7.0, dtype=dtype, device=DEV)
            part = dev[lo:hi]
            ops.norm_rope_mix_write(part[:, : heads * dim].view(hi - lo, heads, dim),
                                    part[:, heads * dim: (heads + kv) * dim].view(hi - lo, kv, dim),
                                    part[:, (heads + kv) * dim: width].view(hi - lo, kv, vdim),
                                    first.to(DEV)[lo:hi] if mix else None, lam, q_out, pos[lo:hi].int().to(DEV),
                                    entry[lo:hi].int().to(DEV), table.to(DEV), k_pool, v_pool, page, inv_freq, rotary, mode,
                                    weights[0], weights[1], eps)
            return q_out, k_pool, v_pool

        q_out, k_pool, v_pool = run(0, tokens)
        bar = _bar(dtype)
        assert plain.relative_error_of(q_out[:, :, :dim].cpu(), qd) < bar
        assert row == dim or float(q_out[:, :, dim:].abs().max()) == 0.0
        for t in range(tokens):
            p, e = int(pos[t]), int(entry[t])
            got_k = k_pool[table[e, p // page], :, p % page].cpu()
            got_v = v_pool[table[e, p // page], :, p % page].cpu()
            assert plain.relative_error_of(got_k[:, :dim], kd[t]) < bar and plain.relative_error_of(got_v[:, :vdim], vd[t]) < bar
            assert float(got_k[:, dim:].abs().sum()) == 0.0 and float(got_v[:, vdim:].abs().sum()) == 0.0
        if tokens >= 256:
            # a long step takes another kernel than a short one: the same bits all the same
            q_short, k_short, v_short = run(10, 60)
            assert torch.equal(q_short, q_out[10:60])
            for t in range(10, 60):
                p, e = int(pos[t]), int(entry[t])
                at = (table[e, p // page], slice(None), p % page)
                assert torch.equal(k_short[at], k_pool[at]) and torch.equal(v_short[at], v_pool[at])


@pytest.mark.parametrize("heads,row", [(4, 96), (3, 10), (32, 64)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gate_per_head_after_attention(heads, row, dtype):
    """The gate of a layer whose attention runs on the plain kernels: one sigmoid per (token, head) over the head's
    row, the logits read as columns of a wider matrix."""
    ops = _ops()
    gen = torch.Generator().manual_seed(row)
    x = torch.randn(19, heads, row, generator=gen).to(dtype)
    wide = torch.randn(19, heads + 5, generator=gen).to(dtype)
    want = x.double() * torch.sigmoid(wide[:, 2: 2 + heads].double())[:, :, None]
    got = x.to(DEV)
    ops.sigmoid_gate_heads(got, wide.to(DEV)[:, 2: 2 + heads])
    assert plain.relative_error_of(got.cpu(), want) < _bar(dtype)


def _attention_case(gen, lengths, heads, kv, dim, page, dtype, rows, far, spike_at, queries):
    """Paged keys and values of some requests, a bias table, queries for chosen (request, position) pairs; a key at
    distance `spike_at` of every query lined up with head 0's query so that it dominates where it is in reach."""
    n_pages, table = _paged(lengths, page, gen)
    keys = [torch.randn(n, kv, dim, generator=gen).to(dtype) for n in lengths]
    values = [torch.randn(n, kv, dim, generator=gen).to(dtype) for n in lengths]
    q_full = [torch.randn(n, heads, dim, generator=gen).to(dtype) for n in lengths]
    rel = torch.randn(rows, heads, generator=gen) if rows else None
    if spike_at is not None:
        for e, p in queries:
            if p - spike_at >= 0:
                direction = q_full[e][p, 0].float() / q_full[e][p, 0].float().norm()
                keys[e][p - spike_at, 0] = (40.0 * direction).to(dtype)
    k_pool = torch.zeros(n_pages, kv, page, dim, dtype=dtype, device=DEV)
    v_pool = torch.zeros_like(k_pool)
    for e, n in enumerate(lengths):
        for j in range(n):
            k_pool[table[e, j // page], :, j % page] = keys[e][j].to(DEV)
            v_pool[table[e, j // page], :, j % page] = values[e][j].to(DEV)
    return table, keys, values, q_full, rel, k_pool, v_pool


def _attention_wanted(keys, values, q_full, rel, far, scale, window, queries):
    full = []
    for e in range(len(keys)):
        n = keys[e].shape[0]
        bias = plain.distance_bias(rel.double(), far, n) if rel is not None else None
        full.append(plain.softmax_attention(q_full[e].double(), keys[e].double(), values[e].double(), scale, window, bias))
    return torch.stack([full[e][p] for e, p in queries])


@pytest.mark.parametrize("window", [None, 7, 16, 21])
@pytest.mark.parametrize("spike", [None, "inside", "outside", "far"])
@pytest.mark.parametrize("rows,far", [(None, None), (12, 40.0), (4, 5.0), (16, 128.0)])
def test_attention_with_a_bias_by_distance_at_window_edges(window, spike, rows, far):
    """The CUDA-core kernel in both dtypes: grouped heads over paged keys, single tokens and prompt rows at page
    borders, a gate per head; one key just inside the window, just outside it, or far back dominates where it is in
    reach; the bias table's rows are spread over distances below and above its reach."""
    from pulsarlm_b200.parts.normed_attention import bias_by_distance

    ops = _ops()
    if spike in ("inside", "outside") and window is None:
        pytest.skip("no window, no edge")
    heads, kv, dim, page, scale = 6, 2, 16, 8, 0.3
    lengths = [170, 33, 8, 129]
    distance = {None: None, "inside": (window or 0) - 1, "outside": window, "far": 150}[spike]
    queries = [(e, p) for e, n in enumerate(lengths) for p in sorted({0, 1, 2, n // 2, n - 2, n - 1}) if p >= 0]
    for dtype in (torch.float32, torch.bfloat16):
        gen = torch.Generator().manual_seed(11)
        table, keys, values, q_full, rel, k_pool, v_pool = _attention_case(gen, lengths, heads, kv, dim, page, dtype, rows,
                                                                          far, distance, queries)
        gate = torch.randn(len(queries), heads, generator=gen).to(dtype)
        want = _attention_wanted(keys, values, q_full, rel, far, scale, window, queries)
        want = want * torch.sigmoid(gate.double())[:, :, None]
        q = torch.stack([q_full[e][p] for e, p in queries]).to(DEV)
        out = torch.empty_like(q)
        ops.attention_simt(q, k_pool, v_pool, table.to(DEV), _i32([p for _, p in queries]), _i32([e for e, _ in queries]),
                           out, page, window, scale, gate=gate.to(DEV),
                           distance_bias=bias_by_distance(rel.to(DEV), far) if rows else None)
        assert plain.relative_error_of(out.cpu(), want) < (1e-5 if dtype == torch.float32 else 1e-2), (dtype, window, spike)


@pytest.mark.parametrize("dim,heads,kv", [(32, 6, 2), (96, 4, 1), (64, 3, 3), (48, 8, 1), (64, 4, 2), (128, 8, 1)])
@pytest.mark.parametrize("window,distance", [(None, None), (None, 150), (24, 23), (24, 24), (37, 36), (37, 37), (16, 15)])
@pytest.mark.parametrize("rows,far", [(12, 40.0), (32, 64.0)])
def test_tensor_core_attention_takes_the_bias_and_the_gate(dim, heads, kv, window, distance, rows, far):
    """The bfloat16 kernels for single tokens (any number of key shares) and for prompt portions with a bias by
    distance and a gate per head; one key at a chosen distance (a window's last key, the first one outside, or far
    back) is lined up with the query."""
    from pulsarlm_b200.parts.normed_attention import bias_by_distance

    ops = _ops()
    page, scale, dtype = 16, 0.25, torch.bfloat16
    lengths = [200, 33, 16, 129]
    if not (ops.attention_decode_supports(dim, heads // kv, page, dtype) and ops.attention_prefill_supports(dim, page, dtype)):
        pytest.skip("a shape for the CUDA-core kernel")

    def case(queries, seed):
        gen = torch.Generator().manual_seed(seed)
        table, keys, values, q_full, rel, k_pool, v_pool = _attention_case(gen, lengths, heads, kv, dim, page, dtype, rows,
                                                                          far, distance, queries)
        gate = torch.randn(len(queries), heads, generator=gen).to(dtype)
        plain_want = _attention_wanted(keys, values, q_full, rel, far, scale, window, queries)
        want = plain_want * torch.sigmoid(gate.double())[:, :, None]
        q = torch.stack([q_full[e][p] for e, p in queries]).to(DEV)
        ungated.append(plain_want)
        return q, k_pool, v_pool, table.to(DEV), gate.to(DEV), bias_by_distance(rel.to(DEV), far), want

    ungated: list = []

    queries = [(e, n - 1) for e, n in enumerate(lengths)] + [(0, 0), (0, 1), (3, 64)]
    q, k_pool, v_pool, table, gate, bias, want = case(queries, 21)
    pos, entry = _i32([p for _, p in queries]), _i32([e for e, _ in queries])
    for splits in (1, 2, 5):
        scratch = torch.empty(ops.attention_decode_scratch_floats(len(queries), heads, dim, splits),
                              dtype=torch.float32, device=DEV) if splits > 1 else None
        out = torch.empty_like(q)
        ops.attention_decode(q, k_pool, v_pool, table, pos, entry, out, page, window, scale, splits, scratch,
                             extras=ops.attention_extras(q, None, gate, True, 0.0, bias))
        assert plain.relative_error_of(out.cpu(), want) < 1e-2, ("single tokens", splits)
    spans = [(0, 120, 200), (3, 0, 129), (1, 32, 33), (2, 0, 16)]
    queries = [(e, p) for e, lo, hi in spans for p in range(lo, hi)]
    q, k_pool, v_pool, table, gate, bias, want = case(queries, 22)
    tile_rows = ops.attention_prefill_tile_rows()
    tiles, at = [], 0
    for e, lo, hi in spans:
        for r in range(0, hi - lo, tile_rows):
            tiles.append((at + r, min(tile_rows, hi - lo - r), lo + r, e))
        at += hi - lo
    out = torch.empty_like(q)
    ops.attention_prefill(q, k_pool, v_pool, table, _i32(tiles), out, page, window, scale,
                          extras=ops.attention_extras(q, None, gate, True, 0.0, bias))
    assert plain.relative_error_of(out.cpu(), want) < 1e-2, "prompt rows"
    # the tcgen05 kernel's build with a bias (keys and values of a page side by side, heads in pairs per kv head)
    both = torch.stack([k_pool, v_pool], dim=1).contiguous()
    if (heads // kv) % 2 == 0 and ops.attention_prefill_tcgen05_supports(q, both[:, 0], page):
        out = torch.empty_like(q)
        ops.attention_prefill_tcgen05(q, both[:, 0], both[:, 1], table, _i32(tiles), out, page, window, scale,
                                      distance_bias=bias)
        assert plain.relative_error_of(out.cpu(), ungated[-1]) < 1e-2, "prompt rows on tcgen05"
        for splits in (2, 3):
            scratch = torch.empty(ops.attention_prefill_scratch_floats(q.shape[0], heads, dim, splits), dtype=torch.float32,
                                  device=DEV)
            out = torch.empty_like(q)
            ops.attention_prefill_tcgen05(q, both[:, 0], both[:, 1], table, _i32(tiles), out, page, window, scale, None,
                                          splits, scratch, distance_bias=bias)
            assert plain.relative_error_of(out.cpu(), ungated[-1]) < 1e-2, ("prompt rows on tcgen05", splits)


@pytest.mark.parametrize("experts,top,groups", [(8, 2, (4, 2)), (16, 3, (4, 3)), (6, 2, (3, 2)), (5, 1, None), (12, 4, (3, 1)),
                                                (64, 6, (8, 3)), (9, 2, (9, 4))])
@pytest.mark.parametrize("tokens", [3, 300])
def test_router_with_sigmoid_scores_and_groups_ranked_by_their_two_best(experts, top, groups, tokens):
    """Choice scores are mostly negative here (large negative corrections on some experts), so a group that was shut out
    by counting as 0 instead of minus infinity would be chosen; weights are the plain scores, not renormalised."""
    ops = _ops()
    gen = torch.Generator().manual_seed(experts)
    hidden = 40
    h = torch.randn(tokens, hidden, generator=gen)
    router = torch.randn(experts, hidden, generator=gen) * 0.5
    correction = torch.randn(experts, generator=gen) - 1.0
    r = {"experts": experts, "top": top}
    if groups:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    ids, weights = plain.route(h.double(), router.double(), correction.double(), r)
    got_ids, got_w = ops.moe_route(h.to(DEV), router.to(DEV), correction.to(DEV), top, groups[0] if groups else 1,
                                   groups[1] if groups else 1, True, 2, False)
    assert torch.equal(got_ids.cpu().long(), ids)
    assert plain.relative_error_of(got_w.cpu(), weights) < 1e-5


@pytest.mark.parametrize("tokens", [5, 130])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_routed_experts_without_gates(tokens, dtype):
    """The feed-forward part alone, few tokens (every pair streams its expert) and many (grouped products)."""
    from pulsarlm_b200.parts.registry import BuildContext, build_part
    from pulsarlm_b200.parts.spec import PartSpec

    _ops()
    gen = torch.Generator().manual_seed(3)
    td = torch.float32 if dtype == "float32" else torch.bfloat16
    width, ff, experts, top, shared = 48, 24, 8, 3, 40
    mlp = pt.routed(ff, experts, top, (4, 3), shared)
    w = {"router": torch.randn(experts, width, generator=gen) * 0.5, "correction": torch.randn(experts, generator=gen) * 0.3,
         "shared.up": torch.randn(shared, width, generator=gen) / width ** 0.5,
         "shared.down": torch.randn(width, shared, generator=gen) / shared ** 0.5}
    for e in range(experts):
        w[f"e{e}.up"] = torch.randn(ff, width, generator=gen) / width ** 0.5
        w[f"e{e}.down"] = torch.randn(width, ff, generator=gen) / ff ** 0.5
    w = {k: v.to(td) for k, v in w.items()}
    h = torch.randn(tokens, width, generator=gen).to(td)
    want = plain.routed_ff(h.double(), {k: v.double() for k, v in w.items()}, mlp, lambda t: t)
    spec = PartSpec("moe", {"hidden_size": width, "expert_size": ff, "n_experts": experts, "top": top, "groups": 4,
                            "keep_groups": 3, "shared_size": shared, "scores": "sigmoid", "group_top": 2,
                            "renormalise": False, "expert": "relu2"},
                    {"router": "router", "correction": "correction", "expert_up": "e{e}.up", "expert_down": "e{e}.down",
                     "shared_up": "shared.up", "shared_down": "shared.down"})
    part = build_part("feed_forward", spec, BuildContext(td, torch.device(DEV)))
    part.load({k: v.to(DEV) for k, v in w.items()})
    got = part.forward(h.to(DEV), None)
    assert plain.relative_error_of(got.cpu(), want) < (1e-5 if dtype == "float32" else 2e-2)


# --------------------------------------------------------------------------- whole models

def _model(key, dtype, seed=1, sharp=1.0):
    return pt.TinyPuvirax(key, dtype, seed, sharp=sharp)


def _portions(tokens, cuts, request="p", want_all=True):
    assert sum(cuts) == len(tokens)
    steps, at = [], 0
    for n in cuts:
        steps.append(([(request, tokens[at: at + n], list(range(n)) if want_all else [n - 1])], []))
        at += n
    return steps


@pytest.mark.parametrize("key", ["A", "B", "C"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_prompts_and_their_first_tokens(key, dtype):
    tm = _model(key, dtype)
    runner = tm.runner(24)
    tokens = {"p": pt.random_tokens(tm.cfg, 75, 3), "q": pt.random_tokens(tm.cfg, 5, 4), "r": pt.random_tokens(tm.cfg, 1, 5)}
    got = harness.replay(runner, [([("p", tokens["p"], list(range(75)))], ["p"]),
                                  ([("q", tokens["q"], list(range(5)))], ["q"]),
                                  ([("r", tokens["r"], [0])], ["r"])])
    tm.check(tokens, got, f"{key} whole")


def test_residual_stream_after_every_layer():
    """float32: the stream after each layer of a prompt fed in two portions, against the plain
    implementation's, so that a fault is placed at its layer."""
    from pulsarlm_b200.engine.runner import StepEntry
    from pulsarlm_b200.parts.basic import settle_pending

    for key in ("A", "B", "C"):
        tm = _model(key, "float32")
        tokens = pt.random_tokens(tm.cfg, 37, 9)
        want: list = []
        plain.forward(tm.cfg, tm.plain_weights, tokens, streams=want)
        runner = tm.runner(8)
        seen: list = []
        for block in runner.model.blocks:
            def wrapped(x, delta, batch, inner=block.forward):
                x, pending = inner(x, delta, batch)
                settled = x.clone()
                settle_pending(settled, pending)
                seen.append(settled.cpu())
                return x, pending
            block.forward = wrapped
        runner.step([StepEntry("p", tokens[:20], [19])])
        runner.step([StepEntry("p", tokens[20:], [16])])
        layers = len(tm.cfg["layers"])
        for i in range(layers):
            got = torch.cat([seen[i], seen[layers + i]])
            assert plain.relative_error_of(got, want[i]) < 2e-5, (key, i)


@pytest.mark.parametrize("key", ["A", "B", "C"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prefill_then_token_by_token(key, dtype):
    """A prompt in one step, then 70 tokens one by one: past every window and over page borders."""
    tm = _model(key, dtype)
    runner = tm.runner(24)
    tokens = {"p": pt.random_tokens(tm.cfg, 110, 5)}
    steps = [([("p", tokens["p"][:40], [0, 1, 39])], [])]
    steps += [([("p", [tokens["p"][i]], [0])], []) for i in range(40, 110)]
    tm.check(tokens, harness.replay(runner, steps), f"{key} decode")


@pytest.mark.parametrize("key", ["A", "B", "C"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_token_by_token_from_the_start(key, dtype):
    """The first tokens of a sequence: the pair table's last row, then the slot's token every step."""
    tm = _model(key, dtype)
    runner = tm.runner(8)
    tokens = {"p": pt.random_tokens(tm.cfg, 30, 6)}
    steps = [([("p", [t], [0])], []) for t in tokens["p"]]
    tm.check(tokens, harness.replay(runner, steps), f"{key} from the start")


@pytest.mark.parametrize("key", ["A", "B", "C"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_portions_of_many_sizes(key, dtype):
    tm = _model(key, dtype)
    runner = tm.runner(24)
    tokens = {"p": pt.random_tokens(tm.cfg, 150, 7)}
    cuts = [2, 2, 3, 1, 1, 7, 16, 2, 33, 1, 2, 17, 31, 2, 30]
    tm.check(tokens, harness.replay(runner, _portions(tokens["p"], cuts)), f"{key} portions")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_float32_bits_do_not_depend_on_the_cut(dtype):
    """In float32 every kernel adds in an order fixed by the token's own place: logits of a prompt
    fed whole and fed in portions are equal bit for bit. (bfloat16: within rounding.)"""
    tm = _model("A", dtype)
    tokens = pt.random_tokens(tm.cfg, 90, 8)
    whole = harness.replay(tm.runner(12), [([("p", tokens, list(range(90)))], [])])["p"]
    cut = harness.replay(tm.runner(12), _portions(tokens, [5, 1, 2, 40, 1, 1, 3, 37]))["p"]
    if dtype == "float32":
        for position in range(90):
            assert torch.equal(whole[position], cut[position]), position
        return
    # (a rounding may tip a router's close call, which moves a row by more than a rounding: most rows are held tight)
    errors = sorted(pt.relative_error(cut[position], whole[position]) for position in range(90))
    assert errors[-1] < 0.25 and errors[45] < 2e-2, errors[-5:]


@pytest.mark.parametrize("key", ["A", "C"])
@pytest.mark.parametrize("sharp", [3.0, 6.0])
def test_sharp_attention_shows_every_key_in_reach(key, sharp):
    """float32, scores multiplied so that each softmax rests on a few keys: a window one token off, a
    far key lost with its page or a bias row read at the wrong distance would move these logits by
    orders more than the bar. Prompt portions whose cuts fall just before, at and just after every
    window's edge, then single tokens until every window has passed over decoded tokens, with
    pages of 16 and of 64."""
    tm = _model(key, "float32", seed=7, sharp=sharp)
    windows = sorted({(layer["mixer"].get("mask") or {}).get("size") for layer in tm.cfg["layers"]} - {None})
    n = 2 * max(windows) + 90
    tokens = {"p": pt.random_tokens(tm.cfg, n, 12)}
    first = max(windows) + 1
    cuts = [windows[0] - 1, 1, 1, first - windows[0] - 1, 2, 15, 1, 16]
    cuts = [c for c in cuts if c > 0]
    rest = n - sum(cuts)
    for page in (16, 64):
        steps = _portions(tokens["p"], cuts + [1] * rest)
        tm.check(tokens, harness.replay(tm.runner(-(-n // page) + 1, page=page), steps), f"{key} sharp x{sharp:g}")
    # the sharpening does what it is for: dropping the oldest key in reach moves the logits
    plain_logits = tm.plain_logits(tokens["p"])
    narrower = json.loads(json.dumps(tm.cfg))
    for layer in narrower["layers"]:
        if (layer["mixer"].get("mask") or {}).get("size"):
            layer["mixer"]["mask"]["size"] -= 1
    off_by_one = plain.forward(narrower, tm.plain_weights, tokens["p"])
    assert pt.relative_error(off_by_one, plain_logits) > 50 * pt.TOLERANCE["float32"]


@pytest.mark.parametrize("key", ["A", "C"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixed_batches_and_reused_pages_and_slots(key, dtype):
    """Up to three live requests of unequal lengths, portions beside single tokens, requests
    that pause, end and are followed by new ones in the same slots and pages (the pool is as
    small as the schedule allows)."""
    tm = _model(key, dtype)
    page = tm.page
    runner = tm.runner(3 * (-(-100 // page) + 1), slots=3)
    lengths = {"a": 100, "b": 37, "c": 64, "d": 90, "e": 3, "f": 45}
    tokens = {r: pt.random_tokens(tm.cfg, n, 10 + i) for i, (r, n) in enumerate(lengths.items())}
    fed = {r: 0 for r in lengths}

    def take(r, n):
        n = min(n, lengths[r] - fed[r])
        part = tokens[r][fed[r]: fed[r] + n]
        fed[r] += n
        return (r, part, list(range(n)))

    steps = []

    def step(*parts):
        entries = [take(r, n) for r, n in parts if fed[r] < lengths[r]]
        ends = [r for r, _, _ in entries if fed[r] == lengths[r]]
        if entries:
            steps.append((entries, ends))

    step(("a", 30), ("b", 2))
    step(("a", 1), ("b", 33), ("c", 17))
    step(("b", 1), ("c", 2))
    step(("a", 50), ("b", 1))            # b ends: its slot and pages go to d
    step(("a", 1), ("c", 40), ("d", 16))
    for _ in range(6):
        step(("a", 1), ("c", 1), ("d", 1))
    step(("a", 19), ("d", 2))            # a ends
    step(("c", 5), ("d", 60), ("e", 3))  # c, e end (e within one step)
    step(("d", 11), ("f", 44))
    step(("d", 1), ("f", 1))
    assert all(fed[r] == lengths[r] for r in lengths)
    got = harness.replay(runner, steps)
    tm.check(tokens, got, f"{key} mixed")
    stats = runner.cache.stats()
    assert stats["slots_used"] == 0 and all(g["used"] == 0 for g in stats["groups"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_batch_equals_each_request_alone(dtype):
    tm = _model("C", dtype)
    tokens = {r: pt.random_tokens(tm.cfg, n, 20 + i) for i, (r, n) in enumerate({"a": 50, "b": 9, "c": 33}.items())}
    alone = {}
    for r, t in tokens.items():
        alone.update(harness.replay(tm.runner(8), [([(r, t[:-3], [len(t) - 4])], [])] +
                                    [([(r, [t[i]], [0])], []) for i in range(len(t) - 3, len(t))]))
    runner = tm.runner(16)
    steps = [([(r, t[:-3], [len(t) - 4]) for r, t in tokens.items()], [])]
    steps += [([(r, [t[len(t) - 3 + i]], [0]) for r, t in tokens.items()], []) for i in range(3)]
    together = harness.replay(runner, steps)
    errors = []
    for r in tokens:
        for position, row in alone[r].items():
            if dtype == "float32":
                assert torch.equal(row, together[r][position])
            else:
                errors.append(pt.relative_error(together[r][position], row))
    if errors:
        errors.sort()
        assert errors[-1] < 0.25 and errors[len(errors) // 2] < 2e-2, errors[-5:]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(dtype):
    """400 tokens one by one: pages of the windowed layers are given back and used again while the
    first tokens stay in reach of the layers without a window."""
    tm = _model("B", dtype)
    runner = tm.runner(16)
    tokens = {"p": pt.random_tokens(tm.cfg, 400, 30)}
    steps = [([("p", tokens["p"][:4], [3])], [])]
    steps += [([("p", [tokens["p"][i]], [0] if i % 9 == 0 or i > 390 else [])], []) for i in range(4, 400)]
    tm.check(tokens, harness.replay(runner, steps), "B long decoding")


def test_a_far_token_is_still_seen():
    """Two prompts that differ in their first token only: 300 tokens on, far past every window and past
    the bias tables' reach, the logits still differ (the layers without a window see every key), and
    the engine reproduces the difference, in a prompt and in a decoded token."""
    tm = _model("A", "float32", sharp=3.0)
    base = pt.random_tokens(tm.cfg, 301, 40)
    other = [(base[0] + 1) % tm.cfg["vocab"]] + base[1:]
    tokens = {"x": base, "y": other}
    got = harness.replay(tm.runner(48), [([("x", base[:300], [299]), ("y", other[:300], [299])], []),
                                         ([("x", base[300:], [0]), ("y", other[300:], [0])], ["x", "y"])])
    tm.check(tokens, got, "A far token")
    for position in (299, 300):
        want = tm.plain_logits(base)[position] - tm.plain_logits(other)[position]
        assert want.abs().max() > 1e-3
        assert pt.relative_error(got["x"][position] - got["y"][position], want) < 0.05


def test_sizes_come_from_the_configuration():
    """Values that a given model may leave equal to one another or at 1: one head, one kv head for many
    query heads, a window of 1 (a token sees only itself), a bias table of two rows, a rotary width of
    the whole head and of two columns, value sizes unlike the key sizes, one expert chosen of two, all
    groups kept, no feed-forward anywhere else, a scale of 1, a pair table of one bucket."""
    cfg, rows = pt._config(50, 32, 1e-3, 1.0, (1, 1, 1), [
        pt.biased_layer("attention_2", 1, 1, 8, 4, 2, 3, None, window=1, scale=1.0, v_mix=False),
        pt.rotary_layer(5, 1, 8, 12, 8, pt.routed(8, 2, 1, (2, 2)), base=10.0),
        pt.biased_layer("attention_3", 3, 3, 4, 20, 6, 4, None, v_mix=False),
        pt.rotary_layer(2, 1, 16, 12, 2, None, scale=1.0, bands=(2.0, 0.5, 2.0, 8)),
        pt.biased_layer("attention_2", 4, 1, 24, 12, 8, 200, pt.dense(8), window=2)])
    for dtype in ("float32", "bfloat16"):
        tm = pt.TinyPuvirax("-", dtype, cfg=cfg, rows=rows)
        tokens = {"p": pt.random_tokens(cfg, 40, 50)}
        steps = [([("p", tokens["p"][:20], list(range(20)))], [])]
        steps += [([("p", [t], [0])], []) for t in tokens["p"][20:]]
        tm.check(tokens, harness.replay(tm.runner(8), steps), "sizes of one")


def test_odd_sizes_and_a_larger_model():
    """A width that is no multiple of four with key and value sizes that are no multiples of eight (every kernel's
    plain form), and a model of wider rows (keys of 128, 112 and 80 beside values of 96, 48 and 24; layers that mix
    values with different head splits of the same row), under prompts, a second request and single tokens."""
    small = pt._config(101, 70, 1e-5, 1.3, (37, 5, 3), [
        pt.biased_layer("attention_3", 3, 3, 10, 6, 7, 33.5, pt.routed(30, 7, 3, None, 18)),
        pt.rotary_layer(6, 3, 14, 6, 6, pt.dense(50), base=77.0, bands=(3.0, 0.5, 2.5, 20)),
        pt.biased_layer("attention_2", 9, 3, 22, 6, 5, 11, pt.routed(10, 9, 4, (3, 2)), window=13),
        pt.rotary_layer(3, 1, 18, 30, 18, None, v_mix=False)])
    large = pt._config(300, 200, 1e-6, 2.5, (509, 97, 11), [
        pt.rotary_layer(8, 2, 80, 48, 40, pt.routed(48, 12, 4, (3, 2), 72), bands=(4.0, 1.0, 2.0, 256)),
        pt.biased_layer("attention_2", 8, 4, 64, 24, 24, 300, pt.dense(352), window=200),
        pt.biased_layer("attention_3", 4, 2, 128, 96, 20, 90, pt.dense(352), v_mix=False),
        pt.biased_layer("attention_3", 8, 2, 48, 48, 16, 150, pt.routed(64, 8, 2, (4, 3), 40)),
        pt.rotary_layer(6, 2, 112, 48, 112, pt.dense(100))])
    # rows wider than the tensor-core kernels take (144 and 160): bias, window and gate on the CUDA-core kernel in both dtypes
    wide = pt._config(90, 48, 1e-5, 1.0, (11, 2, 9), [
        pt.rotary_layer(2, 1, 160, 40, 64, pt.dense(64), scale=0.1),
        pt.biased_layer("attention_2", 4, 2, 136, 20, 8, 50, None, window=30, scale=0.1)])
    for (cfg, rows), length in ((small, 120), (large, 450), (wide, 100)):
        for dtype in ("float32", "bfloat16"):
            tm = pt.TinyPuvirax("-", dtype, cfg=cfg, rows=rows, seed=3)
            tokens = {"p": pt.random_tokens(cfg, length, 50), "q": pt.random_tokens(cfg, 77, 51)}
            p, q, cut = tokens["p"], tokens["q"], length - 40
            steps = [([("p", p[:cut], list(range(0, cut, 7)))], []),
                     ([("q", q[:70], [0, 69]), ("p", p[cut: cut + 1], [0])], [])]
            steps += [([("p", [p[i]], [0])] + ([("q", [q[70 + i - cut - 1]], [0])] if i - cut - 1 < 7 else []), [])
                      for i in range(cut + 1, length)]
            tm.check(tokens, harness.replay(tm.runner(64), steps), "odd sizes and a larger model")


def _random_config(seed: int):
    """Sizes, constants and layer order drawn at random: widths that are no multiple of 8, odd head counts, key and
    value sizes with and without a tensor-core kernel, windows from 1 up, bias tables of any height and reach, layers
    with and without feed-forward, routed ones with and without groups and shared expert."""
    gen = torch.Generator().manual_seed(2000 + seed)

    def pick(options):
        return options[int(torch.randint(0, len(options), (1,), generator=gen))]

    width = pick([36, 52, 64, 100, 136])
    mix_kv, mix_vdim = pick([1, 2, 3]), pick([8, 12, 16, 32, 40])
    layers = []
    for _ in range(pick([2, 3, 4, 5, 6])):
        kind = pick(["attention", "attention_2", "attention_3"])
        v_mix = pick([True, True, False])
        # (layers that mix values agree in kv_heads x vdim, not in how the heads split it)
        kv, vdim = pick([(mix_kv, mix_vdim), (1, mix_kv * mix_vdim)]) if v_mix else (pick([1, 2, 3]), pick([4, 8, 24, 64]))
        heads = kv * pick([1, 2, 3, 4])
        dim = pick([8, 12, 16, 24, 32, 64])
        choice = pick(["none", "dense", "dense", "moe", "moe"])
        if choice == "none":
            mlp = None
        elif choice == "dense":
            mlp = pt.dense(pick([40, 72, 130]))
        else:
            count = pick([1, 2, 4])
            per = pick([1, 2, 3])
            keep = pick(list(range(1, count + 1)))
            mlp = pt.routed(pick([8, 24, 40]), count * per, pick(list(range(1, keep * per + 1))),
                            (count, keep) if pick([True, True, False]) or keep < count else None, pick([None, 16, 48]))
            if "groups" not in mlp["router"]:
                assert keep == count
        scale = pick([0.1, 0.3, dim ** -0.5, 2.0 * dim ** -0.5])
        if kind == "attention":
            layers.append(pt.rotary_layer(heads, kv, dim, vdim, pick([None, 0, 2, dim // 2, dim]), mlp, v_mix=v_mix, scale=scale,
                                          base=pick([50.0, 10000.0, 1000000.0]),
                                          bands=pick([None, (4.0, 0.5, 3.0, 32), (8.0, 0.5, 2.0, 64)])))
        else:
            window = pick([1, 2, 5, 16, 17, 31, 33, 50]) if kind == "attention_2" else None
            rows = pick([2, 4, 6, 12, 16, 32])
            layers.append(pt.biased_layer(kind, heads, kv, dim, vdim, rows, rows // 2 * pick([1.5, 4, 20.5]) + 1, mlp,
                                          window=window, v_mix=v_mix, scale=scale))
    return pt._config(pick([64, 101, 257]), width, pick([1e-6, 1e-5, 1e-3]), pick([1.0, 0.5, 3.0]),
                      (pick([1, 17, 2039]), pick([1, 211, 100003]), pick([1, 13, 65537])), layers)


@pytest.mark.parametrize("seed", list(range(12)))
def test_configurations_drawn_at_random(seed):
    """Each drawn model under a mixed schedule (portions, single tokens, a request that ends and
    one that takes its slot), float32 and bfloat16 against the plain implementation."""
    cfg, rows = _random_config(seed)
    page = [16, 32, 64][seed % 3]
    for dtype in ("float32", "bfloat16"):
        tm = pt.TinyPuvirax("-", dtype, seed=seed, cfg=cfg, rows=rows)
        tokens = {r: pt.random_tokens(cfg, n, 100 + seed + i) for i, (r, n) in enumerate({"a": 70, "b": 23, "c": 41}.items())}
        a, b, c = tokens["a"], tokens["b"], tokens["c"]
        steps = [([("a", a[:35], list(range(35))), ("b", b[:2], [0, 1])], []),
                 ([("a", a[35:36], [0]), ("b", b[2:23], list(range(21)))], ["b"]),
                 ([("a", a[36:37], [0]), ("c", c[:3], [0, 1, 2])], []),
                 ([("c", c[3:40], list(range(37))), ("a", a[37:38], [0])], [])]
        steps += [([("a", [a[i]], [0])] + ([("c", [c[40]], [0])] if i == 38 else []), ["c"] if i == 38 else [])
                  for i in range(38, 70)]
        runner = tm.runner(-(-70 // page) + -(-41 // page) + 2, slots=2, page=page)
        tm.check(tokens, harness.replay(runner, steps), f"random configuration {seed}")


def test_missing_and_misshapen_tensors_are_named():
    from pulsarlm_b200.engine.loading import load_model
    from pulsarlm_b200.weights.loader import WeightsError

    (cfg, rows), _ = pt.CONFIGS["A"]
    weights = pt.random_weights(cfg, rows, 1)
    del weights["l2.mix.k.norm"]
    weights["l0.mix.rel"] = weights["l0.mix.rel"][:, :-1].contiguous()
    tm = pt.TinyPuvirax("A", "float32", weights=weights)
    with pytest.raises((WeightsError, ValueError)) as error:
        load_model(tm.folder, "float32", DEV)
    assert "l2.mix.k.norm" in str(error.value) or "l0.mix.rel" in str(error.value)


# --------------------------------------------------------------------------- the engine

def _plain_greedy(tm, prompt, n_new):
    tokens = list(prompt)
    for _ in range(n_new):
        tokens.append(int(tm.plain_logits(tokens)[-1].argmax()))
    return tokens[len(prompt):]


@pytest.mark.parametrize("cuda_graphs", [False, True])
def test_greedy_generation_through_the_engine(cuda_graphs):
    """Requests of unequal lengths through Engine.submit / step: admission, prompt portions of
    16 tokens beside decoding requests, more requests than slots (so slots and pages are used
    again), eager and captured decode steps; float32 tokens equal the plain implementation's."""
    from pulsarlm_b200.engine.engine import Engine

    tm = _model("A", "float32")
    engine = Engine(tm.folder, dtype="float32", device=DEV, page_size=16, n_pages=40, max_requests=3,
                    prefill_tokens_per_step=16, cuda_graphs=cuda_graphs)
    prompts = [pt.random_tokens(tm.cfg, n, 60 + i) for i, n in enumerate([40, 3, 21, 9, 30])]
    requests = [engine.submit(p, max_tokens=30, ignore_eos=True) for p in prompts]
    for _ in range(600):
        if not engine.has_work():
            break
        engine.step()
    assert not engine.has_work()
    for prompt, request in zip(prompts, requests):
        assert list(request.output) == _plain_greedy(tm, prompt, 30)
    if cuda_graphs:
        assert engine.runner.graph_steps > 0


def test_engine_preempts_and_recomputes_with_the_token_before():
    """So few pages that running requests are preempted (pages and state slot given back, the request
    recomputed from its start later): the tokens are still the plain implementation's, so no token of an
    earlier life of the slot leaks into the pair table's row."""
    from pulsarlm_b200.engine.engine import Engine

    (cfg, rows), _ = pt.CONFIGS["B"]
    tm = pt.TinyPuvirax("-", "float32", seed=4, cfg=cfg, rows=rows)
    engine = Engine(tm.folder, dtype="float32", device=DEV, page_size=16, n_pages=7, max_requests=4,
                    prefill_tokens_per_step=16)
    prompts = [pt.random_tokens(cfg, n, 95 + i) for i, n in enumerate([30, 25, 20])]
    requests = [engine.submit(p, max_tokens=20, ignore_eos=True) for p in prompts]
    for _ in range(600):
        if not engine.has_work():
            break
        engine.step()
    assert not engine.has_work() and engine.scheduler.preemptions > 0
    for prompt, request in zip(prompts, requests):
        assert request.finish_reason == "length"
        assert list(request.output) == _plain_greedy(tm, prompt, 20)


def test_engine_in_bfloat16_stays_close():
    from pulsarlm_b200.engine.engine import Engine

    tm = _model("C", "bfloat16")
    engine = Engine(tm.folder, dtype="bfloat16", device=DEV, page_size=16, n_pages=40, max_requests=4,
                    prefill_tokens_per_step=32, record_logits=True)
    prompts = [pt.random_tokens(tm.cfg, n, 70 + i) for i, n in enumerate([50, 7, 33])]
    requests = [engine.submit(p, max_tokens=20, ignore_eos=True) for p in prompts]
    while engine.has_work():
        engine.step()
    for prompt, request in zip(prompts, requests):
        full = list(prompt) + list(request.output)
        ref = tm.plain_logits(full[:-1])
        for i, row in enumerate(request.logits):
            assert pt.relative_error(row, ref[len(prompt) - 1 + i]) < 0.25


def _write(path, text) -> str:
    with open(path, "w") as f:
        json.dump(text, f)
    return str(path)


def test_command_line_random_model_generate_and_replay(tmp_path, capsys):
    """`models list`, `models random`, `generate` and the trace replay of the command line for
    this architecture: greedy tokens equal the plain implementation's on the written weights,
    and the replayed logits too. (Random weights need the bias tables' heights named in the
    configuration: the optional key `bias_rows`.)"""
    import io

    import numpy as np
    from safetensors.torch import load_file

    from pulsarlm_b200 import cli
    from pulsarlm_b200.engine import trace

    assert cli.main(["models", "list"]) == 0
    assert "Puvirax" in capsys.readouterr().out.split()
    (cfg, rows), _ = pt.CONFIGS["C"]
    cfg = json.loads(json.dumps(cfg))
    for layer, n in zip(cfg["layers"], rows):
        if n is not None:
            layer["mixer"]["bias_rows"] = n
    folder = str(tmp_path / "model")
    assert cli.main(["models", "random", folder, "--config", _write(tmp_path / "c.json", cfg), "--seed", "3",
                     "--dtype", "float32", "--std", "0.3"]) == 0
    capsys.readouterr()
    weights = {k: v.double() for k, v in load_file(folder + "/model.safetensors").items()}
    assert set(weights) | {"l0.mix.vmix"} == set(pt.tensor_shapes(cfg, rows))
    weights.setdefault("l0.mix.vmix", torch.tensor(0.0, dtype=torch.float64))
    prompt = pt.random_tokens(cfg, 19, 90)
    assert cli.main(["generate", folder, "--dtype", "float32", "--prompt_ids", ",".join(map(str, prompt)),
                     "--max_tokens", "8", "--ignore_eos"]) == 0
    record = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    tokens = list(prompt)
    for _ in range(8):
        tokens.append(int(plain.forward(cfg, weights, tokens)[-1].argmax()))
    assert record["output_ids"] == tokens[len(prompt):]
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": tokens[:11], "want": [3, 10]}], "end": []},
             {"step": 1, "entries": [{"id": "b", "tokens": tokens[:2], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": tokens[11:12], "want": [0]},
                                     {"id": "b", "tokens": tokens[2:9], "want": [6]}], "end": ["a", "b"]}]
    out = io.StringIO()
    assert trace.run(["--model", folder, "--dtype", "float32", "--out", str(tmp_path / "out"), "--max-tokens", "128"],
                     stdin=io.StringIO("\n".join(json.dumps(s) for s in steps) + "\n"), stdout=out) == 0
    assert out.getvalue().split() == ["done", "0", "done", "1", "done", "2"]
    ref = plain.forward(cfg, weights, tokens[:12])
    got0 = torch.from_numpy(np.fromfile(str(tmp_path / "out" / "0.f32"), dtype="<f4").reshape(2, -1))
    got2 = torch.from_numpy(np.fromfile(str(tmp_path / "out" / "2.f32"), dtype="<f4").reshape(2, -1))
    assert pt.relative_error(got0, ref[[3, 10]]) < 2e-4 and pt.relative_error(got2, ref[[11, 8]]) < 2e-4
    assert not (tmp_path / "out" / "1.f32").exists()
