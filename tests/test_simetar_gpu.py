"""The Simetar decoder in the engine against the plain implementation (plain_simetar.py):
each mechanism's kernel alone, then whole models under every kind of schedule."""

from __future__ import annotations

import json
import math

import pytest
import torch

import harness
import plain_simetar as plain
import simetar_tiny as st

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


# --------------------------------------------------------------------------- mechanisms alone

@pytest.mark.parametrize("width", [24, 50, 100, 520, 2600, 6000, 8200])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_layer_norm_of_a_sublayers_output_joins_the_stream(width, dtype):
    """x += layernorm(y) * w + b in fp32; the reader's copy is the stream rounded, or (the model's
    last norm) its layer norm; with a row list only those rows are made and x stays."""
    ops = _ops()
    gen = torch.Generator().manual_seed(width)
    tokens = 13
    x = torch.randn(tokens, width, generator=gen) * 3
    y = (torch.randn(tokens, width, generator=gen) * 5 + 2).to(dtype)
    w, b = torch.randn(width, generator=gen), torch.randn(width, generator=gen)
    w2, b2 = torch.randn(width, generator=gen), torch.randn(width, generator=gen)
    eps = 1e-5
    want_x = x.double() + plain.layer_norm(y.double(), w.double(), b.double(), eps)
    xd = x.to(DEV)
    out = torch.empty(tokens, width, dtype=dtype, device=DEV)
    ops.add_layernorm(xd, y.to(DEV), w.to(DEV), b.to(DEV), eps, out)
    assert plain.relative_error(xd.cpu(), want_x) < 1e-6
    assert plain.relative_error(out.cpu(), want_x) < _bar(dtype)
    # the last norm over chosen rows of the settled stream plus a pending sublayer output
    rows = [12, 0, 5]
    xd2 = x.to(DEV)
    normed = torch.empty(len(rows), width, dtype=dtype, device=DEV)
    ops.add_layernorm(xd2, y.to(DEV), w.to(DEV), b.to(DEV), eps, normed, w2.to(DEV), b2.to(DEV), 1e-3, _i32(rows))
    assert torch.equal(xd2.cpu(), x)
    want = plain.layer_norm(want_x[rows], w2.double(), b2.double(), 1e-3)
    assert plain.relative_error(normed.cpu(), want) < _bar(dtype)
    # nothing pending: only the reader's copy
    plain_copy = torch.empty(tokens, width, dtype=dtype, device=DEV)
    ops.add_layernorm(xd, None, None, None, 0.0, plain_copy)
    assert torch.equal(plain_copy.cpu(), xd.cpu().to(dtype))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_tanh_gelu_gate_and_sigmoid_gate(dtype):
    ops = _ops()
    gen = torch.Generator().manual_seed(2)
    gate_up = (torch.randn(7, 2 * 90, generator=gen) * 3).to(dtype)
    out = torch.empty(7, 90, dtype=dtype, device=DEV)
    ops.gated_act(gate_up.to(DEV), out, "gelu_tanh")
    want = plain.gelu_tanh(gate_up[:, :90].double()) * gate_up[:, 90:].double()
    assert plain.relative_error(out.cpu(), want) < _bar(dtype)
    wide = (torch.randn(7, 200, generator=gen) * 2).to(dtype).to(DEV)
    x = torch.randn(7, 60, generator=gen).to(dtype)
    xd = x.to(DEV)
    ops.sigmoid_gate(xd, wide[:, 140:])
    want = x.double() * torch.sigmoid(wide[:, 140:].cpu().double())
    assert plain.relative_error(xd.cpu(), want) < _bar(dtype)
    # columns that start off a four-element border, and a width that is no multiple of four
    for first, width in ((137, 60), (140, 57)):
        x = torch.randn(7, width, generator=gen).to(dtype)
        xd = x.to(DEV)
        ops.sigmoid_gate(xd, wide[:, first: first + width])
        want = x.double() * torch.sigmoid(wide[:, first: first + width].cpu().double())
        assert plain.relative_error(xd.cpu(), want) < _bar(dtype)


def _paged(lengths, page, gen):
    """A block table over pages handed out in a scrambled order."""
    n_pages = sum(-(-n // page) for n in lengths) + 2
    order = torch.randperm(n_pages, generator=gen).tolist()
    table = torch.full((len(lengths), max(-(-n // page) for n in lengths)), -1, dtype=torch.int32)
    for e, n in enumerate(lengths):
        for j in range(-(-n // page)):
            table[e, j] = order.pop()
    return n_pages, table


@pytest.mark.parametrize("taps,heads,kv,dim,rotary", [(3, 4, 2, 16, 16), (1, 3, 3, 8, 4), (4, 6, 2, 12, 0), (2, 2, 1, 32, 24),
                                                      (5, 2, 1, 16, 8), (4, 36, 4, 128, 64), (3, 5, 1, 10, 6)])
@pytest.mark.parametrize("pairs", [True, False])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_convolution_norm_and_rotation_on_the_way_to_the_cache(taps, heads, kv, dim, rotary, pairs, dtype):
    """Two requests; the first step brings portions of 5 and 1 tokens (so the second request's
    filter starts in the middle of a batch), the second a portion and a single token that reach
    back into the stored inputs, the third single tokens of both (the launch that also moves the
    stored inputs on). Queries, key pages and value pages against the plain functions."""
    ops = _ops()
    gen = torch.Generator().manual_seed(taps * 10 + dim)
    page, eps = 4, 1e-5
    lengths = [11, 7]
    channels = (heads + kv) * dim
    proj = [(torch.randn(n, channels + 8, generator=gen) * 2).to(dtype) for n in lengths]   # (8 more columns: a wider matrix)
    bias = torch.randn(channels, generator=gen)
    conv = torch.randn(channels, taps, generator=gen)
    q_norm, k_norm = torch.rand(heads * dim, generator=gen) + 0.5, torch.rand(kv * dim, generator=gen) + 0.5
    rot = {"base": 100.0, "dims": rotary, "scaling": {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 32}}
    freqs = plain.banded_frequencies(rot) if rotary else None
    n_pages, table = _paged(lengths, page, gen)
    k_pool = torch.zeros(n_pages, kv, page, dim, dtype=dtype, device=DEV)
    v_pool = torch.zeros_like(k_pool)
    states = torch.zeros(3, max(taps - 1, 1), channels, dtype=dtype, device=DEV)[:, : taps - 1]
    states = states.contiguous()
    slots = _i32([2, 0])
    want_q, want_k, want_v = [], [], []
    for e, n in enumerate(lengths):
        u = proj[e][:, :channels].double() + bias.double()
        y = plain.causal_conv(u, conv.double())
        yq, yk = y[:, : heads * dim], y[:, heads * dim:]
        positions = torch.arange(n)
        q = (plain.rms(yq, eps) * q_norm.double()).view(n, heads, dim)
        k = (plain.rms(yk, eps) * k_norm.double()).view(n, kv, dim)
        if rotary:
            def turn(x):
                if pairs:
                    return plain.rotate_neighbours(x, positions, freqs)
                return torch.cat([plain.rotate_halves(x[..., :rotary], positions, freqs, 1.0), x[..., rotary:]], dim=-1)
            q, k = turn(q), turn(k)
        want_q.append(q.reshape(n, heads * dim))
        want_k.append(k)
        want_v.append(yk.view(n, kv, dim))
    got_q = [torch.zeros(n, heads * dim) for n in lengths]
    fed = [0, 0]
    for portions in ([(0, 5), (1, 1)], [(1, 5), (0, 1)], [(0, 1), (1, 1)], [(0, 4)]):
        single = all(n == 1 for _, n in portions)
        rows = torch.cat([proj[e][fed[e]: fed[e] + n] for e, n in portions]).to(DEV)
        pos = _i32([fed[e] + i for e, n in portions for i in range(n)])
        entry = _i32([e for e, n in portions for _ in range(n)])
        q_out = torch.empty(rows.shape[0], heads * dim, dtype=dtype, device=DEV)
        ops.conv_norm_rope_write(rows[:, :channels], bias.to(DEV), conv.to(DEV), states, slots, single,
                                 q_norm.to(DEV), k_norm.to(DEV), eps, freqs.to(DEV) if rotary else None, rotary, pairs,
                                 1.0, pos, entry, table.to(DEV), q_out, k_pool, v_pool, page, heads, kv, dim)
        if taps > 1 and not single:
            ops.short_conv_state_strided(rows[:, :channels], entry, slots, states)
        at = 0
        for e, n in portions:
            got_q[e][fed[e]: fed[e] + n] = q_out[at: at + n].float().cpu()
            at += n
            fed[e] += n
    for e in range(2):
        n = fed[e]
        assert plain.relative_error(got_q[e][:n], want_q[e][:n]) < _bar(dtype), "queries"
        pages = table[e].tolist()
        got_k = torch.stack([k_pool[pages[j // page], :, j % page].float().cpu() for j in range(n)])
        got_v = torch.stack([v_pool[pages[j // page], :, j % page].float().cpu() for j in range(n)])
        assert plain.relative_error(got_k, want_k[e][:n]) < _bar(dtype), "cached keys"
        assert plain.relative_error(got_v, want_v[e][:n]) < _bar(dtype), "cached values"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_convolution_kernel_gives_the_same_bits_in_a_long_step_and_in_short_ones(dtype):
    """Queries, keys, values and the stored inputs come out the same bits whether 400 tokens
    arrive at once or in pieces, single tokens among them."""
    ops = _ops()
    gen = torch.Generator().manual_seed(3)
    taps, heads, kv, dim, page, n = 4, 6, 2, 32, 16, 400
    channels = (heads + kv) * dim
    proj = (torch.randn(n, channels, generator=gen) * 2).to(dtype).to(DEV)
    bias, conv = torch.randn(channels, generator=gen).to(DEV), torch.randn(channels, taps, generator=gen).to(DEV)
    q_norm, k_norm = (torch.rand(heads * dim, generator=gen) + 0.5).to(DEV), (torch.rand(kv * dim, generator=gen) + 0.5).to(DEV)
    freqs = plain.banded_frequencies({"base": 100.0, "dims": dim, "scaling": None}).to(DEV)
    n_pages, table = _paged([n], page, gen)
    results = []
    for cuts in ([n], [100, 1, 1, 198, 100]):
        k_pool = torch.zeros(n_pages, kv, page, dim, dtype=dtype, device=DEV)
        v_pool = torch.zeros_like(k_pool)
        states = torch.zeros(2, taps - 1, channels, dtype=dtype, device=DEV)
        q_out = torch.empty(n, heads * dim, dtype=dtype, device=DEV)
        at = 0
        for m in cuts:
            rows = proj[at: at + m]
            entry = _i32([0] * m)
            ops.conv_norm_rope_write(rows, bias, conv, states, _i32([1]), m == 1, q_norm, k_norm, 1e-6, freqs, dim, True, 1.0,
                                     _i32(list(range(at, at + m))), entry, table.to(DEV), q_out[at: at + m], k_pool, v_pool,
                                     page, heads, kv, dim)
            if m > 1:
                ops.short_conv_state_strided(rows, entry, _i32([1]), states)
            at += m
        results.append((q_out, k_pool, v_pool, states))
    for a, b in zip(*results):
        assert torch.equal(a, b)


@pytest.mark.parametrize("heads,dim,rot,rank", [(3, 16, 8, 40), (2, 8, 4, 24), (4, 32, 16, 48), (1, 16, 32, 20)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_latent_rows_and_the_rotated_query_part(heads, dim, rot, rank, dtype):
    """The cached row [normed latent | rotated shared key part] and the queries' rotated columns
    (halves paired, cos and sin times the ramp's amplitude), at positions over several pages;
    a reader of another layer's rows (no z) writes nothing."""
    ops = _ops()
    gen = torch.Generator().manual_seed(rank)
    page, eps = 4, 1e-5
    lengths = [9, 6]
    mixer = {"kv_rank": rank, "rot_dim": rot,
             "rot": {"base": 100.0, "dims": rot, "scaling": {"factor": 4.0, "original": 16, "fast": 8.0, "slow": 1.0}}}
    freqs, amplitude = plain.ramped_frequencies(mixer["rot"])
    assert amplitude > 1.0
    norm = torch.rand(rank, generator=gen) + 0.5
    n_pages, table = _paged(lengths, page, gen)
    pool = torch.zeros(n_pages, 1, page, rank + rot, dtype=dtype, device=DEV)
    tokens = sum(lengths)
    q = (torch.randn(tokens, heads, dim + rot, generator=gen) * 2).to(dtype)
    z = (torch.randn(tokens, rank + rot + 6, generator=gen) * 2).to(dtype)
    pos = [p for n in lengths for p in range(n)]
    entry = [e for e, n in enumerate(lengths) for _ in range(n)]
    q_out = torch.zeros(tokens, heads, rank + rot, dtype=dtype, device=DEV)
    ops.latent_rope_write(q.to(DEV), q_out, z.to(DEV)[:, : rank + rot], norm.to(DEV), eps, rank, rot, freqs.to(DEV), False,
                          amplitude, _i32(pos), _i32(entry), table.to(DEV), pool, page)
    positions = torch.tensor(pos)
    want_q = plain.rotate_halves(q[..., dim:].double(), positions, freqs, amplitude)
    assert plain.relative_error(q_out[..., rank:].cpu(), want_q) < _bar(dtype)
    assert float(q_out[..., :rank].abs().max()) == 0.0        # (the latent part of the query row is another product's)
    latent = plain.rms(z[:, :rank].double(), eps) * norm.double()
    shared = plain.rotate_halves(z[:, None, rank: rank + rot].double(), positions, freqs, amplitude)[:, 0]
    for t in range(tokens):
        row = pool[table[entry[t], pos[t] // page], 0, pos[t] % page].float().cpu()
        assert plain.relative_error(row[:rank], latent[t]) < _bar(dtype)
        assert plain.relative_error(row[rank:], shared[t]) < _bar(dtype)
    before = pool.clone()
    ops.latent_rope_write(q.to(DEV), q_out, None, None, eps, rank, rot, freqs.to(DEV), False, amplitude, _i32(pos),
                          _i32(entry), table.to(DEV), pool, page)
    assert torch.equal(before, pool)


@pytest.mark.parametrize("window", [None, 7, 16, 21])
@pytest.mark.parametrize("spike", [None, "inside", "outside", "far"])
@pytest.mark.parametrize("cap", [None, 4.0])
def test_capped_attention_with_a_sink_at_window_edges(window, spike, cap):
    """Grouped heads over paged keys with values apart from the keys, single tokens and prompt rows
    at page borders; one key just inside the window, just outside it, or far back is lined up
    with the query so that it dominates where it is in reach; a cap flattens it again. Rows'
    weights add up to less than 1 (the sink), most visibly at a request's first tokens."""
    ops = _ops()
    if spike in ("inside", "outside") and window is None:
        pytest.skip("no window, no edge")
    heads, kv, dim, page, scale = 6, 2, 16, 8, 0.3
    lengths = [70, 33, 8, 129]
    distance = {None: None, "inside": (window or 0) - 1, "outside": window, "far": 60}[spike]
    for dtype in (torch.float32, torch.bfloat16):
        gen = torch.Generator().manual_seed(11)
        n_pages, table = _paged(lengths, page, gen)
        keys = [torch.randn(n, kv, dim, generator=gen).to(dtype) for n in lengths]
        values = [torch.randn(n, kv, dim, generator=gen).to(dtype) for n in lengths]
        queries = [(e, p) for e, n in enumerate(lengths) for p in sorted({0, 1, 2, n // 2, n - 2, n - 1}) if p >= 0]
        q = torch.randn(len(queries), heads, dim, generator=gen).to(dtype)
        if distance is not None:
            for i, (e, p) in enumerate(queries):
                if p - distance >= 0:
                    direction = q[i, 0].float() / q[i, 0].float().norm()
                    keys[e][p - distance, 0] = (40.0 * direction).to(dtype)
        k_pool = torch.zeros(n_pages, kv, page, dim, dtype=dtype, device=DEV)
        v_pool = torch.zeros_like(k_pool)
        for e, n in enumerate(lengths):
            for j in range(n):
                k_pool[table[e, j // page], :, j % page] = keys[e][j].to(DEV)
                v_pool[table[e, j // page], :, j % page] = values[e][j].to(DEV)
        want = torch.zeros(len(queries), heads, dim, dtype=torch.float64)
        for i, (e, p) in enumerate(queries):
            see = plain.visible(lengths[e], window)[p: p + 1]
            for h in range(heads):
                g = h // (heads // kv)
                want[i, h] = plain.capped_attention_with_sink(q[i, h].double()[None], keys[e][:, g].double(),
                                                              values[e][:, g].double(), see, scale, cap)[0]
        out = torch.empty(len(queries), heads, dim, dtype=dtype, device=DEV)
        ops.attention_simt(q.to(DEV), k_pool, v_pool, table.to(DEV), _i32([p for _, p in queries]),
                           _i32([e for e, _ in queries]), out, page, window, scale, softcap=cap or 0.0,
                           sinks=torch.zeros(heads, device=DEV))
        assert plain.relative_error(out.cpu(), want) < (1e-5 if dtype == torch.float32 else 1e-2), (dtype, window, spike)


@pytest.mark.parametrize("dim,heads,kv", [(32, 6, 2), (96, 4, 1), (64, 3, 3)])
@pytest.mark.parametrize("window,distance", [(None, None), (None, 150), (24, 23), (24, 24), (37, 36), (37, 37), (16, 15)])
@pytest.mark.parametrize("cap", [None, 3.0, 50.0])
def test_tensor_core_attention_takes_the_cap_and_the_sink(dim, heads, kv, window, distance, cap):
    """The bfloat16 kernels for single tokens (any number of key shares) and for prompt portions,
    with values apart from the keys, a score cap and a sink of logit 0; one key at a chosen
    distance (a window's last key, the first one outside, or far back) is lined up with the query."""
    ops = _ops()
    page, scale, dtype = 16, 0.25, torch.bfloat16
    lengths = [200, 33, 16, 129]
    if not (ops.attention_decode_supports(dim, heads // kv, page, dtype) and ops.attention_prefill_supports(dim, page, dtype)):
        pytest.skip("a shape for the CUDA-core kernel")
    sinks = torch.zeros(heads, device=DEV)

    def case(queries, seed):
        gen = torch.Generator().manual_seed(seed)
        n_pages, table = _paged(lengths, page, gen)
        keys = [torch.randn(n, kv, dim, generator=gen).to(dtype) for n in lengths]
        values = [torch.randn(n, kv, dim, generator=gen).to(dtype) for n in lengths]
        q = torch.randn(len(queries), heads, dim, generator=gen).to(dtype)
        if distance is not None:
            for i, (e, p) in enumerate(queries):
                if p - distance >= 0:
                    direction = q[i, 0].float() / q[i, 0].float().norm()
                    keys[e][p - distance, 0] = (60.0 * direction).to(dtype)
        k_pool = torch.zeros(n_pages, kv, page, dim, dtype=dtype, device=DEV)
        v_pool = torch.zeros_like(k_pool)
        for e, n in enumerate(lengths):
            for j in range(n):
                k_pool[table[e, j // page], :, j % page] = keys[e][j].to(DEV)
                v_pool[table[e, j // page], :, j % page] = values[e][j].to(DEV)
        want = torch.zeros(len(queries), heads, dim, dtype=torch.float64)
        for i, (e, p) in enumerate(queries):
            see = plain.visible(lengths[e], window)[p: p + 1]
            for h in range(heads):
                g = h // (heads // kv)
                want[i, h] = plain.capped_attention_with_sink(q[i, h].double()[None], keys[e][:, g].double(),
                                                              values[e][:, g].double(), see, scale, cap)[0]
        return q.to(DEV), k_pool, v_pool, table.to(DEV), want

    queries = [(e, n - 1) for e, n in enumerate(lengths)] + [(0, 0), (0, 1), (3, 64)]
    # (a request has one single token in a step; here each query row stands for a request of its own)
    q, k_pool, v_pool, table, want = case(queries, 21)
    pos, entry = _i32([p for _, p in queries]), _i32([e for e, _ in queries])
    for splits in (1, 2, 5):
        scratch = torch.empty(ops.attention_decode_scratch_floats(len(queries), heads, dim, splits),
                              dtype=torch.float32, device=DEV) if splits > 1 else None
        out = torch.empty_like(q)
        ops.attention_decode(q, k_pool, v_pool, table, pos, entry, out, page, window, scale, splits, scratch,
                             extras=ops.attention_extras(q, sinks, None, True, cap or 0.0))
        assert plain.relative_error(out.cpu(), want) < 1e-2, ("single tokens", splits)
    spans = [(0, 120, 200), (3, 0, 129), (1, 32, 33), (2, 0, 16)]
    queries = [(e, p) for e, lo, hi in spans for p in range(lo, hi)]
    q, k_pool, v_pool, table, want = case(queries, 22)
    rows = ops.attention_prefill_tile_rows()
    tiles, at = [], 0
    for e, lo, hi in spans:
        for r in range(0, hi - lo, rows):
            tiles.append((at + r, min(rows, hi - lo - r), lo + r, e))
        at += hi - lo
    out = torch.empty_like(q)
    ops.attention_prefill(q, k_pool, v_pool, table, _i32(tiles), out, page, window, scale,
                          extras=ops.attention_extras(q, sinks, None, True, cap or 0.0))
    assert plain.relative_error(out.cpu(), want) < 1e-2, "prompt rows"


# --------------------------------------------------------------------------- whole models

def _model(key, dtype, seed=1, sharp=1.0):
    return st.TinySimetar(key, dtype, seed, sharp=sharp)


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
    tokens = {"p": st.random_tokens(tm.cfg, 75, 3), "q": st.random_tokens(tm.cfg, 5, 4), "r": st.random_tokens(tm.cfg, 1, 5)}
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
        tokens = st.random_tokens(tm.cfg, 37, 9)
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
            assert plain.relative_error(got, want[i]) < 2e-5, (key, i)


@pytest.mark.parametrize("key", ["A", "B", "C"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prefill_then_token_by_token(key, dtype):
    """A prompt in one step, then 70 tokens one by one: past every window and over page borders."""
    tm = _model(key, dtype)
    runner = tm.runner(24)
    tokens = {"p": st.random_tokens(tm.cfg, 110, 5)}
    steps = [([("p", tokens["p"][:40], [0, 1, 39])], [])]
    steps += [([("p", [tokens["p"][i]], [0])], []) for i in range(40, 110)]
    tm.check(tokens, harness.replay(runner, steps), f"{key} decode")


@pytest.mark.parametrize("key", ["A", "B", "C"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_token_by_token_from_the_start(key, dtype):
    """The first tokens of a sequence, where the filters still read zeros and the sink holds
    most of a row's weight."""
    tm = _model(key, dtype)
    runner = tm.runner(8)
    tokens = {"p": st.random_tokens(tm.cfg, 30, 6)}
    steps = [([("p", [t], [0])], []) for t in tokens["p"]]
    tm.check(tokens, harness.replay(runner, steps), f"{key} from the start")


@pytest.mark.parametrize("key", ["A", "B", "C"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_portions_of_many_sizes(key, dtype):
    tm = _model(key, dtype)
    runner = tm.runner(24)
    tokens = {"p": st.random_tokens(tm.cfg, 150, 7)}
    cuts = [2, 2, 3, 1, 1, 7, 16, 2, 33, 1, 2, 17, 31, 2, 30]
    tm.check(tokens, harness.replay(runner, _portions(tokens["p"], cuts)), f"{key} portions")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_float32_bits_do_not_depend_on_the_cut(dtype):
    """In float32 every kernel adds in an order fixed by the token's own place: logits of a prompt
    fed whole and fed in portions are equal bit for bit. (bfloat16: within rounding.)"""
    tm = _model("A", dtype)
    tokens = st.random_tokens(tm.cfg, 90, 8)
    whole = harness.replay(tm.runner(12), [([("p", tokens, list(range(90)))], [])])["p"]
    cut = harness.replay(tm.runner(12), _portions(tokens, [5, 1, 2, 40, 1, 1, 3, 37]))["p"]
    for position in range(90):
        if dtype == "float32":
            assert torch.equal(whole[position], cut[position]), position
        else:
            assert st.relative_error(cut[position], whole[position]) < 4e-2


@pytest.mark.parametrize("key", ["A", "C"])
@pytest.mark.parametrize("sharp", [3.0, 6.0])
def test_sharp_attention_shows_every_key_in_reach(key, sharp):
    """float32, scores multiplied so that each softmax rests on a few keys: a window one token off,
    a far latent row lost with its page, or a sink left out would move these logits by orders
    more than the bar. Prompt portions whose cuts fall just before, at and just after every
    window's edge, then single tokens until every window has passed over decoded tokens, with
    pages of 16 and of 64."""
    tm = _model(key, "float32", seed=7, sharp=sharp)
    windows = sorted({(layer["mixer"].get("mask") or {}).get("size") for layer in tm.cfg["layers"]} - {None})
    n = 2 * max(windows) + 90
    tokens = {"p": st.random_tokens(tm.cfg, n, 12)}
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
    assert st.relative_error(off_by_one, plain_logits) > 50 * st.TOLERANCE["float32"]


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
    tokens = {r: st.random_tokens(tm.cfg, n, 10 + i) for i, (r, n) in enumerate(lengths.items())}
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
    tokens = {r: st.random_tokens(tm.cfg, n, 20 + i) for i, (r, n) in enumerate({"a": 50, "b": 9, "c": 33}.items())}
    alone = {}
    for r, t in tokens.items():
        alone.update(harness.replay(tm.runner(8), [([(r, t[:-3], [len(t) - 4])], [])] +
                                    [([(r, [t[i]], [0])], []) for i in range(len(t) - 3, len(t))]))
    runner = tm.runner(16)
    steps = [([(r, t[:-3], [len(t) - 4]) for r, t in tokens.items()], [])]
    steps += [([(r, [t[len(t) - 3 + i]], [0]) for r, t in tokens.items()], []) for i in range(3)]
    together = harness.replay(runner, steps)
    for r in tokens:
        for position, row in alone[r].items():
            if dtype == "float32":
                assert torch.equal(row, together[r][position])
            else:
                assert st.relative_error(together[r][position], row) < 4e-2


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(dtype):
    """400 tokens one by one: pages of the windowed layers are given back and used again while
    the latent rows of the first tokens stay in reach."""
    tm = _model("B", dtype)
    runner = tm.runner(16)
    tokens = {"p": st.random_tokens(tm.cfg, 400, 30)}
    steps = [([("p", tokens["p"][:4], [3])], [])]
    steps += [([("p", [tokens["p"][i]], [0] if i % 9 == 0 or i > 390 else [])], []) for i in range(4, 400)]
    tm.check(tokens, harness.replay(runner, steps), "B long decoding")


def test_a_far_token_is_still_seen_by_the_latent_layers():
    """Two prompts that differ in their first token only: 300 tokens on, far past every window,
    the logits still differ (latent attention has no window), and the engine reproduces the
    difference, in a prompt and in a decoded token."""
    tm = _model("A", "float32", sharp=3.0)
    base = st.random_tokens(tm.cfg, 301, 40)
    other = [(base[0] + 1) % tm.cfg["vocab"]] + base[1:]
    tokens = {"x": base, "y": other}
    got = harness.replay(tm.runner(48), [([("x", base[:300], [299]), ("y", other[:300], [299])], []),
                                         ([("x", base[300:], [0]), ("y", other[300:], [0])], ["x", "y"])])
    tm.check(tokens, got, "A far token")
    for position in (299, 300):
        want = tm.plain_logits(base)[position] - tm.plain_logits(other)[position]
        assert want.abs().max() > 1e-3
        assert st.relative_error(got["x"][position] - got["y"][position], want) < 0.05


def test_sizes_come_from_the_configuration():
    """Values that a given model may leave equal to one another or at 1: one head, one kv head
    for many query heads, a window of 1 (a token sees only itself and the sink), a single tap
    that is still a factor per channel, a rotary width below the head's, a value size unlike
    the key size, a rank below the head size, a reader right after its owner, no feed-forward
    anywhere, a scale of 1."""
    cfg = {
        "architecture": "Simetar", "vocab": 50, "width": 32, "norm": {"eps": 1e-3},
        "layers": [st.attention_layer(1, 1, 8, 1, 2, 1, None, softcap=None, scale=1.0),
                   st.latent_layer(1, 16, 2, 4, 8, None, scale=1.0),
                   st.latent_layer(3, 4, 2, 20, 8, st.dense(8), kv_from=1),
                   st.attention_layer(5, 1, 8, 2, 8, 2, None, softcap=1.0),
                   st.latent_layer(2, 8, 6, 8, 12, None, ramp=(2.0, 8, 2.0, 1.0))],
    }
    for dtype in ("float32", "bfloat16"):
        tm = st.TinySimetar("-", dtype, cfg=cfg)
        tokens = {"p": st.random_tokens(cfg, 40, 50)}
        steps = [([("p", tokens["p"][:20], list(range(20)))], [])]
        steps += [([("p", [t], [0])], []) for t in tokens["p"][20:]]
        tm.check(tokens, harness.replay(tm.runner(8), steps), "sizes of one")


def test_latent_rows_wider_than_512():
    """A latent of 560 with a rotated part of 32: cached rows of 592 attend on the CUDA-core kernel's
    build with more accumulators a lane."""
    cfg = {
        "architecture": "Simetar", "vocab": 60, "width": 48, "norm": {"eps": 1e-5},
        "layers": [st.latent_layer(2, 16, 32, 8, 560, st.dense(64), scale=0.2, ramp=(4.0, 32, 16.0, 1.0)),
                   st.attention_layer(2, 1, 16, 9, 8, 3, None, softcap=8.0),
                   st.latent_layer(3, 8, 32, 24, 560, None, scale=0.2, ramp=(4.0, 32, 16.0, 1.0), kv_from=0)],
    }
    for dtype in ("float32", "bfloat16"):
        tm = st.TinySimetar("-", dtype, cfg=cfg)
        tokens = {"p": st.random_tokens(cfg, 45, 51)}
        steps = [([("p", tokens["p"][:30], list(range(30)))], [])]
        steps += [([("p", [t], [0])], []) for t in tokens["p"][30:]]
        tm.check(tokens, harness.replay(tm.runner(8), steps), "rows of 592")


def _random_config(seed: int) -> dict:
    """Sizes, constants and layer order drawn at random: widths that are no multiple of 8, odd
    head counts, head sizes and ranks with and without a tensor-core kernel, windows from 1 up,
    layers with and without feed-forward, cap, window, convolution or frequency scaling; readers
    of an earlier latent layer's rows."""
    gen = torch.Generator().manual_seed(1000 + seed)

    def pick(options):
        return options[int(torch.randint(0, len(options), (1,), generator=gen))]

    width = pick([36, 52, 64, 100, 136])
    layers, owners = [], []
    for i in range(pick([2, 3, 4, 5, 6])):
        ff = pick([None, 40, 72, 130])
        mlp = st.dense(ff) if ff else None
        if pick([0, 1]) == 0:
            kv = pick([1, 2, 3])
            dim = pick([8, 12, 16, 24, 32, 64])
            layers.append(st.attention_layer(kv * pick([1, 2, 3, 4]), kv, dim, pick([None, 1, 2, 5, 16, 17, 31, 33, 50]),
                                             pick([0, 2, dim // 2, dim]), pick([1, 2, 3, 4, 5]), mlp,
                                             softcap=pick([None, 1.5, 10.0, 50.0]), scale=pick([0.1, 0.3, dim ** -0.5]),
                                             base=pick([50.0, 10000.0, 500000.0]),
                                             bands=pick([None, (4.0, 1.0, 4.0, 32), (8.0, 0.5, 2.0, 64)])))
        elif owners and pick([0, 1]) == 0:
            j = pick(owners)
            m = layers[j]["mixer"]
            ramp = m["rot"].get("scaling")
            layers.append(st.latent_layer(pick([1, 2, 3, 5]), pick([8, 12, 16, 32]), m["rot_dim"], pick([4, 8, 24, 40]),
                                          m["kv_rank"], mlp, scale=pick([0.1, 0.25]), base=m["rot"]["base"],
                                          ramp=tuple(ramp[k] for k in ("factor", "original", "fast", "slow")) if ramp else None,
                                          kv_from=j))
        else:
            owners.append(i)
            layers.append(st.latent_layer(pick([1, 2, 3, 4, 7]), pick([8, 12, 16, 20, 32]), pick([2, 4, 8, 16, 32]),
                                          pick([4, 8, 16, 24, 40]), pick([8, 24, 32, 40, 48, 64, 80, 96, 112, 136]), mlp,
                                          scale=pick([0.1, 0.25]), base=pick([100.0, 10000.0]),
                                          ramp=pick([None, (4.0, 32, 16.0, 1.0), (40.0, 64, 32.0, 2.0)])))
    return {"architecture": "Simetar", "vocab": pick([64, 101, 257]), "width": width,
            "norm": {"eps": pick([1e-6, 1e-5, 1e-3])}, "layers": layers}


@pytest.mark.parametrize("seed", list(range(12)))
def test_configurations_drawn_at_random(seed):
    """Each drawn model under a mixed schedule (portions, single tokens, a request that ends and
    one that takes its slot), float32 and bfloat16 against the plain implementation."""
    cfg = _random_config(seed)
    page = [16, 32, 64][seed % 3]
    for dtype in ("float32", "bfloat16"):
        tm = st.TinySimetar("-", dtype, seed=seed, cfg=cfg)
        tokens = {r: st.random_tokens(cfg, n, 100 + seed + i) for i, (r, n) in enumerate({"a": 70, "b": 23, "c": 41}.items())}
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

    cfg, _ = st.CONFIGS["A"]
    weights = st.random_weights(cfg, 1)
    del weights["l1.mix.dkv.norm"]
    weights["l0.mix.k.conv"] = weights["l0.mix.k.conv"][:, :-1].contiguous()
    tm = st.TinySimetar("A", "float32", weights=weights)
    with pytest.raises((WeightsError, ValueError)) as error:
        load_model(tm.folder, "float32", DEV)
    assert "l1.mix.dkv.norm" in str(error.value) or "l0.mix.k.conv" in str(error.value)


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
    prompts = [st.random_tokens(tm.cfg, n, 60 + i) for i, n in enumerate([40, 3, 21, 9, 30])]
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


def test_engine_preempts_and_recomputes_with_states():
    """So few pages that running requests are preempted (pages and state slot given back, the
    request recomputed from its start later): the tokens are still the plain implementation's,
    so no filter input or cached row of an earlier life leaks into the recomputation."""
    from pulsarlm_b200.engine.engine import Engine

    cfg = json.loads(json.dumps(st.CONFIGS["B"][0]))   # (its latent layers keep every page)
    tm = st.TinySimetar("-", "float32", seed=4, cfg=cfg)
    engine = Engine(tm.folder, dtype="float32", device=DEV, page_size=16, n_pages=7, max_requests=4,
                    prefill_tokens_per_step=16)
    prompts = [st.random_tokens(cfg, n, 95 + i) for i, n in enumerate([30, 25, 20])]
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
    prompts = [st.random_tokens(tm.cfg, n, 70 + i) for i, n in enumerate([50, 7, 33])]
    requests = [engine.submit(p, max_tokens=20, ignore_eos=True) for p in prompts]
    while engine.has_work():
        engine.step()
    for prompt, request in zip(prompts, requests):
        full = list(prompt) + list(request.output)
        ref = tm.plain_logits(full[:-1])
        for i, row in enumerate(request.logits):
            assert st.relative_error(row, ref[len(prompt) - 1 + i]) < 0.25


def _write(path, text) -> str:
    with open(path, "w") as f:
        json.dump(text, f)
    return str(path)


def test_command_line_random_model_generate_and_replay(tmp_path, capsys):
    """`models list`, `models random`, `generate` and the trace replay of the command line for
    this architecture: greedy tokens equal the plain implementation's on the written weights,
    and the replayed logits too."""
    import io

    import numpy as np
    from safetensors.torch import load_file

    from pulsarlm_b200 import cli
    from pulsarlm_b200.engine import trace

    assert cli.main(["models", "list"]) == 0
    assert "Simetar" in capsys.readouterr().out.split()
    cfg = json.loads(json.dumps(st.CONFIGS["C"][0]))
    folder = str(tmp_path / "model")
    assert cli.main(["models", "random", folder, "--config", _write(tmp_path / "c.json", cfg), "--seed", "3",
                     "--dtype", "float32", "--std", "0.3"]) == 0
    capsys.readouterr()
    weights = {k: v.double() for k, v in load_file(folder + "/model.safetensors").items()}
    assert set(weights) == set(st.tensor_shapes(cfg))
    prompt = st.random_tokens(cfg, 19, 90)
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
    assert st.relative_error(got0, ref[[3, 10]]) < 2e-4 and st.relative_error(got2, ref[[11, 8]]) < 2e-4
    assert not (tmp_path / "out" / "1.f32").exists()
