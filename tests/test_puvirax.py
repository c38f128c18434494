"""The Puvirax decoder without a GPU: its configuration reader, its description as data, the bias
table's expansion, and the plain implementation's own consistency."""

from __future__ import annotations

import json

import pytest
import torch

import plain_puvirax as plain
import puvirax_tiny as pt

from pulsarlm_b200.config.base import ConfigError
from pulsarlm_b200.config.puvirax import PuviraxConfig
from pulsarlm_b200.config.registry import read_model_config, registered_architectures
from pulsarlm_b200.models.model import tensor_needs_of
from pulsarlm_b200.parts.normed_attention import bias_by_distance, distance_bucket
from pulsarlm_b200.weights.loader import shape_fits


@pytest.mark.parametrize("key", ["A", "B", "C"])
def test_configuration_is_read_by_its_keys_and_written_back(key):
    (text, _), _ = pt.CONFIGS[key]
    assert "Puvirax" in registered_architectures()
    arch, cfg = read_model_config(text)
    assert arch.name == "Puvirax" and isinstance(cfg, PuviraxConfig)
    assert PuviraxConfig.from_text(json.loads(json.dumps(cfg.to_text()))) == cfg
    for layer, entry in zip(cfg.layers, text["layers"]):
        m = entry["mixer"]
        assert (layer.heads, layer.kv_heads, layer.dim, layer.value_dim) == (m["heads"], m["kv_heads"], m["dim"], m["vdim"])
        assert layer.window == (m.get("mask") or {}).get("size") and layer.scale == m["scale"]
        assert (layer.mlp is None) == (entry["mlp"] is None)
    assert cfg.logit_scale == text["logit_scale"] and cfg.pairs.buckets == text["embedding"]["bigram"]["buckets"]


@pytest.mark.parametrize("key", ["A", "B", "C"])
def test_described_model_needs_exactly_the_stored_tensors(key):
    (text, rows), _ = pt.CONFIGS[key]
    arch, cfg = read_model_config(text)
    needs = tensor_needs_of(arch.describe(cfg))
    shapes = pt.tensor_shapes(text, rows)
    assert {n for n, need in needs.items() if not need.optional} <= set(shapes) and set(shapes) <= set(needs)
    for name, shape in shapes.items():
        assert shape_fits(shape, needs[name].shape), name


def test_bad_configurations_are_refused():
    (text, _), _ = pt.CONFIGS["A"]
    for change in (lambda t: t["layers"][0].update(type="attention_9"),
                   lambda t: t["layers"][1]["mixer"].update(kv_heads=3),
                   lambda t: t["layers"][1]["mixer"]["rot"].update(dims=7),
                   lambda t: t["layers"][0]["mixer"].pop("bias_max"),
                   lambda t: t["layers"][2]["mixer"].update(vdim=8),           # (layers that mix values must agree in kv_heads x vdim)
                   lambda t: t["layers"][0]["mlp"]["router"].update(top=5),
                   lambda t: t["layers"][0]["mlp"]["router"]["groups"].update(count=3),
                   lambda t: t.pop("vocab")):
        bad = json.loads(json.dumps(text))
        change(bad)
        with pytest.raises(ConfigError):
            PuviraxConfig.from_text(bad)


@pytest.mark.parametrize("rows,far", [(16, 128.0), (12, 40.0), (4, 5.0), (2, 3.0), (32, 64.0), (10, 1000.5)])
def test_bias_table_by_distance(rows, far):
    """One row per distance up to the first that reads the table's last row; below half the table's height a
    distance is its own row; the rows never go back; every later distance reads the last row."""
    table = torch.arange(rows * 3, dtype=torch.float32).view(rows, 3)
    by_distance = bias_by_distance(table, far)
    assert by_distance.shape[0] == 3
    picks = [int(value) // 3 for value in by_distance[0]]
    assert picks[: rows // 2] == list(range(rows // 2)) and picks[-1] == rows - 1 and picks == sorted(picks)
    assert picks == [plain.distance_bucket(d, rows, far) for d in range(len(picks))]
    for d in (len(picks), int(far), int(far) + 1, 10 * int(far)):
        assert distance_bucket(d, rows, far) == rows - 1 == plain.distance_bucket(d, rows, far)


def test_plain_implementation_is_causal_and_its_pieces_fit():
    (cfg, rows), _ = pt.CONFIGS["A"]
    weights = {k: v.double() for k, v in pt.random_weights(cfg, rows, 2).items()}
    tokens = pt.random_tokens(cfg, 50, 1)
    whole = plain.forward(cfg, weights, tokens)
    assert plain.relative_error_of(plain.forward(cfg, weights, tokens[:31]), whole[:31]) < 1e-12
    # a window of the sequence's length is no window; a window of 1 sees the token itself only
    q, k, v = torch.randn(9, 4, 8).double(), torch.randn(9, 2, 8).double(), torch.randn(9, 2, 6).double()
    assert torch.equal(plain.softmax_attention(q, k, v, 0.3, 9, None), plain.softmax_attention(q, k, v, 0.3, None, None))
    alone = plain.softmax_attention(q, k, v, 0.3, 1, None)
    assert plain.relative_error_of(alone[:, 3], v[:, 1]) < 1e-12
    # the pair table: a portion that starts inside a sequence reads the token before it
    table, pairs = weights["embed"], weights["bigram"]
    both = plain.pair_embedding(tokens, table, pairs, cfg)
    assert torch.equal(plain.pair_embedding(tokens[20:], table, pairs, cfg, before=tokens[19]), both[20:])
    assert not torch.equal(plain.pair_embedding(tokens[20:], table, pairs, cfg), both[20:])
    # shut-out groups count as minus infinity: with every correction far below zero the choice still comes from kept groups
    r = {"experts": 8, "top": 2, "groups": {"count": 4, "keep": 1}}
    h, router = torch.randn(5, 16).double(), torch.randn(8, 16).double()
    ids, w = plain.route(h, router, torch.full((8,), -5.0).double(), r)
    assert all(int(a) // 2 == int(b) // 2 for a, b in ids.tolist()) and bool((w > 0).all())


def test_stored_but_unused_tensors_are_allowed_and_others_are_not():
    """A layer without feed-forward may store its second norm, and a layer that mixes nothing a mixing factor: they
    load (nothing reads them). A tensor the design has no place for is still an error."""
    from pulsarlm_b200.weights.loader import WeightsError, check_names

    (text, rows), _ = pt.CONFIGS["B"]   # (its last layer has no feed-forward and mixes nothing)
    arch, cfg = read_model_config(text)
    needs = tensor_needs_of(arch.describe(cfg))
    shapes = pt.tensor_shapes(text, rows)
    shapes.update({"l3.norm2": (text["width"],), "l3.mix.vmix": (), "l0.mix.vmix": ()})
    check_names("a folder", needs, shapes)
    shapes["l3.mix.g"] = (5, text["width"])
    with pytest.raises(WeightsError):
        check_names("a folder", needs, shapes)
