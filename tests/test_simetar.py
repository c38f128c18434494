"""The Simetar decoder's configuration, description and plain implementation, on the CPU."""

from __future__ import annotations

import json
import math

import pytest
import torch

import plain_simetar as plain
import simetar_tiny as st
from pulsarlm_b200.config.base import ConfigError
from pulsarlm_b200.config.registry import read_model_config, registered_architectures
from pulsarlm_b200.models.model import tensor_needs_of
from pulsarlm_b200.parts.basic import ramped_frequencies, rope_inverse_frequencies


def test_the_architecture_is_registered():
    assert "Simetar" in registered_architectures()


@pytest.mark.parametrize("key", ["A", "B", "C"])
def test_configuration_round_trip_and_tensor_names(key):
    cfg_text, _ = st.CONFIGS[key]
    arch, cfg = read_model_config(cfg_text)
    assert arch.name == "Simetar"
    assert arch.read_config(cfg.to_text()) == cfg
    assert arch.read_config(json.loads(json.dumps(cfg.to_text()))) == cfg
    needs = tensor_needs_of(arch.describe(cfg))
    shapes = st.tensor_shapes(cfg_text)
    assert set(needs) == set(shapes)
    for name, need in needs.items():
        assert tuple(need.shape) == shapes[name], name


def test_a_reader_of_another_layers_rows_has_no_down_projection():
    arch, cfg = read_model_config(st.CONFIG_B)
    spec = arch.describe(cfg)
    assert spec.layers[1].mixer.params["cache_from"] == 0 and spec.layers[0].mixer.params["cache_from"] is None
    needs = tensor_needs_of(spec)
    assert "l0.mix.dkv" in needs and "l1.mix.dkv" not in needs and "l1.mix.dkv.norm" not in needs
    assert spec.layers[0].feed_forward is None and "l0.norm2" not in needs


def test_bad_configurations_are_refused():
    def broken(change, base=st.CONFIG_A):
        text = json.loads(json.dumps(base))
        change(text)
        with pytest.raises(ConfigError):
            read_model_config(text)

    broken(lambda t: t["layers"][0].update(type="other"))
    broken(lambda t: t["layers"][0]["mixer"].update(kv_heads=3))
    broken(lambda t: t["layers"][0]["mixer"]["rot"].update(dims=7))
    broken(lambda t: t["layers"][0]["mixer"]["rot"].update(dims=18))       # more than a head has
    broken(lambda t: t["layers"][0]["mixer"].update(vdim=8))               # the values are the keys
    broken(lambda t: t["layers"][0]["mlp"].update(kind="other"))
    broken(lambda t: t["layers"][3]["mixer"].update(kv_from=0))            # layer 0 caches no latent
    broken(lambda t: t["layers"][3]["mixer"].update(kv_from=3))            # not an earlier layer
    broken(lambda t: t["layers"][3]["mixer"].update(kv_rank=32))           # differs from its owner's
    broken(lambda t: t.pop("norm"))


def test_frequency_tables_of_the_engine_and_the_plain_implementation_agree():
    for rot in ({"base": 50000.0, "dims": 32, "scaling": {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 256}},
                {"base": 100.0, "dims": 8}, {"base": 10000.0, "dims": 16,
                                              "scaling": {"factor": 8.0, "low": 2.0, "high": 2.0, "original": 64}}):
        s = rot.get("scaling")
        bands = None if s is None else {"factor": s["factor"], "low_freq_factor": s["low"],
                                        "high_freq_factor": s["high"], "original_max_position_embeddings": s["original"]}
        got = rope_inverse_frequencies(rot["base"], rot["dims"], rot["dims"], bands)
        assert torch.allclose(torch.tensor(got, dtype=torch.float64), plain.banded_frequencies(rot), rtol=1e-12)
    for rot in ({"base": 10000.0, "dims": 32, "scaling": {"factor": 8.0, "original": 512, "fast": 32.0, "slow": 1.0}},
                {"base": 100.0, "dims": 4, "scaling": {"factor": 2.0, "original": 16, "fast": 4.0, "slow": 4.0}},
                {"base": 500.0, "dims": 64, "scaling": {"factor": 40.0, "original": 4096, "fast": 64.0, "slow": 0.5}}):
        got, amplitude = ramped_frequencies(rot["base"], rot["dims"], rot["scaling"])
        want, want_amplitude = plain.ramped_frequencies(rot)
        assert torch.allclose(torch.tensor(got, dtype=torch.float64), want, rtol=1e-12)
        assert amplitude == pytest.approx(want_amplitude) == pytest.approx(0.1 * math.log(rot["scaling"]["factor"]) + 1)


def test_banded_frequencies_keep_short_waves_and_divide_long_ones():
    rot = {"base": 10000.0, "dims": 64, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 128}}
    plain_f = 10000.0 ** (-2.0 * torch.arange(32, dtype=torch.float64) / 64)
    got = plain.banded_frequencies(rot)
    waves = 2 * math.pi / plain_f
    assert torch.equal(got[waves < 32], plain_f[waves < 32])
    assert torch.allclose(got[waves > 128], plain_f[waves > 128] / 8.0)
    between = (waves >= 32) & (waves <= 128)
    assert between.any() and ((got[between] <= plain_f[between]) & (got[between] >= plain_f[between] / 8.0)).all()


def test_plain_rotations_pair_neighbours_or_halves_and_keep_the_rest():
    x = torch.randn(5, 3, 12, dtype=torch.float64)
    freqs = torch.tensor([0.5, 0.1], dtype=torch.float64)
    y = plain.rotate_neighbours(x, torch.arange(5), freqs)
    assert torch.equal(y[..., 4:], x[..., 4:]) and torch.equal(y[0], x[0])
    a = 3 * 0.1
    assert torch.allclose(y[3, :, 2], x[3, :, 2] * math.cos(a) - x[3, :, 3] * math.sin(a))
    assert torch.allclose(y[3, :, 3], x[3, :, 3] * math.cos(a) + x[3, :, 2] * math.sin(a))
    z = plain.rotate_halves(x, torch.arange(5), freqs, 1.5)
    assert torch.equal(z[..., 4:], x[..., 4:])
    assert torch.allclose(z[0, :, :4], 1.5 * x[0, :, :4])
    assert torch.allclose(z[3, :, 1], 1.5 * (x[3, :, 1] * math.cos(a) - x[3, :, 3] * math.sin(a)))
    assert torch.allclose(z[3, :, 3], 1.5 * (x[3, :, 3] * math.cos(a) + x[3, :, 1] * math.sin(a)))


def test_plain_convolution_window_and_norms():
    u = torch.randn(6, 2, dtype=torch.float64)
    taps = torch.tensor([[1.0, 2.0, 3.0], [0.5, 0.0, -1.0]], dtype=torch.float64)
    y = plain.causal_conv(u, taps)
    assert torch.allclose(y[0], taps[:, 2] * u[0])
    assert torch.allclose(y[4], taps[:, 0] * u[2] + taps[:, 1] * u[3] + taps[:, 2] * u[4])
    see = plain.visible(6, 3)
    assert see[4].tolist() == [False, False, True, True, True, False]
    assert plain.visible(4, None)[3].all()
    x = torch.randn(3, 10, dtype=torch.float64)
    got = plain.layer_norm(x, torch.full((10,), 2.0, dtype=torch.float64), torch.ones(10, dtype=torch.float64), 0.0)
    assert torch.allclose(got.mean(-1), torch.ones(3, dtype=torch.float64))
    assert torch.allclose(got.var(-1, unbiased=False), torch.full((3,), 4.0, dtype=torch.float64))


def test_the_sink_takes_its_share_of_the_first_token():
    """One token, one head: the output is the value times e^s / (1 + e^s), and the gate's sigmoid."""
    mixer = {"heads": 1, "kv_heads": 1, "dim": 4, "vdim": 4, "conv": 1, "scale": 0.5,
             "rot": {"base": 100.0, "dims": 0}}
    gen = torch.Generator().manual_seed(0)
    w = {"q": torch.randn(4, 6, generator=gen), "k": torch.randn(4, 6, generator=gen), "q.b": torch.randn(4, generator=gen),
         "k.b": torch.randn(4, generator=gen), "q.conv": torch.ones(4, 1), "k.conv": torch.ones(4, 1),
         "q.norm": torch.ones(4), "k.norm": torch.ones(4), "g": torch.randn(4, 6, generator=gen), "o": torch.eye(4)}
    w = {k: v.double() for k, v in w.items()}
    h = torch.randn(1, 6, generator=gen).double()
    got = plain.conv_attention(mixer, w, "", h, 1e-6)
    q, k = h @ w["q"].T + w["q.b"], h @ w["k"].T + w["k.b"]
    s = float((plain.rms(q, 1e-6) * plain.rms(k, 1e-6)).sum() * 0.5)
    want = k * (math.exp(s) / (1.0 + math.exp(s))) * torch.sigmoid(h @ w["g"].T)
    assert torch.allclose(got, want)


def test_plain_prefix_does_not_depend_on_what_follows():
    cfg = st.CONFIG_A
    weights = st.random_weights(cfg, 3)
    tokens = st.random_tokens(cfg, 40, 1)
    whole = plain.forward(cfg, weights, tokens)
    part = plain.forward(cfg, weights, tokens[:25])
    assert plain.relative_error(whole[:25], part) < 1e-12
