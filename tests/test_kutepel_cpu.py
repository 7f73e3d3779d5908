"""Kutepel without a GPU: the plain implementation against itself (whole sequences
against token-by-token forms over explicit key lists) and against values worked out by
hand; the configuration, its errors and the model-as-data it becomes."""
import copy
import json
import math

import numpy as np
import pytest
import torch

import kutepel_tiny as tiny
import plain_kutepel as plain

F = torch.float64


def double(weights):
    return {k: v.double() for k, v in weights.items()}


def spec_of(doc):
    from foundry_b200.config.registry import resolve_architecture
    arch = resolve_architecture(doc)
    return arch.build_spec(arch.parse_config(doc))


# ------------------------------------------------------------ the plain model itself
def test_frequency_bands_by_hand():
    """base 10, 8 rotated elements: f = 1, 10^-1/4, 10^-1/2, 10^-3/4; wavelengths 6.28,
    11.2, 19.9, 35.3. With original 40, high 4 (kept below 10), low 2 (slowed above 20):
    the first is kept, the last slowed, the two between blended by their own place."""
    rot = {"base": 10.0, "dims": 8, "scaling": {"factor": 5.0, "low": 2.0, "high": 4.0, "original": 40}}
    f = [10.0 ** (-i / 4) for i in range(4)]
    got = plain.frequencies(rot)
    assert got[0].item() == pytest.approx(f[0], rel=1e-14)
    assert got[3].item() == pytest.approx(f[3] / 5.0, rel=1e-14)
    for i in (1, 2):
        s = (40.0 / (2 * math.pi / f[i]) - 2.0) / (4.0 - 2.0)
        assert 0.0 < s < 1.0
        assert got[i].item() == pytest.approx((1 - s) * f[i] / 5.0 + s * f[i], rel=1e-13)
    # without scaling: the plain powers
    plain_f = plain.frequencies({"base": 10.0, "dims": 8})
    assert torch.allclose(plain_f, torch.tensor(f, dtype=F), rtol=1e-14, atol=0)


def test_the_library_frequencies_equal_the_plain_ones():
    from foundry_b200.parts.rope import banded_frequencies
    for rot in ({"base": 10000.0, "dims": 64, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 512}},
                {"base": 500000.0, "dims": 24, "scaling": {"factor": 16.0, "low": 2.0, "high": 8.0, "original": 256}},
                {"base": 100.0, "dims": 12}, {"base": 7.0, "dims": 2}):
        s = rot.get("scaling") or {}
        got = banded_frequencies(rot["dims"], rot["base"], **s)
        assert np.allclose(got, plain.frequencies(rot).numpy(), rtol=1e-13, atol=0), rot


def test_rotation_by_hand():
    """Pairs (2i, 2i + 1) turn by p f_i; elements behind the rotated ones pass."""
    x = torch.tensor([[[1.0, 0.0, 0.0, 2.0, 5.0, 7.0]]], dtype=F)
    freq = torch.tensor([0.5, 0.25], dtype=F)
    out = plain.rotate(x, torch.tensor([3]), freq)[0, 0]
    a, b = 1.5, 0.75
    want = [math.cos(a), math.sin(a), -2.0 * math.sin(b), 2.0 * math.cos(b), 5.0, 7.0]
    assert torch.allclose(out, torch.tensor(want, dtype=F), atol=1e-14)


def test_router_by_hand():
    """Four experts in two groups, one group kept, two chosen. Scores are sigmoid(z);
    the correction moves the choice and never a weight."""
    router = {"experts": 4, "top": 2, "scale": 3.0, "groups": {"count": 2, "keep": 1}}
    s = torch.tensor([[0.9, 0.1, 0.6, 0.55]], dtype=F)
    z = torch.log(s / (1 - s))
    # no correction: group 0 sums 1.0, group 1 sums 1.15 -> group 1, experts 2 and 3
    chosen, weights = plain.route(router, z, torch.zeros(4, dtype=F))
    assert chosen.tolist() == [[2, 3]]
    assert torch.allclose(weights, torch.tensor([[0.6, 0.55]], dtype=F) / 1.15 * 3.0, atol=1e-12)
    # a correction lifts expert 1 to 0.6: group 0 sums 0.9 + 0.6 = 1.5 -> experts 0 and 1
    # in this order, weighted by their uncorrected scores 0.9 and 0.1
    chosen, weights = plain.route(router, z, torch.tensor([0.0, 0.5, 0.0, 0.0], dtype=F))
    assert chosen.tolist() == [[0, 1]]
    assert torch.allclose(weights, torch.tensor([[0.9, 0.1]], dtype=F) / 1.0 * 3.0, atol=1e-12)
    # negative choice values: a group whose experts are all pushed below zero still ranks
    # above nothing, and experts outside the kept group are never chosen
    chosen, _ = plain.route(router, z, torch.tensor([-2.0, -2.0, -3.0, -3.0], dtype=F))
    assert chosen.tolist() == [[0, 1]]
    # no groups at all: the two largest choice values
    chosen, _ = plain.route({"experts": 4, "top": 2, "scale": 1.0}, z, torch.zeros(4, dtype=F))
    assert chosen.tolist() == [[0, 2]]


@pytest.mark.parametrize("name", list(tiny.CONFIGS))
def test_whole_sequence_forms_equal_the_stepwise_ones(name):
    cfg, w = tiny.CONFIGS[name], double(tiny.random_weights(name))
    torch.manual_seed(3)
    T = 37
    h = torch.randn(T, cfg["width"], dtype=F)
    positions = torch.arange(T)
    kept = {}
    for i, layer in enumerate(cfg["layers"]):
        m, p = layer["mixer"], f"l{i}.mix"
        if layer["type"] == "latent_attention":
            whole = plain.latent_attention(m, w, p, h, positions, cfg["norm"]["eps"])
            steps = plain.latent_attention_stepwise(m, w, p, h, positions, cfg["norm"]["eps"])
        else:
            kv = None
            if m.get("kv_from") is None:
                kept[i] = plain.attention_keys_values(m, w, p, h, positions)
            else:
                kv = kept[m["kv_from"]]
            whole = plain.attention(m, w, p, h, positions, kv=kv)
            steps = plain.attention_stepwise(m, w, p, h, positions, kv=kv)
        assert torch.allclose(whole, steps, rtol=1e-10, atol=1e-11), (name, i)


def test_a_prefix_of_a_sequence_gives_the_same_logits():
    cfg, w = tiny.CONFIGS["mixed"], tiny.random_weights("mixed")
    tokens = [int(t) for t in np.random.default_rng(1).integers(0, cfg["vocab"], 30)]
    whole = plain.forward(cfg, w, tokens)
    part = plain.forward(cfg, w, tokens[:11])
    assert torch.allclose(whole[:11], part, rtol=1e-10, atol=1e-10)


def test_the_sink_and_the_gate_matter_in_the_plain_model():
    cfg, w = tiny.CONFIGS["mixed"], double(tiny.random_weights("mixed"))
    torch.manual_seed(4)
    h = torch.randn(20, cfg["width"], dtype=F)
    positions = torch.arange(20)
    m = cfg["layers"][1]["mixer"]
    base = plain.attention(m, w, "l1.mix", h, positions)
    silent = dict(w, **{"l1.mix.sink": torch.full((m["heads"],), -1e4, dtype=F)})
    assert (plain.attention(m, silent, "l1.mix", h, positions) - base).norm() > 0.05 * base.norm()
    # the first token sees itself and the sink only: its output is the value's share
    one = plain.attention(m, w, "l1.mix", h[:1], positions[:1])
    assert torch.allclose(one, base[:1], atol=1e-12)
    lm = cfg["layers"][0]["mixer"]
    gated = plain.latent_attention(lm, w, "l0.mix", h, positions, 1e-5)
    open_gate = dict(w, **{"l0.mix.g": torch.zeros_like(w["l0.mix.g"])})  # sigmoid(0) = 1/2
    half = plain.latent_attention(lm, open_gate, "l0.mix", h, positions, 1e-5)
    assert (gated - half).norm() > 0.05 * gated.norm()


# ------------------------------------------------------------------ configuration
@pytest.mark.parametrize("name", list(tiny.CONFIGS))
def test_configuration_round_trip_and_spec(name):
    from foundry_b200.config.kutepel import KutepelConfig
    from foundry_b200.engine.model import expected_tensors
    doc = tiny.CONFIGS[name]
    cfg = KutepelConfig.parse(json.dumps(doc))
    assert cfg.to_json() == doc
    spec = spec_of(doc)
    want = tiny.tensor_shapes(doc)
    got = expected_tensors(spec)
    assert set(got) == set(want)
    assert all(tuple(got[k].shape) == tuple(want[k]) for k in want)
    assert spec.output_head_name is None  # the embedding table is the output head
    for i, (layer, entry) in enumerate(zip(doc["layers"], spec.schedule)):
        source = layer["mixer"].get("kv_from")
        assert entry.layer == i
        assert (entry.cache, entry.writes_cache) == ((i, True) if source is None else (source, False))


def test_absent_keys_mean_none():
    from foundry_b200.config.kutepel import KutepelConfig
    doc = copy.deepcopy(tiny.CONFIGS["other"])
    del doc["layers"][0]["mlp"]["router"]["groups"]
    del doc["layers"][0]["mixer"]["rot"]["scaling"]
    del doc["layers"][1]["mixer"]["rot"]["scaling"]
    doc["layers"][2]["mlp"] = None
    cfg = KutepelConfig.parse(doc)
    assert cfg.layers[0].mlp.group_count == 1 and cfg.layers[0].rot_scaling is None
    assert cfg.layers[2].mlp is None
    assert cfg.to_json() == doc


def test_configuration_errors():
    from foundry_b200.config import errors
    from foundry_b200.config.kutepel import KutepelConfig

    def broken(change):
        doc = copy.deepcopy(tiny.CONFIGS["mixed"])
        change(doc)
        return doc

    cases = [
        (lambda d: d["layers"][3]["mixer"].update(kv_from=3), errors.ConfigJson),   # itself
        (lambda d: d["layers"][3]["mixer"].update(kv_from=0), errors.ConfigJson),   # a latent layer
        (lambda d: d["layers"][4]["mixer"].update(kv_from=3), errors.ConfigJson),   # a reader
        (lambda d: d["layers"][3]["mixer"].update(dim=32), errors.ConfigJson),      # other key size
        (lambda d: d["layers"][1]["mixer"].update(kv_heads=4), errors.HeadRatio),
        (lambda d: d["layers"][1]["mixer"]["rot"].update(dims=18), errors.ConfigJson),
        (lambda d: d["layers"][1]["mixer"]["rot"].update(dims=5), errors.ConfigJson),
        (lambda d: d["layers"][0]["mlp"]["router"]["groups"].update(count=4), errors.ConfigJson),
        (lambda d: d["layers"][0]["mlp"]["router"].update(top=5), errors.ConfigJson),
        (lambda d: d["layers"][0]["mlp"].update(kind="dense"), errors.UnsupportedOption),
        (lambda d: d["layers"][0].update(type="delta"), errors.UnsupportedOption),
        (lambda d: d.pop("residual_mult"), errors.ConfigJson),
        (lambda d: d.update(architecture="Other"), errors.ModelType),
    ]
    for change, error in cases:
        with pytest.raises(error):
            KutepelConfig.parse(broken(change))


def test_random_weights_folder(tmp_path):
    """The random-weights mode writes the design's own tensor names, and the loader's
    check accepts the folder."""
    from foundry_b200.config.kutepel import KutepelConfig
    from foundry_b200.weights.random_init import write_model_folder
    from foundry_b200.weights.safetensors_io import WeightFiles
    folder = write_model_folder(str(tmp_path / "m"), KutepelConfig.parse(tiny.CONFIGS["other"]), 3)
    files = WeightFiles.open(folder)
    assert set(files.names()) == set(tiny.tensor_shapes(tiny.CONFIGS["other"]))
