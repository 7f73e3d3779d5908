"""Vikarax without a GPU: configuration, the model as data, the tensor list,
the cache entry that holds pages and a state row, and the plain
implementation against its own token-by-token form and against cases worked
by hand."""
import json
import math

import pytest
import torch

import plain_vikarax as plain
import vikarax_tiny as tiny


def parsed(name):
    from foundry_b200.config.vikarax import VikaraxConfig
    return VikaraxConfig.parse(tiny.CONFIGS[name])


def double(weights):
    return {k: v.double() for k, v in weights.items()}


@pytest.mark.parametrize("name", list(tiny.CONFIGS))
def test_config_round_trip_and_registry(name):
    from foundry_b200.config.registry import resolve_architecture
    cfg = parsed(name)
    assert type(cfg).parse(json.dumps(cfg.to_json())) == cfg
    assert resolve_architecture(tiny.CONFIGS[name]).name == "Vikarax"
    doc = tiny.CONFIGS[name]
    assert cfg.width == doc["width"] and len(cfg.layers) == len(doc["layers"])
    assert cfg.logit_softcap == doc["logit_softcap"]
    for layer, entry in zip(cfg.layers, doc["layers"]):
        assert layer.left.chunk == entry["mixer"]["left"]["mask"]["size"]
        assert layer.right.taps == entry["mixer"]["right"]["conv"]
        assert (layer.mlp is None) == (entry["mlp"] is None)


def test_config_defaults_of_absent_keys():
    doc = json.loads(json.dumps(tiny.CONFIGS["other"]))
    left = doc["layers"][0]["mixer"]["left"]
    del left["mask"], left["rot"]
    del doc["layers"][1]["mlp"]["router"]["groups"]
    del doc["logit_softcap"]
    from foundry_b200.config.vikarax import VikaraxConfig
    cfg = VikaraxConfig.parse(doc)
    assert cfg.layers[0].left.chunk is None and cfg.layers[0].left.rot_dims == 0
    assert (cfg.layers[1].mlp.group_count, cfg.layers[1].mlp.group_keep) == (1, 1)
    assert cfg.layers[1].mlp.shared_ff == 0 and cfg.logit_softcap is None


def test_config_refusals():
    from foundry_b200.config import errors
    from foundry_b200.config.vikarax import VikaraxConfig
    fresh = lambda: json.loads(json.dumps(tiny.CONFIGS["mixed"]))
    doc = fresh()
    doc["layers"][0]["mixer"]["left"]["kv_heads"] = 4
    with pytest.raises(errors.HeadRatio):
        VikaraxConfig.parse(doc)
    doc = fresh()
    doc["layers"][1]["type"] = "serial"
    with pytest.raises(errors.UnsupportedOption):
        VikaraxConfig.parse(doc)
    doc = fresh()
    doc["layers"][0]["mlp"]["router"]["groups"]["count"] = 4  # 6 experts in 4 groups
    with pytest.raises(errors.ConfigJson):
        VikaraxConfig.parse(doc)
    doc = fresh()
    doc["layers"][0]["mlp"]["router"]["groups"]["keep"] = 1  # 3 chosen out of one group of 2
    with pytest.raises(errors.ConfigJson):
        VikaraxConfig.parse(doc)
    doc = fresh()
    doc["layers"][0]["mixer"]["left"]["rot"]["dims"] = 26  # more than the head has
    with pytest.raises(errors.ConfigJson):
        VikaraxConfig.parse(doc)
    doc = fresh()
    doc["layers"][1]["mixer"]["right"]["norm_groups"] = 5
    with pytest.raises(errors.ConfigJson):
        VikaraxConfig.parse(doc)
    doc = fresh()
    del doc["norm"]
    with pytest.raises(errors.ConfigJson):
        VikaraxConfig.parse(doc)


@pytest.mark.parametrize("name", list(tiny.CONFIGS))
def test_tensor_list_and_the_model_as_data(name):
    from foundry_b200.cache import JointRequest
    from foundry_b200.engine.model import Model, expected_tensors
    from foundry_b200.models.vikarax import build_vikarax_spec
    spec = build_vikarax_spec(parsed(name))
    listed = expected_tensors(spec)
    assert {k: tuple(v.shape) for k, v in listed.items()} == tiny.tensor_shapes(tiny.CONFIGS[name])
    assert [(e.layer, e.cache) for e in spec.schedule] == [(i, i) for i in range(len(spec.layers))]
    assert spec.logit_softcap == tiny.CONFIGS[name]["logit_softcap"]
    model = Model(spec, torch.bfloat16, torch.device("meta"))
    for i, (block, entry) in enumerate(zip(model.blocks, tiny.CONFIGS[name]["layers"])):
        assert block.depth == i + 1 and block.needs_embedding_output
        want = block.cache_request()
        left, right = entry["mixer"]["left"], entry["mixer"]["right"]
        assert isinstance(want, JointRequest)
        assert (want.kv.kv_heads, want.kv.head_dim, want.kv.v_head_dim, want.kv.window) == \
            (left["kv_heads"], left["dim"], left["vdim"], None)
        channels = right["heads"] * right["vdim"] + 2 * right["groups"] * right["state"]
        assert want.state.shape == ((right["conv"] - 1) * channels +
                                    right["heads"] * right["state"] * right["vdim"],)
        assert want.state.dtype == torch.float32


def test_a_cache_entry_with_pages_and_a_state_row():
    from foundry_b200.cache import (JointRequest, JointView, KVRequest, KVView, SequenceCache,
                                    StateRequest, StateView)
    kv = KVRequest(2, 8, None, 4)
    requests = {0: JointRequest(kv, StateRequest((6,))), 1: KVRequest(2, 8, None, 4),
                2: StateRequest((3,)), 3: JointRequest(kv, StateRequest((5,)))}
    cache = SequenceCache(requests, 256, 3, torch.float32, torch.device("cpu"))
    assert len(cache.groups) == 1 and cache.groups[0].entries == [0, 1, 3]
    view = cache.view(0, True)
    assert isinstance(view, JointView) and view.kv.k.shape[-1] == 8 and view.kv.v.shape[-1] == 4
    assert view.state.rows.shape == (4, 6) and cache.view(3, True).state.rows.shape == (4, 5)
    assert isinstance(cache.view(1, True), KVView) and isinstance(cache.view(2, True), StateView)
    slot = cache.open_sequence()
    cache.view(0, True).state.rows[slot] += 2.0
    cache.reserve({slot: 70})
    cache.close_sequence(slot)
    again = cache.open_sequence()
    assert again == slot and float(cache.view(0, True).state.rows[slot].abs().sum()) == 0.0
    cache.table.check()


@pytest.mark.parametrize("name", list(tiny.CONFIGS))
def test_plain_state_space_equals_its_stepwise_form(name):
    cfg, w = tiny.CONFIGS[name], double(tiny.random_weights(name))
    torch.manual_seed(3)
    h = torch.randn(13, cfg["width"], dtype=torch.float64)
    for i, layer in enumerate(cfg["layers"]):
        a = plain.state_space(layer["mixer"]["right"], w, f"l{i}.mix.right", h, cfg["norm"]["eps"])
        b = plain.state_space_stepwise(layer["mixer"]["right"], w, f"l{i}.mix.right", h,
                                       cfg["norm"]["eps"])
        assert float((a - b).abs().max()) < 1e-10 * max(1.0, float(a.abs().max()))


def test_plain_sigmoid_attention_by_hand():
    """One head over four tokens in chunks of three: unnormalised sigmoid weights, the
    bias a head inside the sigmoid, the output gate, unit values, no key from the chunk
    before."""
    m = {"heads": 1, "kv_heads": 1, "dim": 2, "vdim": 2, "scale": 0.5, "mask": {"size": 3}}
    eye = torch.eye(2, dtype=torch.float64)
    w = {"a.q": eye, "a.k": eye, "a.v": eye, "a.o": eye, "a.g": torch.tensor([[0.0, 1.0]], dtype=plain.F),
         "a.q.norm": torch.ones(2, dtype=plain.F), "a.k.norm": torch.ones(2, dtype=plain.F),
         "a.pb": torch.tensor([-0.25], dtype=plain.F)}
    h = torch.tensor([[1.0, 0.0], [0.0, 2.0], [3.0, 0.0], [0.0, 1.0]], dtype=plain.F)
    out = plain.sigmoid_attention(m, w, "a", h, 1e-12)
    r2 = math.sqrt(2.0)  # every q, k and v is sqrt(2) times a unit vector
    sig = lambda z: 1.0 / (1.0 + math.exp(-z))
    # token 2 (chunk 0) sees tokens 0, 1, 2; its query lies along the first axis
    w0, w1 = sig(0.5 * 2.0 - 0.25), sig(-0.25)
    gate2 = sig(0.0)
    assert abs(float(out[2, 0]) - gate2 * (w0 + w0) * r2) < 1e-9
    assert abs(float(out[2, 1]) - gate2 * w1 * r2) < 1e-9
    # token 3 opens chunk 1 and sees itself only
    assert abs(float(out[3, 0])) < 1e-9
    assert abs(float(out[3, 1]) - sig(1.0) * w0 * r2) < 1e-9
    assert plain.chunk_visible(5, 3, 3) and not plain.chunk_visible(5, 2, 3)
    assert not plain.chunk_visible(4, 5, 3) and plain.chunk_visible(700, 0, None)


def test_plain_rotation_pairs_halves_and_leaves_the_rest():
    x = torch.tensor([[[1.0, 2.0, 0.0, 0.0, 7.0, 9.0]]], dtype=plain.F).repeat(3, 1, 1)
    y = plain.rotate_half(x, [0, 1, 5], 4, 100.0)
    assert torch.equal(y[0], x[0]) and torch.equal(y[:, :, 4:], x[:, :, 4:])
    # element 0 turns with element 2 by p * 1, element 1 with element 3 by p * 100^(-1/2)
    assert abs(float(y[2, 0, 0]) - math.cos(5.0)) < 1e-12 and abs(float(y[2, 0, 2]) - math.sin(5.0)) < 1e-12
    assert abs(float(y[1, 0, 1]) - 2.0 * math.cos(0.1)) < 1e-12
    assert abs(float(y[1, 0, 3]) - 2.0 * math.sin(0.1)) < 1e-12


def test_plain_router_groups_by_hand():
    mlp = {"router": {"experts": 6, "top": 2, "groups": {"count": 3, "keep": 1}}}
    # the largest single score sits in group 0, but group 2 has the largest two together
    scores = torch.tensor([0.9, 0.1, 0.5, 0.45, 0.6, 0.55], dtype=plain.F)
    assert plain.route(mlp, scores) == [4, 5]
    mlp["router"]["groups"]["keep"] = 2  # groups 2 (1.15) and 0 (1.0) stay
    assert plain.route(mlp, scores) == [0, 4]
    mlp["router"]["groups"] = {"count": 1, "keep": 1}
    assert plain.route(mlp, scores) == [0, 4]
    mlp["router"] = {"experts": 6, "top": 3, "groups": {"count": 6, "keep": 3}}  # groups of one
    assert plain.route(mlp, scores) == [0, 4, 5]


@pytest.mark.parametrize("name", list(tiny.CONFIGS))
def test_plain_model_is_causal_and_keeps_every_stream(name):
    cfg, w = tiny.CONFIGS[name], double(tiny.random_weights(name))
    gen = torch.Generator().manual_seed(4)
    tokens = torch.randint(0, cfg["vocab"], (27,), generator=gen).tolist()
    streams = []
    full = plain.forward(cfg, w, tokens, streams)
    assert len(streams) == len(cfg["layers"]) and full.shape == (27, cfg["vocab"])
    assert float(full.abs().max()) < cfg["logit_softcap"]
    head = plain.forward(cfg, w, tokens[:12])
    assert float((full[:12] - head).abs().max()) < 1e-9
    # the weighted sum over the streams: changing the weight of the embedding's stream in
    # the last layer moves the logits
    w2 = dict(w)
    last = len(cfg["layers"]) - 1
    w2[f"l{last}.dwa"] = w[f"l{last}.dwa"].clone()
    w2[f"l{last}.dwa"][0] += 0.5
    assert float((plain.forward(cfg, w2, tokens) - full).abs().max()) > 1e-3
