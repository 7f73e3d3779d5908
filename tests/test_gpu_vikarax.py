"""Vikarax on the GPU against the plain implementation (tests/plain_vikarax.py):
every mechanism alone, then whole models in every cutting of the same tokens
(whole prompts, token by token, portions down to two tokens, mixed batches),
slots and pages that are used again, keys far back, at the borders of cache
pages and on both sides of every chunk's edge, states whose first token still
weighs on the last, long decoding, and greedy generation through the engine's
own loop and the command line."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_vikarax as plain
import vikarax_tiny as tiny

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
ROOT = os.path.normpath(os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
DTYPES = [torch.float32, torch.bfloat16]


def rel_error(got, want):
    """Largest row error: rms of the difference over rms of the wanted values."""
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    assert got.shape == want.shape and np.isfinite(got).all()
    scale = max(np.sqrt((want ** 2).mean()), 1e-12)
    return float(np.sqrt(((got - want) ** 2).mean(-1)).max() / scale)


def bound(dtype, loose=1.0):
    return (3e-5 if dtype in (torch.float32, "float32") else 4e-2) * loose


def double(weights):
    return {k: v.double() for k, v in weights.items()}


def make_ctx(cache, slots, counts, vocab=1000):
    from foundry_b200.engine import SequenceStep, build_context
    return build_context(cache, [SequenceStep(s, [0] * n, []) for s, n in zip(slots, counts)],
                         vocab, DEV)


def spec_of(doc):
    from foundry_b200.config.registry import resolve_architecture
    arch = resolve_architecture(doc)
    return arch.build_spec(arch.parse_config(doc))


def loader(weights, dtype):
    return lambda n: weights[n].to(DEV).to(dtype if weights[n].dim() > 1 else torch.float32)


def one_layer(m, W, eps, mlp=None):
    return {"architecture": "Vikarax", "vocab": 8, "width": W, "norm": {"eps": eps},
            "logit_softcap": 10.0, "layers": [{"type": "parallel", "mixer": m, "mlp": mlp}]}


def mixer_part(m, W, eps, weights, dtype, prefix="a", side=None):
    """The parallel mixer of the library, built the way the architecture builds it; or
    one of its sides alone (`side`: "left" or "right"; tensors under `prefix.side`)."""
    from foundry_b200.parts import MIXERS
    spec = spec_of(one_layer(m, W, eps)).layers[0].mixer
    if side is not None:
        spec, prefix = spec.params[side], f"{prefix}.{side}"
    part = MIXERS.build(spec, dtype=dtype, device=DEV)
    mine = {k for k in weights if k.startswith(prefix + ".")}
    assert set(part.expected_tensors(prefix)) == mine
    part.load(prefix, loader(weights, dtype))
    return part


def run_mixer(part, cache, xs, cuts, dtype):
    """Feed the sequences `xs` through the mixer in rounds (`cuts[k]`: the rows sequence k
    brings round by round); every sequence's outputs in order."""
    slots = [cache.open_sequence() for _ in xs]
    pieces, done = [[] for _ in xs], [0] * len(xs)
    for step in range(max(len(c) for c in cuts)):
        live = [k for k in range(len(xs)) if step < len(cuts[k])]
        counts = [cuts[k][step] for k in live]
        x = torch.cat([xs[k][done[k]:done[k] + c] for k, c in zip(live, counts)]).to(DEV).to(dtype)
        out = part.forward(make_ctx(cache, [slots[k] for k in live], counts), x, cache.view(0, True))
        from foundry_b200.kernels import ops
        out = out.sum(torch.float32) if isinstance(out, ops.Planes) else out
        for k, rows in zip(live, torch.split(out, counts)):
            pieces[k].append(rows.float().cpu())
            done[k] += rows.shape[0]
    for s in slots:
        cache.close_sequence(s)
    return [torch.cat(p) for p in pieces]


def new_cache(part, tokens, slots, dtype):
    from foundry_b200.cache import SequenceCache
    return SequenceCache({0: part.cache_request()}, tokens, slots, dtype, DEV)


PLAIN_SIDE = {"left": plain.sigmoid_attention, "right": plain.state_space}


# ------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(tiny.CONFIGS))
def test_each_side_and_the_pair_in_two_cuttings(name, dtype):
    """Every layer's attention alone, its state-space layer alone, and the two side by
    side, each with a cache of its own: two sequences of unequal lengths in one step,
    then on the slots and pages that were just given back the same rows as a prompt
    part, portions of two tokens and single tokens."""
    cfg, weights = tiny.CONFIGS[name], tiny.random_weights(name)
    eps, W = cfg["norm"]["eps"], cfg["width"]
    torch.manual_seed(5)
    lens = [139, 6]
    xs = [torch.randn(n, W).to(dtype).float() for n in lens]
    for i, layer in enumerate(cfg["layers"]):
        prefix, m = f"l{i}.mix", layer["mixer"]
        mine = {k: v for k, v in weights.items() if k.startswith(prefix + ".")}
        for side in ("left", "right", None):
            part = mixer_part(m, W, eps, mine, dtype, prefix, side)
            cache = new_cache(part, 1024, 4, dtype)
            if side is None:
                want = [plain.parallel_mixer(m, double(mine), prefix, x.double(), eps) for x in xs]
            else:
                want = [PLAIN_SIDE[side](m[side], double(mine), f"{prefix}.{side}", x.double(), eps)
                        for x in xs]
            for cuts in ([[139], [6]], [[70, 2, 1, 1, 63, 2], [3, 2, 1]]):
                got = run_mixer(part, cache, xs, cuts, dtype)
                for g, w in zip(got, want):
                    assert rel_error(g, w) < bound(dtype), (name, i, side, cuts)


OTHER_SIZES = [
    # keys and values of the tensor-core prompt kernel's sizes, chunks of one page, of two,
    # of a size no page divides; one key head for all; every element rotated, none rotated
    {"left": {"heads": 4, "kv_heads": 1, "dim": 64, "vdim": 64, "scale": 0.125,
              "mask": {"size": 64}, "rot": {"dims": 64, "base": 10000.0}},
     "right": {"heads": 1, "vdim": 64, "state": 16, "groups": 1, "conv": 4, "norm_groups": 1},
     "left_scale": 1.0, "right_scale": 1.0},
    {"left": {"heads": 2, "kv_heads": 2, "dim": 128, "vdim": 128, "scale": 0.09,
              "mask": {"size": 128}},
     "right": {"heads": 8, "vdim": 8, "state": 128, "groups": 2, "conv": 5, "norm_groups": 8},
     "left_scale": 0.25, "right_scale": 2.0},
    {"left": {"heads": 3, "kv_heads": 3, "dim": 32, "vdim": 64, "scale": 0.2,
              "mask": {"size": 77}, "rot": {"dims": 16, "base": 77.0}},
     "right": {"heads": 3, "vdim": 36, "state": 20, "groups": 3, "conv": 1, "norm_groups": 2},
     "left_scale": 1.5, "right_scale": 0.1},
    # no chunks at all (every earlier key visible), odd sizes everywhere
    {"left": {"heads": 5, "kv_heads": 5, "dim": 12, "vdim": 20, "scale": 0.4,
              "rot": {"dims": 2, "base": 3.0}},
     "right": {"heads": 6, "vdim": 10, "state": 6, "groups": 2, "conv": 2, "norm_groups": 5},
     "left_scale": 0.9, "right_scale": 0.9},
    # a chunk of one position: a token sees itself only
    {"left": {"heads": 2, "kv_heads": 1, "dim": 16, "vdim": 16, "scale": 0.3,
              "mask": {"size": 1}, "rot": {"dims": 8, "base": 100.0}},
     "right": {"heads": 2, "vdim": 16, "state": 8, "groups": 1, "conv": 3, "norm_groups": 2},
     "left_scale": 1.0, "right_scale": 1.0},
    # a chunk longer than every sequence of the test
    {"left": {"heads": 8, "kv_heads": 4, "dim": 64, "vdim": 128, "scale": 0.1,
              "mask": {"size": 4096}, "rot": {"dims": 16, "base": 5000.0}},
     "right": {"heads": 4, "vdim": 64, "state": 64, "groups": 4, "conv": 4, "norm_groups": 1},
     "left_scale": 0.8, "right_scale": 1.25},
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", range(len(OTHER_SIZES)))
def test_mixers_at_other_sizes(case, dtype):
    m = OTHER_SIZES[case]
    W, eps = 96, 1e-5
    weights = tiny.random_tensors(tiny.mixer_shapes("a", m, W), seed=case)
    part = mixer_part(m, W, eps, weights, dtype)
    cache = new_cache(part, 1024, 3, dtype)
    torch.manual_seed(8 + case)
    xs = [torch.randn(n, W).to(dtype).float() for n in (300, 90)]
    want = [plain.parallel_mixer(m, double(weights), "a", x.double(), eps) for x in xs]
    for cuts in ([[300], [90]], [[130, 2, 100, 1, 1, 66], [66, 2, 20, 1, 1]]):
        got = run_mixer(part, cache, xs, cuts, dtype)
        for g, w in zip(got, want):
            assert rel_error(g, w) < bound(dtype), (m, cuts)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(tiny.CONFIGS))
def test_feed_forwards_alone(name, dtype):
    """The dense feed-forward with the square of relu and the routed experts (sigmoid
    scores, groups of experts, a shared expert or none) at few, some and many rows."""
    from foundry_b200.kernels import ops
    from foundry_b200.parts import FEED_FORWARDS
    cfg, weights = tiny.CONFIGS[name], tiny.random_weights(name)
    spec, wd = spec_of(cfg), double(weights)
    torch.manual_seed(6)
    for rows in (3, 37, 200):
        x = torch.randn(rows, cfg["width"]).to(dtype)
        for i, layer in enumerate(cfg["layers"]):
            mlp = layer["mlp"]
            if not mlp:
                continue
            part = FEED_FORWARDS.build(spec.layers[i].feed_forward, dtype=dtype, device=DEV)
            part.load(f"l{i}.mlp", loader(weights, dtype))
            got = part.forward(None, x.to(DEV))
            got = got.sum(torch.float32) if isinstance(got, ops.Planes) else got
            want = plain.dense_feed_forward(wd, f"l{i}.mlp", x.double()) if mlp["kind"] == "dense" \
                else plain.routed_experts(mlp, wd, f"l{i}.mlp", x.double())
            assert rel_error(got.float().cpu(), want) < bound(dtype), (name, i, rows)


@pytest.mark.parametrize("chunk", [37, 64, 150, 1000, None])
@pytest.mark.parametrize("sizes", [(64, 64, 4, 2), (128, 128, 2, 1), (96, 64, 3, 3), (32, 128, 2, 2)])
def test_prompt_attention_on_the_tensor_cores(sizes, chunk):
    """The bfloat16 prompt kernel against the plain attention and against the CUDA-core
    kernel on the same cache: chunks that end inside a block of 64 queries and inside a
    cache page, portions that begin in the middle of a chunk and of a page, three unequal
    sequences a step; and the kernel counted, so that no other path stands in for it."""
    from foundry_b200.kernels import ops
    d, e, heads, kv_heads = sizes
    left = {"heads": heads, "kv_heads": kv_heads, "dim": d, "vdim": e, "scale": d ** -0.5,
            "rot": {"dims": d // 2, "base": 1000.0}}
    if chunk:
        left["mask"] = {"size": chunk}
    W, eps = 64, 1e-5
    shapes = {k: v for k, v in tiny.mixer_shapes("a", {"left": left, "right": {
        "heads": 1, "vdim": 8, "state": 8, "groups": 1, "conv": 2, "norm_groups": 1}}, W).items()
        if k.startswith("a.left.")}
    weights = tiny.random_tensors(shapes, seed=d + e)
    from foundry_b200.parts import MIXERS
    spec = spec_of(one_layer({"left": left, "left_scale": 1.0, "right_scale": 1.0, "right": {
        "heads": 1, "vdim": 8, "state": 8, "groups": 1, "conv": 2, "norm_groups": 1}}, W, eps))
    part = MIXERS.build(spec.layers[0].mixer.params["left"], dtype=torch.bfloat16, device=DEV)
    part.load("a.left", loader(weights, torch.bfloat16))
    cache = new_cache(part, 2048, 3, torch.bfloat16)
    torch.manual_seed(d)
    xs = [torch.randn(n, W).to(torch.bfloat16).float() for n in (333, 70, 129)]
    want = [plain.sigmoid_attention(left, double(weights), "a.left", x.double(), eps) for x in xs]
    results = {}
    for tc in (True, False):
        ops.SIGMOID_ATTENTION_TC = tc
        try:
            for cuts in ([[333], [70], [129]], [[100, 133, 2, 98], [5, 65], [64, 65]]):
                ops.PROFILER.start("steps")
                got = run_mixer(part, cache, xs, cuts, torch.bfloat16)
                counts = ops.PROFILER.take()["kernels"]
                ops.PROFILER.start(None)
                n = sum(v["dispatch_count"] for k, v in counts.items()
                        if k.startswith("attention_sigmoid_mma"))
                assert n == (len(cuts[0]) if tc else 0), counts
                results[tc, len(cuts[0])] = got
                for g, w in zip(got, want):
                    assert rel_error(g, w) < bound(torch.bfloat16), (sizes, chunk, tc, cuts)
        finally:
            ops.SIGMOID_ATTENTION_TC = True
    for g, w in zip(results[True, 1], results[False, 1]):  # the two kernels agree more closely
        assert rel_error(g, w) < 0.5 * bound(torch.bfloat16)


# --------------------------------------------- one key that stands out, anywhere
def crafted_attention(W, d, e, chunk, heads=1, kv_heads=1):
    """A parallel mixer whose right side is silent (its constant is 0) and whose
    attention is made so that a query that carries input 1 matches only a key that
    carries input 2: after the heads' norms that score is 20, every other key's about
    +-1, and the bias a head of -10 leaves the others a weight of 1e-4. Queries and keys
    live in the elements behind the rotated ones, so the rotation runs but turns zeros.
    Values are inputs 4..8; the gate is open half way (its weights are zero)."""
    rot = d // 2
    left = {"heads": heads, "kv_heads": kv_heads, "dim": d, "vdim": e, "scale": 20.0 / d,
            "rot": {"dims": rot, "base": 100.0}}
    if chunk:
        left["mask"] = {"size": chunk}
    m = {"left": left, "left_scale": 1.0, "right_scale": 0.0,
         "right": {"heads": 1, "vdim": 8, "state": 8, "groups": 1, "conv": 2, "norm_groups": 1}}
    w = tiny.random_tensors(tiny.mixer_shapes("a", m, W), seed=1)
    q, k = torch.zeros(heads * d, W), torch.zeros(kv_heads * d, W)
    for h in range(heads):
        q[h * d + rot, 1] = 1.0
    for g in range(kv_heads):
        k[g * d + rot, 2] = 1.0
        k[g * d + rot + 1, 0] = 1.0
    val = torch.zeros(kv_heads * e, W)
    for g in range(kv_heads):
        val[g * e:g * e + 4, 4:8] = torch.eye(4)
    out = torch.zeros(W, heads * e)
    n = min(W, e)
    for h in range(heads):
        out[:n, h * e:h * e + n] += torch.eye(n)
    w.update({"a.left.q": q, "a.left.k": k, "a.left.v": val, "a.left.o": out,
              "a.left.g": torch.zeros(heads, W), "a.left.q.norm": torch.ones(d),
              "a.left.k.norm": torch.ones(d), "a.left.pb": torch.full((heads,), -10.0)})
    return m, w


def marked_inputs(query_at, marker_at, width):
    """Rows in which only the query of `query_at` (input 1) and the key of `marker_at`
    (input 2) match; ordinary rows carry input 0. The marker's value (inputs 4..8) is
    unlike every other. With query and marker at the same place the row carries both."""
    gen = torch.Generator().manual_seed(query_at * 1000 + marker_at)
    x = torch.zeros(query_at + 1, width)
    x[:, 0] = 1.0
    x += 0.05 * torch.randn(x.shape, generator=gen)
    x[query_at] = 0.05 * torch.randn(width, generator=gen)
    x[query_at, 0] += 1.0  # (its own key is an ordinary one)
    x[query_at, 1] = 1.0
    if marker_at != query_at:
        x[marker_at] = 0.05 * torch.randn(width, generator=gen)
    x[marker_at, 2] = 1.0
    x[marker_at, 4:8] += 3.0
    return x.to(torch.bfloat16).float()


def places(chunk):
    """(query position, marker position, visible): the chunk's first key and the key in
    front of it, the first token of the sequence, the query itself and its neighbour,
    for queries at the first tokens, on both sides of page borders and far out."""
    out = []
    for q in (5, 64, 65, 129, 200, 700):
        lo = (q // chunk) * chunk if chunk else 0
        seen = {lo, q, max(lo, q - 1)}
        hidden = {lo - 1, 0, lo - 64} if lo > 0 else set()
        out += [(q, j, True) for j in sorted(seen)]
        out += [(q, j, False) for j in sorted(hidden) if j >= 0]
    return out


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("chunk", [64, 100, 640, None])
@pytest.mark.parametrize("sizes", [(8, 8, 1, 1), (64, 64, 2, 1), (32, 128, 2, 2)])
def test_one_key_that_stands_out_on_both_sides_of_every_edge(sizes, chunk, dtype):
    """A crafted attention in which one key dominates one query. The key lies just inside
    or just outside the query's chunk, at the sequence's first token, on both sides of
    cache pages' borders, hundreds of tokens back, or is the query's own; the query is
    the last token of a prompt or a token decoded alone. Sizes of the CUDA-core kernel
    and sizes whose bfloat16 prompts run on the tensor cores."""
    d, e, heads, kv_heads = sizes
    W = 32
    m, weights = crafted_attention(W, d, e, chunk, heads, kv_heads)
    part = mixer_part(m, W, 1e-6, weights, dtype)
    cache = new_cache(part, 2048, 2, dtype)
    wd = double(weights)
    for query_at, marker_at, visible in places(chunk):
        x = marked_inputs(query_at, marker_at, W)
        want = plain.parallel_mixer(m, wd, "a", x.double(), 1e-6)[-1]
        # the plain implementation itself sees the marker where it should and only there
        assert (float(want.norm()) > 0.5) == visible, (query_at, marker_at, float(want.norm()))
        for cut in ([query_at + 1], [query_at, 1]):
            got = run_mixer(part, cache, [x], [cut], dtype)[0][-1].double()
            err = float((got - want).norm()) / max(float(want.norm()), 0.05)
            assert err < bound(dtype, 5.0), (query_at, marker_at, visible, cut, err)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("chunk", [None, 650, 400])
def test_single_tokens_whose_keys_fill_several_runs(chunk, dtype, monkeypatch):
    """The single-token kernel cuts a long range of keys into runs (here of 256 keys, so
    that a few hundred tokens make several) and adds the runs' shares: six query heads on
    one key head with random weights (two blocks a key head, the second partly filled),
    the last tokens decoded alone, against the plain attention; then the crafted key in
    the first run, on both sides of a border between runs, in the last run and just
    outside the chunk. The tokens decoded alone behind 800 others begin a chunk of 400,
    so that all runs of the grid but the first hold no key."""
    from foundry_b200.kernels import ops
    monkeypatch.setattr(ops, "SIGMOID_RUN_KEYS", 256)
    left = {"heads": 6, "kv_heads": 1, "dim": 24, "vdim": 40, "scale": 0.3,
            "rot": {"dims": 8, "base": 50.0}}
    if chunk:
        left["mask"] = {"size": chunk}
    m = {"left": left, "left_scale": 1.0, "right_scale": 0.5,
         "right": {"heads": 2, "vdim": 8, "state": 8, "groups": 1, "conv": 2, "norm_groups": 1}}
    W, eps = 48, 1e-5
    weights = tiny.random_tensors(tiny.mixer_shapes("a", m, W), seed=21)
    part = mixer_part(m, W, eps, weights, dtype)
    cache = new_cache(part, 2048, 2, dtype)
    torch.manual_seed(22)
    x = torch.randn(820, W).to(dtype).float()
    want = plain.parallel_mixer(m, double(weights), "a", x.double(), eps)
    got = run_mixer(part, cache, [x], [[300, 500] + [1] * 20], dtype)[0]
    assert rel_error(got, want) < bound(dtype)

    m, weights = crafted_attention(32, 64, 64, chunk, 2, 1)
    part = mixer_part(m, 32, 1e-6, weights, dtype)
    cache = new_cache(part, 2048, 2, dtype)
    wd = double(weights)
    query_at = 780
    lo = (query_at // chunk) * chunk if chunk else 0
    for marker_at in (lo, lo + 255, lo + 256, lo + 300, query_at - 1, query_at, lo - 1, 0):
        if marker_at < 0 or marker_at > query_at:
            continue
        xm = marked_inputs(query_at, marker_at, 32)
        wanted = plain.parallel_mixer(m, wd, "a", xm.double(), 1e-6)[-1]
        assert (float(wanted.norm()) > 0.5) == (marker_at >= lo), (marker_at, float(wanted.norm()))
        found = run_mixer(part, cache, [xm], [[query_at, 1]], dtype)[0][-1].double()
        err = float((found - wanted).norm()) / max(float(wanted.norm()), 0.05)
        assert err < bound(dtype, 5.0), (chunk, marker_at, err)


@pytest.mark.parametrize("dtype", DTYPES)
def test_state_and_tail_survive_every_cutting(dtype):
    """Decays close to one, so that the first tokens still weigh on the last: the state
    and the convolution's tail carried through portions of one and two tokens equal the
    whole prompt's; the attention beside it is silent."""
    m = {"left": {"heads": 1, "kv_heads": 1, "dim": 8, "vdim": 8, "scale": 0.3, "mask": {"size": 7}},
         "right": {"heads": 4, "vdim": 16, "state": 24, "groups": 2, "conv": 4, "norm_groups": 2},
         "left_scale": 0.0, "right_scale": 1.0}
    weights = tiny.random_tensors(tiny.mixer_shapes("a", m, 48), seed=3)
    weights["a.right.A_log"] = torch.tensor([-6.0, -4.0, -5.0, -7.0])
    part = mixer_part(m, 48, 1e-6, weights, dtype)
    cache = new_cache(part, 1024, 3, dtype)
    torch.manual_seed(4)
    xs = [torch.randn(n, 48).to(dtype).float() for n in (150, 9)]
    wd = double(weights)
    want = [plain.parallel_mixer(m, wd, "a", x.double(), 1e-6) for x in xs]
    moved = xs[0].clone()
    moved[0] += 1.0  # (the plain form itself: the first token still matters at the end)
    assert rel_error(plain.parallel_mixer(m, wd, "a", moved.double(), 1e-6)[-1:], want[0][-1:]) > 1e-3
    for cuts in ([[150], [9]], [[1, 2, 1, 3, 2, 64, 2, 1] + [1] * 10 + [64], [2, 2, 2, 2, 1]]):
        got = run_mixer(part, cache, xs, cuts, dtype)
        for g, w in zip(got, want):
            assert rel_error(g, w) < bound(dtype, 2.0), cuts


def test_a_state_row_starts_at_zero_on_a_slot_that_was_used(dtype=torch.float32):
    """A sequence that opens on a slot whose last owner left a large state and a full
    convolution tail gives what it gives on a fresh cache."""
    m = tiny.CONFIGS["other"]["layers"][0]["mixer"]
    weights = tiny.random_tensors(tiny.mixer_shapes("a", m, 64), seed=9)
    part = mixer_part(m, 64, 1e-6, weights, dtype)
    cache = new_cache(part, 512, 1, dtype)
    torch.manual_seed(1)
    loud, x = 30.0 * torch.randn(80, 64), torch.randn(21, 64)
    want = plain.parallel_mixer(m, double(weights), "a", x.double(), 1e-6)
    run_mixer(part, cache, [loud], [[80]], dtype)
    for cut in ([21], [1] * 21):
        assert rel_error(run_mixer(part, cache, [x], [cut], dtype)[0], want) < bound(dtype)


# ---------------------------------------------------------------- whole models
@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("vikarax")
    return {name: tiny.write_folder(str(root / name), name) for name in tiny.CONFIGS}


CLOSE_CALL, CLOSE_CALL_REACH = 0.01, 12


def settled_rows(name, weights, tokens):
    """Rows whose logits rounding cannot move by much: a router whose two candidates lie
    closer than CLOSE_CALL may choose the other one in bfloat16, and that token then
    weighs on the next ones through the states and the chunk it is in; such rows and the
    CLOSE_CALL_REACH after them are compared in float32 only."""
    margins = []
    plain.forward(tiny.CONFIGS[name], double(weights), tokens, margins=margins)
    ok = np.ones(len(tokens), bool)
    for per_layer in margins:
        for t, gap in enumerate(per_layer):
            if gap < CLOSE_CALL:
                ok[t:t + 1 + CLOSE_CALL_REACH] = False
    return ok


def plain_logits(name, weights, tokens):
    return plain.forward(tiny.CONFIGS[name], double(weights), tokens).numpy()


def run_cutting(engine, prompts, cuts):
    """Feed `prompts` through `engine.step` in rounds; `cuts[k]` are the token
    counts sequence k brings round by round. Logits of every position."""
    from foundry_b200.engine import SequenceStep
    slots = [engine.open_sequence() for _ in prompts]
    done = [0] * len(prompts)
    rows = [[] for _ in prompts]
    for r in range(max(len(c) for c in cuts)):
        live = [k for k in range(len(prompts)) if r < len(cuts[k])]
        steps = [SequenceStep(slots[k], prompts[k][done[k]:done[k] + cuts[k][r]],
                              list(range(cuts[k][r]))) for k in live]
        logits = engine.step(steps).cpu().numpy()
        at = 0
        for k in live:
            n = cuts[k][r]
            rows[k].append(logits[at:at + n])
            at += n
            done[k] += n
            if done[k] == len(prompts[k]):
                engine.close_sequence(slots[k])
    assert done == [len(p) for p in prompts]
    return [np.concatenate(r) for r in rows]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(tiny.CONFIGS))
def test_model_in_every_cutting(name, dtype, folders):
    """Whole prompts alone; token by token from the first token on; portions of
    several sizes down to two tokens; a batch of unequal requests decoded
    together while the shorter ones end; all on slots and pages that the
    earlier cuttings used and gave back."""
    import foundry_b200 as fb
    folder, weights = folders[name]
    vocab = tiny.CONFIGS[name]["vocab"]
    rng = np.random.default_rng(11)
    prompts = [[int(t) for t in rng.integers(0, vocab, n)] for n in (150, 1, 3, 81)]
    want = [plain_logits(name, weights, p) for p in prompts]
    engine = fb.Engine.from_folder(folder, dtype=dtype, max_tokens=1024, max_slots=6)
    results = {}
    results["whole, alone"] = [run_cutting(engine, [p], [[len(p)]])[0] for p in prompts]
    results["token by token"] = [run_cutting(engine, [prompts[k]], [[1] * len(prompts[k])])[0]
                                 for k in (2, 3)]
    results["portions"] = run_cutting(engine, [prompts[0], prompts[3]],
                                      [[2, 62, 1, 64, 2, 17, 2], [77, 2, 2]])
    results["batch, then decoded together"] = run_cutting(
        engine, prompts, [[120] + [1] * 30, [1], [2, 1], [70] + [1] * 11])
    wanted = {"whole, alone": want, "token by token": [want[2], want[3]],
              "portions": [want[0], want[3]], "batch, then decoded together": want}
    rows = {len(p): settled_rows(name, weights, p) if dtype == "bfloat16" else slice(None)
            for p in prompts}
    for cutting, got in results.items():
        for g, w in zip(got, wanted[cutting]):
            assert np.isfinite(g).all()
            keep = rows[len(w)]
            assert rel_error(g[keep], w[keep]) < bound(dtype, 2.0 if dtype == "float32" else 3.0), \
                (name, dtype, cutting, len(w))
    if dtype == "float32":  # the cuttings agree with each other to rounding
        assert rel_error(results["portions"][0], results["whole, alone"][0]) < 2e-5
        assert rel_error(results["batch, then decoded together"][3], results["whole, alone"][3]) < 2e-5
    engine.cache.table.check()
    assert engine.free_slots() == 6


@pytest.mark.parametrize("name", list(tiny.CONFIGS))
def test_long_decoding_and_reused_slots(name, folders):
    """260 tokens decoded one by one behind a short prompt (across cache pages and many
    chunks), twice on the same slot with another sequence between."""
    import foundry_b200 as fb
    folder, weights = folders[name]
    vocab = tiny.CONFIGS[name]["vocab"]
    rng = np.random.default_rng(12)
    tokens = [int(t) for t in rng.integers(0, vocab, 265)]
    other = [int(t) for t in rng.integers(0, vocab, 40)]
    want = plain_logits(name, weights, tokens)
    engine = fb.Engine.from_folder(folder, dtype="float32", max_tokens=512, max_slots=2)
    first = run_cutting(engine, [tokens], [[5] + [1] * 260])[0]
    run_cutting(engine, [other], [[40]])
    again = run_cutting(engine, [tokens], [[5] + [1] * 260])[0]
    assert rel_error(first, want) < bound("float32", 2.0)
    assert np.array_equal(first, again)


def test_sizes_that_fit_no_tensor_core_product_and_layers_in_another_order(tmp_path):
    """Width 52 and inner sizes that are no multiples of 8 (in bfloat16 every product takes
    the CUDA-core kernel); a routed layer first, a layer without feed-forward in the
    middle, one expert group of all experts, every expert chosen, every group kept, constants of 1."""
    import foundry_b200 as fb
    from foundry_b200.weights.safetensors_io import SINGLE_FILE, save_file
    left = {"heads": 3, "kv_heads": 3, "dim": 10, "vdim": 14, "scale": 0.3, "mask": {"size": 33},
            "rot": {"dims": 6, "base": 777.0}}
    right = {"heads": 3, "vdim": 6, "state": 5, "groups": 1, "conv": 3, "norm_groups": 3}
    mixer = {"left": left, "right": right, "left_scale": 1.0, "right_scale": 1.0}
    other = {"left": dict(left, heads=2, kv_heads=1, vdim=9, mask={"size": 2}),
             "right": dict(right, heads=4, groups=4, norm_groups=1, conv=2),
             "left_scale": 0.3, "right_scale": 1.0}
    doc = {"architecture": "Vikarax", "vocab": 77, "width": 52, "norm": {"eps": 1e-5},
           "logit_softcap": 4.0,
           "layers": [
               {"type": "parallel", "mixer": mixer,
                "mlp": {"kind": "moe", "expert": {"ff": 18},
                        "router": {"experts": 3, "top": 3, "groups": {"count": 1, "keep": 1}},
                        "shared": {"ff": 7}}},
               {"type": "parallel", "mixer": other, "mlp": None},
               {"type": "parallel", "mixer": mixer, "mlp": {"kind": "dense", "ff": 90}},
               {"type": "parallel", "mixer": other,
                "mlp": {"kind": "moe", "expert": {"ff": 44},
                        "router": {"experts": 10, "top": 2, "groups": {"count": 5, "keep": 5}}}}]}
    weights = tiny.random_tensors(tiny.tensor_shapes(doc), seed=31)
    folder = tmp_path / "odd"
    folder.mkdir()
    save_file({k: v.to(torch.bfloat16) for k, v in weights.items()}, str(folder / SINGLE_FILE),
              metadata={"format": "pt"})
    (folder / "config.json").write_text(json.dumps(doc))
    rng = np.random.default_rng(3)
    prompts = [[int(t) for t in rng.integers(0, 77, n)] for n in (70, 9)]
    want = [plain.forward(doc, double(weights), p).numpy() for p in prompts]
    for dtype in ("float32", "bfloat16"):
        engine = fb.Engine.from_folder(str(folder), dtype=dtype, max_tokens=512, max_slots=3)
        got = run_cutting(engine, prompts, [[66, 2, 1, 1], [5, 1, 2, 1]])
        for g, w in zip(got, want):
            assert rel_error(g, w) < bound(dtype, 2.0), dtype


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_engine(dtype, folders):
    """`Engine.generate` (the scheduler's batches, graphs, slot reuse) against the
    plain model's greedy tokens; five prompts through batches of two."""
    import foundry_b200 as fb
    folder, weights = folders["mixed"]
    cfg = tiny.CONFIGS["mixed"]
    rng = np.random.default_rng(13)
    prompts = [[int(t) for t in rng.integers(0, cfg["vocab"], n)] for n in (9, 1, 30, 4, 17)]
    engine = fb.Engine.from_folder(folder, dtype=dtype, max_tokens=512, max_slots=4)
    got = engine.generate(prompts, 8, eos_token_id=[], max_batch=2).token_ids
    wd = double(weights)
    for g, p in zip(got, prompts):
        w = plain.greedy_generate(cfg, wd, p, 8)
        if g == w:
            continue
        k = next(i for i, (a, b) in enumerate(zip(g, w)) if a != b)
        logits = plain.forward(cfg, wd, list(p) + w[:k])[-1]
        gap = float(logits[w[k]] - logits[g[k]])
        assert dtype == "bfloat16" and gap < 0.05 * float(logits.abs().max()), (g, w, gap)


def test_trace_replay_and_command_line(folders, tmp_path):
    """`bin/trace_run` on a Vikarax folder: a prompt step of two requests, then
    single tokens, one request ending early; and `foundry run` generating."""
    folder, weights = folders["other"]
    cfg = tiny.CONFIGS["other"]
    rng = np.random.default_rng(14)
    a = [int(t) for t in rng.integers(0, cfg["vocab"], 12)]
    b = [int(t) for t in rng.integers(0, cfg["vocab"], 5)]
    lines = [{"step": 0, "entries": [{"id": "a", "tokens": a[:10], "want": [0, 9]},
                                     {"id": "b", "tokens": b[:4], "want": [3]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[10:11], "want": []},
                                     {"id": "b", "tokens": b[4:], "want": [0]}], "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": a[11:], "want": [0]}], "end": ["a"]}]
    out = tmp_path / "out"
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder,
                           "--dtype", "float32", "--out", str(out), "--max-tokens", "128"],
                          input="".join(json.dumps(l) + "\n" for l in lines), capture_output=True,
                          text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.split("\n") if l.startswith("done")] == ["done 0", "done 1", "done 2"]
    wa, wb = plain_logits("other", weights, a), plain_logits("other", weights, b)
    V = cfg["vocab"]
    got0 = np.fromfile(out / "0.f32", dtype="<f4").reshape(-1, V)
    got1 = np.fromfile(out / "1.f32", dtype="<f4").reshape(-1, V)
    got2 = np.fromfile(out / "2.f32", dtype="<f4").reshape(-1, V)
    assert rel_error(got0, np.stack([wa[0], wa[9], wb[3]])) < bound("float32", 2.0)
    assert rel_error(got1, wb[4:5]) < bound("float32", 2.0)
    assert rel_error(got2, wa[11:12]) < bound("float32", 2.0)
    run = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "foundry"), "run", "--model",
                          folder, "--dtype", "float32", "--prompt-ids", ",".join(map(str, a)),
                          "--max-new-tokens", "4", "--ignore-eos"], capture_output=True, text=True,
                         timeout=600)
    assert run.returncode == 0, run.stderr[-2000:]
    want = plain.greedy_generate(cfg, double(weights), a, 4)
    assert json.loads(run.stdout.strip().split("\n")[-1]) == want


def test_command_line_bench_on_a_vikarax_folder(folders, tmp_path):
    """`foundry bench` (prompt step, decode steps, report with bytes and operations)
    on a model whose cache entries hold pages and a state row at once."""
    folder, _ = folders["mixed"]
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "foundry"), "bench", "--model",
                           folder, "--prompt-tokens", "20", "--new-tokens", "5", "--runs", "2",
                           "--batch-size", "3", "--out", str(tmp_path)],
                          capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    report = json.loads((tmp_path / "report.json").read_text())
    assert len(report["runs"]) == 2 and all(len(r) == 5 for r in report["runs"][0]["token_ids"])
    assert report["runs"][0]["token_ids"] == report["runs"][1]["token_ids"]
