"""Kutepel on the GPU against the plain implementation (tests/plain_kutepel.py):
every mechanism alone, then whole models in every cutting of the same tokens (whole
prompts, token by token, portions down to two tokens, mixed batches), slots and pages
that are used again, keys far back and at the borders of cache pages, the sink, the
gate, a layer that reads another's keys and values, the router's every rule, long
decoding, and greedy generation through the engine's own loop and the command line."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import kutepel_tiny as tiny
import plain_kutepel as plain

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


def layer_doc(kind, m, W, eps, mlp=None, before=()):
    return {"architecture": "Kutepel", "vocab": 8, "width": W, "norm": {"eps": eps},
            "residual_mult": 1.0,
            "layers": list(before) + [{"type": kind, "mixer": m, "mlp": mlp}]}


def mixer_part(kind, m, W, eps, weights, dtype, prefix="a", before=()):
    """A mixer of the library built the way the architecture builds it."""
    from foundry_b200.parts import MIXERS
    part = MIXERS.build(spec_of(layer_doc(kind, m, W, eps, before=before)).layers[-1].mixer,
                        dtype=dtype, device=DEV)
    assert set(part.expected_tensors(prefix)) == set(weights)
    part.load(prefix, loader(weights, dtype))
    return part


def plain_mixer(kind, m, weights, prefix, x, eps, kv=None):
    positions = torch.arange(x.shape[0])
    if kind == "latent_attention":
        return plain.latent_attention(m, weights, prefix, x, positions, eps)
    return plain.attention(m, weights, prefix, x, positions, kv=kv)


def run_mixer(parts, cache, xs, cuts, dtype):
    """Feed the sequences `xs` through the mixers `parts` (run one after the other on the
    same input and the same cache entry: the first writes it, the others only read it) in
    rounds (`cuts[k]`: the rows sequence k brings round by round); per part, every
    sequence's outputs in order."""
    parts = parts if isinstance(parts, (list, tuple)) else [parts]
    slots = [cache.open_sequence() for _ in xs]
    pieces = [[[] for _ in xs] for _ in parts]
    done = [0] * len(xs)
    for step in range(max(len(c) for c in cuts)):
        live = [k for k in range(len(xs)) if step < len(cuts[k])]
        counts = [cuts[k][step] for k in live]
        x = torch.cat([xs[k][done[k]:done[k] + c] for k, c in zip(live, counts)]).to(DEV).to(dtype)
        ctx = make_ctx(cache, [slots[k] for k in live], counts)
        for n, part in enumerate(parts):
            out = part.forward(ctx, x, cache.view(0, n == 0))
            for k, rows in zip(live, torch.split(out, counts)):
                pieces[n][k].append(rows.float().cpu())
        for k, c in zip(live, counts):
            done[k] += c
    for s in slots:
        cache.close_sequence(s)
    out = [[torch.cat(p) for p in per_part] for per_part in pieces]
    return out if len(parts) > 1 else out[0]


# ------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(tiny.CONFIGS))
def test_each_mixer_alone_in_two_cuttings(name, dtype):
    """Every mixer of both configurations that has keys and values of its own, with a
    cache of its own: two sequences of unequal lengths in one step, then on the slots and
    pages that were just given back the same rows as a prompt part, portions of two tokens
    and single tokens."""
    from foundry_b200.cache import SequenceCache
    cfg, weights = tiny.CONFIGS[name], tiny.random_weights(name)
    eps = cfg["norm"]["eps"]
    torch.manual_seed(5)
    for i, layer in enumerate(cfg["layers"]):
        if layer["mixer"].get("kv_from") is not None:
            continue
        prefix = f"l{i}.mix"
        mine = {k: v for k, v in weights.items() if k.startswith(prefix + ".")}
        part = mixer_part(layer["type"], layer["mixer"], cfg["width"], eps, mine, dtype, prefix)
        cache = SequenceCache({0: part.cache_request()}, 1024, 4, dtype, DEV)
        lens = [139, 6]
        xs = [torch.randn(n, cfg["width"]).to(dtype).float() for n in lens]
        want = [plain_mixer(layer["type"], layer["mixer"], double(mine), prefix, x.double(), eps)
                for x in xs]
        for cuts in ([[139], [6]], [[70, 2, 1, 1, 63, 2], [3, 2, 1]]):
            got = run_mixer(part, cache, xs, cuts, dtype)
            for g, w in zip(got, want):
                assert rel_error(g, w) < bound(dtype), (name, i, layer["type"], cuts)


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_mixer_that_reads_another_ones_keys_and_values(dtype):
    """Two readers beside the owner of a cache entry (other head counts, scales and sinks,
    no key and value tensors of their own): in one step, and cut up so that the readers
    see keys that earlier steps wrote."""
    from foundry_b200.cache import SequenceCache
    cfg, weights = tiny.CONFIGS["mixed"], tiny.random_weights("mixed")
    W, eps = cfg["width"], cfg["norm"]["eps"]
    owner_doc = cfg["layers"][1]
    parts, mine = [], []
    for i in (1, 3, 4):
        prefix = f"l{i}.mix"
        mine.append({k: v for k, v in weights.items() if k.startswith(prefix + ".")})
        parts.append(mixer_part("attention", cfg["layers"][i]["mixer"], W, eps, mine[-1], dtype,
                                prefix, before=[owner_doc] * (i > 1) * 2))
    assert not any(k.endswith((".k", ".v")) for k in list(mine[1]) + list(mine[2]))
    assert parts[0].cache_request() == parts[1].cache_request() == parts[2].cache_request()
    cache = SequenceCache({0: parts[0].cache_request()}, 1024, 4, dtype, DEV)
    torch.manual_seed(15)
    xs = [torch.randn(n, W).to(dtype).float() for n in (131, 5)]
    positions = [torch.arange(x.shape[0]) for x in xs]
    kv = [plain.attention_keys_values(owner_doc["mixer"], double(mine[0]), "l1.mix", x.double(), p)
          for x, p in zip(xs, positions)]
    for cuts in ([[131], [5]], [[64, 2, 1, 62, 2], [2, 2, 1]]):
        got = run_mixer(parts, cache, xs, cuts, dtype)
        for n, i in enumerate((1, 3, 4)):
            for k, x in enumerate(xs):
                want = plain.attention(cfg["layers"][i]["mixer"], double(mine[n]), f"l{i}.mix",
                                       x.double(), positions[k], kv=None if n == 0 else kv[k])
                assert rel_error(got[n][k], want) < bound(dtype), (i, k, cuts)


MIXER_CASES = [
    # one key head for five heads; keys of 40 beside values of 12; two rotated elements
    ("attention", {"heads": 5, "kv_heads": 1, "dim": 40, "vdim": 12, "scale": 0.1,
                   "rot": {"base": 3.0, "dims": 2}}),
    # nothing rotated; one head
    ("attention", {"heads": 1, "kv_heads": 1, "dim": 16, "vdim": 16, "scale": 0.3,
                   "rot": {"base": 10000.0, "dims": 0}}),
    # sizes of the tensor-core prompt kernels (bfloat16): 64 and 128, groups of 4 and 1
    ("attention", {"heads": 4, "kv_heads": 1, "dim": 64, "vdim": 64, "scale": 0.1,
                   "rot": {"base": 10000.0, "dims": 64,
                           "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 32}}}),
    ("attention", {"heads": 2, "kv_heads": 2, "dim": 128, "vdim": 128, "scale": 0.08,
                   "rot": {"base": 500000.0, "dims": 96}}),
    ("attention", {"heads": 2, "kv_heads": 1, "dim": 32, "vdim": 32, "scale": 0.2,
                   "rot": {"base": 100.0, "dims": 32}}),
    # keys of 128 beside values of 64 (no tensor-core prompt kernel of one size)
    ("attention", {"heads": 2, "kv_heads": 1, "dim": 128, "vdim": 64, "scale": 0.08,
                   "rot": {"base": 100.0, "dims": 64}}),
    # latent rows of 288 + 32 (several pieces a lane) and of a size that fits no vector
    ("latent_attention", {"heads": 2, "dim": 24, "rot_dim": 32, "vdim": 40, "kv_rank": 288,
                          "scale": 0.05, "rot": {"base": 500.0, "dims": 32}}),
    ("latent_attention", {"heads": 5, "dim": 8, "rot_dim": 6, "vdim": 12, "kv_rank": 21,
                          "scale": 0.4, "rot": {"base": 10000.0, "dims": 6}}),
    # sizes of the tensor-core forms (bfloat16): expanded prompts with keys of 64 + 32 and
    # values of 64; latent rows of 128 + 16 and 256 + 32 on the heads-as-rows kernel
    ("latent_attention", {"heads": 3, "dim": 64, "rot_dim": 32, "vdim": 64, "kv_rank": 48,
                          "scale": 0.1, "rot": {"base": 10000.0, "dims": 32}}),
    ("latent_attention", {"heads": 5, "dim": 16, "rot_dim": 16, "vdim": 24, "kv_rank": 128,
                          "scale": 0.1, "rot": {"base": 10000.0, "dims": 16}}),
    ("latent_attention", {"heads": 3, "dim": 64, "rot_dim": 32, "vdim": 64, "kv_rank": 256,
                          "scale": 0.07, "rot": {"base": 10000.0, "dims": 32}}),
]


@pytest.mark.parametrize("dtype", DTYPES)
def test_mixers_at_other_sizes(dtype):
    from foundry_b200.cache import SequenceCache
    W, eps = 80, 1e-5
    torch.manual_seed(8)
    for n, (kind, m) in enumerate(MIXER_CASES):
        weights = tiny.random_mixer(kind, m, W, seed=n)
        part = mixer_part(kind, m, W, eps, weights, dtype)
        cache = SequenceCache({0: part.cache_request()}, 512, 2, dtype, DEV)
        x = torch.randn(90, W).to(dtype).float()
        want = plain_mixer(kind, m, double(weights), "a", x.double(), eps)
        for cuts in ([[90]], [[66, 2, 20, 1, 1]]):
            got = run_mixer(part, cache, [x], cuts, dtype)[0]
            assert rel_error(got, want) < bound(dtype), (kind, m, cuts)


ROUTERS = [
    {"experts": 6, "top": 2, "scale": 1.5, "groups": {"count": 3, "keep": 2}},
    {"experts": 4, "top": 3, "scale": 0.7, "groups": {"count": 4, "keep": 3}},   # groups of one
    {"experts": 5, "top": 1, "scale": 1.0},                                        # no groups
    {"experts": 64, "top": 6, "scale": 2.5, "groups": {"count": 8, "keep": 3}},  # two experts a lane
    {"experts": 12, "top": 12, "scale": 1.0, "groups": {"count": 2, "keep": 2}},  # everyone chosen
]


@pytest.mark.parametrize("router", ROUTERS)
def test_the_router_chooses_and_weighs_as_the_plain_one(router):
    """The routing kernel alone on float32 logits: corrections that push choice values
    below zero, groups ranked by their two best choice values, weights from the
    uncorrected scores as shares of their sum, times the constant."""
    from foundry_b200.kernels import ops
    E, top = router["experts"], router["top"]
    groups = router.get("groups") or {"count": 1, "keep": 1}
    gen = torch.Generator().manual_seed(E * 10 + top)
    z = 2.0 * torch.randn(300, E, generator=gen)
    correction = 0.8 * torch.randn(E, generator=gen) - 0.5
    chosen = torch.empty((300, top), dtype=torch.int32, device=DEV)
    weights = torch.empty((300, top), dtype=torch.float32, device=DEV)
    ops.moe_route(z.to(DEV), None, top, chosen, weights, "sigmoid", groups["count"], groups["keep"],
                  correction=correction.to(DEV), normalise=True, sum_floor=plain.WEIGHT_SUM_FLOOR,
                  weight_scale=router["scale"])
    want_chosen, want_weights = plain.route(router, z.double(), correction.double())
    assert (torch.sigmoid(z.double()) + correction.double()).min() < 0  # negative choice values occur
    assert chosen.cpu().tolist() == want_chosen.tolist()
    assert torch.allclose(weights.cpu().double(), want_weights, rtol=2e-6, atol=1e-7)


@pytest.mark.parametrize("router", ROUTERS)
def test_choice_and_sort_in_one_launch_equal_the_two_kernels(router):
    """For the few tokens of a single-token step the choice and the sort of the pairs by
    expert are one launch of one block: the same choice, weights and tables as the two
    kernels, at 1, 9 and 64 tokens (a warp takes several tokens in turn)."""
    from foundry_b200.kernels import ops
    E, top = router["experts"], router["top"]
    groups = router.get("groups") or {"count": 1, "keep": 1}
    gen = torch.Generator().manual_seed(E + top)
    correction = (0.8 * torch.randn(E, generator=gen) - 0.5).to(DEV)
    rule = dict(score="sigmoid", groups=groups["count"], keep=groups["keep"], correction=correction,
                normalise=True, sum_floor=plain.WEIGHT_SUM_FLOOR, weight_scale=router["scale"])
    for T in (1, 9, 64):
        assert T <= ops.MOE_ROUTE_SORT_ROWS
        z = (2.0 * torch.randn(T, E, generator=gen)).to(DEV)
        one = [torch.empty((T, top), dtype=torch.int32, device=DEV),
               torch.empty((T, top), dtype=torch.float32, device=DEV)]
        two = [torch.empty_like(one[0]), torch.empty_like(one[1])]
        fused = ops.moe_route_sorted(z, None, top, one[0], one[1], **rule)
        ops.moe_route(z, None, top, two[0], two[1], **rule)
        apart = ops.ExpertOrder(two[0], E)
        assert torch.equal(one[0], two[0]) and torch.equal(one[1], two[1])
        for field in ("counts", "starts", "place", "pair_at"):
            assert torch.equal(getattr(fused, field), getattr(apart, field)), (T, field)
        want_chosen, _ = plain.route(router, z.double().cpu(), correction.double().cpu())
        assert one[0].cpu().tolist() == want_chosen.tolist()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(tiny.CONFIGS))
def test_routed_experts_alone_and_beside_an_addend(name, dtype):
    """The feed-forward at 3, 37 and 200 rows (the forms for few rows and for many), alone
    and with rows of another part joining its sum. Tokens whose choice hangs on less than
    bfloat16 rounding are compared in float32 only."""
    from foundry_b200.parts import FEED_FORWARDS
    cfg, weights = tiny.CONFIGS[name], tiny.random_weights(name)
    spec, wd = spec_of(cfg), double(weights)
    W = cfg["width"]
    torch.manual_seed(6)
    for rows in (3, 37, 200):
        x = torch.randn(rows, W).to(dtype)
        addend = torch.randn(rows, W)
        for i, layer in enumerate(cfg["layers"]):
            if not layer["mlp"]:
                continue
            part = FEED_FORWARDS.build(spec.layers[i].feed_forward, dtype=dtype, device=DEV)
            part.load(f"l{i}.mlp", loader(weights, dtype))
            want = plain.routed_experts(layer["mlp"], wd, f"l{i}.mlp", x.double())
            clear = plain.router_margins(layer["mlp"], wd, f"l{i}.mlp", x.double()) > (
                0.0 if dtype == torch.float32 else 0.02)
            assert clear.sum() >= rows // 2
            got = part.forward(None, x.to(DEV)).float().cpu()
            assert rel_error(got[clear], want[clear]) < bound(dtype), (name, i, rows)
            both = part.forward(None, x.to(DEV), addend=addend.to(DEV)).float().cpu()
            assert rel_error(both[clear], (want + addend.double())[clear]) < bound(dtype), (name, i, rows)


@pytest.mark.parametrize("dtype", DTYPES)
def test_layer_norm_without_bias_and_the_scaled_sum(dtype):
    """resid += m * y and the layer norm of the sum (weight, no bias) in one pass; widths
    of whole 16-byte pieces and not."""
    from foundry_b200.kernels import ops
    from foundry_b200.parts import NORMS
    from foundry_b200.config.spec import PartSpec
    for W in (96, 50):
        norm = NORMS.build(PartSpec("layer_norm", {"size": W, "eps": 2e-5, "weight_suffix": "",
                                                   "bias_suffix": None}), dtype=dtype, device=DEV)
        gen = torch.Generator().manual_seed(W)
        w = (1.0 + 0.3 * torch.randn(W, generator=gen))
        assert set(norm.expected_tensors("n")) == {"n"}
        norm.load("n", lambda name: w.to(DEV))
        resid = (torch.randn(37, W, generator=gen) * 4 + 1).to(DEV)
        y = (torch.randn(37, W, generator=gen) * 2 - 3).to(DEV)
        total = resid.double().cpu() + 0.37 * y.double().cpu()
        out = norm.add_norm(resid, ops.ScaledDelta(y, 0.37))
        assert rel_error(resid.cpu(), total) < 1e-6
        assert rel_error(out.float().cpu(), plain.layer_norm(total, w.double(), 2e-5)) < bound(dtype, 0.3)
        first = norm.add_norm(resid, None)  # the first norm of a model has nothing to add
        assert rel_error(first.float().cpu(), plain.layer_norm(total, w.double(), 2e-5)) < bound(dtype, 0.3)


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_block_alone_with_and_without_experts(dtype):
    """One norm, both parts on its output, one sum times the constant: the stream after
    the block against the plain layer, for a layer with experts and one without."""
    from foundry_b200.cache import SequenceCache
    from foundry_b200.parts import BLOCKS
    cfg = dict(tiny.CONFIGS["mixed"])
    weights = tiny.random_weights("mixed")
    spec, wd = spec_of(cfg), double(weights)
    torch.manual_seed(9)
    for i in (0, 1, 2):
        layer = spec.layers[i]
        block = BLOCKS.build(layer.block, layer=layer, dtype=dtype, device=DEV)
        block.load(layer.prefix, loader(weights, dtype))
        cache = SequenceCache({0: block.cache_request()}, 256, 2, dtype, DEV)
        x = torch.randn(45, cfg["width"])
        want = plain.layer_update(cfg, wd, i, x.double(), torch.arange(45), {})
        slot = cache.open_sequence()
        ctx = make_ctx(cache, [slot], [45])
        ctx.shared = {}
        resid = x.to(DEV).clone()
        delta = block.forward(ctx, resid, None, cache.view(0, True))
        from foundry_b200.kernels import ops
        assert isinstance(delta, ops.ScaledDelta) and delta.scale == cfg["residual_mult"]
        got = resid.double().cpu() + delta.scale * delta.values.double().cpu()
        rows = torch.ones(45, dtype=torch.bool)
        if cfg["layers"][i]["mlp"] and dtype == torch.bfloat16:
            h = plain.layer_norm(x.double(), wd[f"l{i}.norm1"], cfg["norm"]["eps"])
            rows = plain.router_margins(cfg["layers"][i]["mlp"], wd, f"l{i}.mlp", h) > 0.05
        assert rel_error((got - x.double())[rows], (want - x.double())[rows]) < bound(dtype), i
        cache.close_sequence(slot)


# --------------------------------------------- one key that stands out, anywhere
def marked_inputs(query_at, marker_at, width, lift=3.0):
    """Rows in which the query of `query_at` (input 1) matches only the key of
    `marker_at` (input 2): that score stands far above the rest, so an output that
    sees the marker differs plainly from one that does not. The marker's value
    (inputs 4..8) is unlike every other."""
    gen = torch.Generator().manual_seed(query_at * 1000 + marker_at)
    x = torch.zeros(query_at + 1, width)
    x[:, 0] = 1.0
    x += 0.05 * torch.randn(x.shape, generator=gen)
    x[query_at] = 0.05 * torch.randn(width, generator=gen)
    x[query_at, 1] = 1.0
    x[marker_at] = 0.05 * torch.randn(width, generator=gen)
    x[marker_at, 2] = 1.0
    x[marker_at, 4:8] += lift
    return x.to(torch.bfloat16).float()


PLACES = [  # (query position, marker position): page borders, the first tokens, far back
    (5, 0), (63, 0), (64, 0), (64, 63), (65, 64), (127, 63), (128, 64), (129, 127), (200, 1),
    (700, 2), (700, 63), (700, 64), (700, 639), (700, 640), (700, 699),
]


def crafted_attention(W, d=8, e=8, heads=2):
    """Every head's query reads input 1 and its key input 2, both in an element that the
    rotation leaves alone (the last of the head); values are inputs 4..8."""
    m = {"heads": heads, "kv_heads": 1, "dim": d, "vdim": e, "scale": 24.0,
         "rot": {"base": 100.0, "dims": d - 2}}
    q, k = torch.zeros(heads * d, W), torch.zeros(d, W)
    for a in range(heads):
        q[a * d + d - 1, 1] = 1.0
    k[d - 1, 2] = 1.0
    val = torch.zeros(e, W)
    val[:4, 4:8] = torch.eye(4)
    out = torch.zeros(W, heads * e)
    out[:4, :4] = torch.eye(4)
    out[4:8, e:e + 4] = torch.eye(4)
    return m, {"a.q": q, "a.k": k, "a.v": val, "a.o": out, "a.sink": torch.tensor([1.0, 3.0][:heads])}


def crafted_latent(W, d=4, c=4, e=4, r=8):
    """The query reads input 1, the key input 2 of the cached latent, values the latent's
    elements 4..8; the rotated parts are idle in the scores (their query rows are zero)
    but are written and read all the same; the gate stands half open."""
    # (only 8 of the latent's r elements are fed: the norm over all r makes them
    # sqrt(r / 8) larger, which the scale takes back)
    m = {"heads": 1, "dim": d, "rot_dim": c, "vdim": e, "kv_rank": r,
         "scale": 5.0 * (8.0 / r) ** 0.5, "rot": {"base": 100.0, "dims": c}}
    q = torch.zeros(d + c, W)
    q[0, 1] = 5.0
    dkv = torch.zeros(r + c, W)
    dkv[:8, :8] = torch.eye(8)
    dkv[r:, 8:8 + c] = torch.eye(c)
    uk, uv = torch.zeros(d, r), torch.zeros(e, r)
    uk[0, 2] = 1.0
    uv[:4, 4:8] = torch.eye(4)
    out = torch.zeros(W, e)
    out[:4, :4] = torch.eye(4)
    return m, {"a.q": q, "a.dkv": dkv, "a.dkv.norm": torch.ones(r), "a.uk": uk, "a.uv": uv,
               "a.g": torch.zeros(e, W), "a.o": out}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("kind, sizes", [
    ("attention", "small"), ("attention", "tensor-core 64"), ("attention", "tensor-core 128"),
    ("latent_attention", "small"), ("latent_attention", "tensor-core"),
    ("latent_attention", "folded")])
def test_one_key_that_stands_out_is_found_wherever_it_lies(kind, sizes, dtype):
    """Crafted mixers in which one key dominates one query: at the first tokens, on both
    sides of page borders, hundreds of tokens back; as the last token of a prompt and
    as a token decoded alone. Once at sizes that only the CUDA-core kernels take, once at
    sizes whose bfloat16 steps run on the tensor cores."""
    from foundry_b200.cache import SequenceCache
    W = 32
    if kind == "attention":
        m, weights = {"small": crafted_attention(W), "tensor-core 64": crafted_attention(W, 64, 64),
                      "tensor-core 128": crafted_attention(W, 128, 128)}[sizes]
    elif sizes == "folded":  # latent rows of 128 + 16: every bfloat16 step on the heads-as-rows kernel
        m, weights = crafted_latent(W, 8, 16, 24, 128)
    else:
        m, weights = crafted_latent(W) if sizes == "small" else crafted_latent(W, 32, 16, 16)
    part = mixer_part(kind, m, W, 1e-6, weights, dtype)
    cache = SequenceCache({0: part.cache_request()}, 2048, 2, dtype, DEV)
    for query_at, marker_at in PLACES:
        x = marked_inputs(query_at, marker_at, W, lift=3.0 if kind == "attention" else 1.0)
        want = plain_mixer(kind, m, double(weights), "a", x.double(), 1e-6)[-1]
        # the plain implementation itself sees the marker: without it the output is another
        hidden = x.clone()
        hidden[marker_at] = hidden[max(0, marker_at - 1) if marker_at else 1]
        blind = plain_mixer(kind, m, double(weights), "a", hidden.double(), 1e-6)[-1]
        assert float((want - blind).norm() / want.norm()) > 0.2, (query_at, marker_at)
        for cut in ([query_at + 1], [query_at, 1]):
            got = run_mixer(part, cache, [x], [cut], dtype)[0][-1]
            assert rel_error(got[None], want[None]) < bound(dtype, 5.0), (query_at, marker_at, cut)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("size", [24, 64])
def test_a_sink_that_takes_most_of_the_sum(size, dtype):
    """Sink scores far above and far below the keys' scores, a head each: the output
    shrinks by the sink's share, in a prompt, for its first token, and for tokens decoded
    alone (where the visible keys are cut into runs and the sink joins once, at the merge)."""
    from foundry_b200.cache import SequenceCache
    m = {"heads": 4, "kv_heads": 2, "dim": size, "vdim": size, "scale": 0.2,
         "rot": {"base": 1000.0, "dims": size}}
    weights = tiny.random_mixer("attention", m, 96, seed=4)
    weights["a.sink"] = torch.tensor([6.0, -3.0, 2.5, 0.0])
    part = mixer_part("attention", m, 96, 1e-5, weights, dtype)
    cache = SequenceCache({0: part.cache_request()}, 1024, 2, dtype, DEV)
    torch.manual_seed(2)
    x = torch.randn(300, 96).to(dtype).float()
    want = plain_mixer("attention", m, double(weights), "a", x.double(), 1e-5)
    silent = dict(weights, **{"a.sink": torch.full((4,), -1e4)})
    assert rel_error(plain_mixer("attention", m, double(silent), "a", x.double(), 1e-5), want) > 0.3
    for cuts in ([[300]], [[1] + [1] * 8 + [280] + [1] * 11]):
        got = run_mixer(part, cache, [x], cuts, dtype)[0]
        assert rel_error(got, want) < bound(dtype), cuts


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_gate_that_closes_some_outputs(dtype):
    """Gate rows that shut some of the heads' outputs and open others wide."""
    from foundry_b200.cache import SequenceCache
    m = dict(tiny.CONFIGS["mixed"]["layers"][0]["mixer"])
    weights = tiny.random_mixer("latent_attention", m, 96, seed=6)
    weights["a.g"] = (weights["a.g"] * 6.0).to(torch.bfloat16).float()
    part = mixer_part("latent_attention", m, 96, 1e-5, weights, dtype)
    cache = SequenceCache({0: part.cache_request()}, 512, 2, dtype, DEV)
    torch.manual_seed(3)
    x = torch.randn(70, 96).to(dtype).float()
    want = plain_mixer("latent_attention", m, double(weights), "a", x.double(), 1e-5)
    for cuts in ([[70]], [[1, 2, 60] + [1] * 7]):
        got = run_mixer(part, cache, [x], cuts, dtype)[0]
        assert rel_error(got, want) < bound(dtype), cuts


# ---------------------------------------------------------------- whole models
@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("kutepel")
    return {name: tiny.write_folder(str(root / name), name) for name in tiny.CONFIGS}


def plain_logits(cfg, weights, tokens):
    return plain.forward(cfg, double(weights), tokens).numpy()


def clear_rows(cfg, weights, tokens, margin):
    """The positions none of whose layers' routers hangs on less than `margin`: a bfloat16
    run may choose another expert where two choice values lie closer than its rounding
    of the router's input, and such a row differs by an expert's output. (Later rows see
    it only as one key among many.)"""
    w = double(weights)
    _, streams = plain.forward(cfg, w, tokens, return_streams=True)
    x = w["embed"][torch.as_tensor(tokens)]
    ok = torch.ones(len(tokens), dtype=torch.bool)
    for i, layer in enumerate(cfg["layers"]):
        if layer["mlp"]:
            h = plain.layer_norm(x, w[f"l{i}.norm1"], cfg["norm"]["eps"])
            ok &= plain.router_margins(layer["mlp"], w, f"l{i}.mlp", h) > margin
        x = streams[i]
    return ok.numpy()


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
    cfg = tiny.CONFIGS[name]
    rng = np.random.default_rng(11)
    prompts = [[int(t) for t in rng.integers(0, cfg["vocab"], n)] for n in (150, 1, 3, 81)]
    want = [plain_logits(cfg, weights, p) for p in prompts]
    # float32: every row; bfloat16: the rows without a close call of a router
    rows = [np.ones(len(p), bool) if dtype == "float32" else clear_rows(cfg, weights, p, 0.05)
            for p in prompts]
    assert sum(int(r.sum()) for r in rows) > 60
    engine = fb.Engine.from_folder(folder, dtype=dtype, max_tokens=1024, max_slots=6)
    results = {}
    results["whole, alone"] = [run_cutting(engine, [p], [[len(p)]])[0] for p in prompts]
    results["token by token"] = [run_cutting(engine, [prompts[k]], [[1] * len(prompts[k])])[0]
                                 for k in (2, 3)]
    results["portions"] = run_cutting(engine, [prompts[0], prompts[3]],
                                      [[2, 62, 1, 64, 2, 17, 2], [77, 2, 2]])
    results["batch, then decoded together"] = run_cutting(
        engine, prompts, [[120] + [1] * 30, [1], [2, 1], [70] + [1] * 11])
    order = {"whole, alone": [0, 1, 2, 3], "token by token": [2, 3], "portions": [0, 3],
             "batch, then decoded together": [0, 1, 2, 3]}
    for cutting, got in results.items():
        for g, k in zip(got, order[cutting]):
            assert np.isfinite(g).all()
            if rows[k].any():
                assert rel_error(g[rows[k]], want[k][rows[k]]) < bound(
                    dtype, 2.0 if dtype == "float32" else 3.0), (name, dtype, cutting, k)
    if dtype == "float32":  # the cuttings agree with each other to rounding
        assert rel_error(results["portions"][0], results["whole, alone"][0]) < 2e-5
        assert rel_error(results["batch, then decoded together"][3], results["whole, alone"][3]) < 2e-5
    engine.cache.table.check()
    assert engine.free_slots() == 6


@pytest.mark.parametrize("name", list(tiny.CONFIGS))
def test_long_decoding_and_reused_slots(name, folders):
    """260 tokens decoded one by one behind a short prompt (across cache pages), twice on
    the same slot with another sequence between."""
    import foundry_b200 as fb
    folder, weights = folders[name]
    cfg = tiny.CONFIGS[name]
    rng = np.random.default_rng(12)
    tokens = [int(t) for t in rng.integers(0, cfg["vocab"], 265)]
    other = [int(t) for t in rng.integers(0, cfg["vocab"], 40)]
    want = plain_logits(cfg, weights, tokens)
    engine = fb.Engine.from_folder(folder, dtype="float32", max_tokens=512, max_slots=2)
    first = run_cutting(engine, [tokens], [[5] + [1] * 260])[0]
    run_cutting(engine, [other], [[40]])
    again = run_cutting(engine, [tokens], [[5] + [1] * 260])[0]
    assert rel_error(first, want) < bound("float32", 2.0)
    assert np.array_equal(first, again)


@pytest.mark.parametrize("width", [52, 100])
def test_sizes_that_fit_no_tensor_core_product(width, tmp_path):
    """Widths 52 and 100 (the latter long enough for a tensor-core K block, and no whole
    16-byte pieces) and inner sizes that are no multiples of 8: in bfloat16 every product
    takes the CUDA-core kernel and the experts the form that streams a token's own experts."""
    import foundry_b200 as fb
    doc = {"architecture": "Kutepel", "vocab": 77, "width": width, "norm": {"eps": 1e-5},
           "residual_mult": 0.25,
           "layers": [
               {"type": "attention",
                "mixer": {"heads": 3, "kv_heads": 3, "dim": 10, "vdim": 14, "scale": 0.3,
                          "rot": {"base": 777.0, "dims": 6}},
                "mlp": {"kind": "moe", "expert": {"ff": 44},
                        "router": {"experts": 3, "top": 2, "scale": 0.5}}},
               {"type": "latent_attention",
                "mixer": {"heads": 2, "dim": 10, "rot_dim": 6, "vdim": 14, "kv_rank": 18,
                          "scale": 0.25, "rot": {"base": 777.0, "dims": 6}}, "mlp": None},
               {"type": "attention",
                "mixer": {"heads": 6, "kv_heads": 3, "dim": 10, "vdim": 14, "scale": 0.2, "kv_from": 0,
                          "rot": {"base": 777.0, "dims": 6}},
                "mlp": {"kind": "moe", "expert": {"ff": 90},
                        "router": {"experts": 2, "top": 1, "scale": 1.0,
                                   "groups": {"count": 2, "keep": 1}}}}]}
    gen = torch.Generator().manual_seed(31)
    weights = {k: tiny.draw(k, shape, gen) for k, shape in tiny.tensor_shapes(doc).items()}
    folder, _ = tiny.write_folder(str(tmp_path / "odd"), None, doc=doc, weights=weights)
    rng = np.random.default_rng(3)
    prompts = [[int(t) for t in rng.integers(0, 77, n)] for n in (70, 9)]
    want = [plain_logits(doc, weights, p) for p in prompts]
    for dtype in ("float32", "bfloat16"):
        rows = [np.ones(len(p), bool) if dtype == "float32" else clear_rows(doc, weights, p, 0.05)
                for p in prompts]
        engine = fb.Engine.from_folder(folder, dtype=dtype, max_tokens=512, max_slots=3)
        got = run_cutting(engine, prompts, [[66, 2, 1, 1], [5, 1, 2, 1]])
        for g, w, r in zip(got, want, rows):
            assert r.sum() > len(r) // 4 and rel_error(g[r], w[r]) < bound(dtype, 3.0), dtype


def greedy(cfg, weights, prompt, count):
    tokens = list(prompt)
    for _ in range(count):
        tokens.append(int(plain.forward(cfg, weights, tokens)[-1].argmax()))
    return tokens[len(prompt):]


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
        w = greedy(cfg, wd, p, 8)
        if g == w:
            continue
        k = next(i for i, (a, b) in enumerate(zip(g, w)) if a != b)
        logits = plain.forward(cfg, wd, list(p) + w[:k])[-1]
        gap = float(logits[w[k]] - logits[g[k]])
        assert dtype == "bfloat16" and gap < 0.05 * float(logits.abs().max()), (g, w, gap)


def test_trace_replay_and_command_line(folders, tmp_path):
    """`bin/trace_run` on a Kutepel folder: a prompt step of two requests, then
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
    wa, wb = plain_logits(cfg, weights, a), plain_logits(cfg, weights, b)
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
    want = greedy(cfg, double(weights), a, 4)
    assert json.loads(run.stdout.strip().split("\n")[-1]) == want


def test_command_line_bench_on_a_kutepel_folder(folders, tmp_path):
    """`foundry bench` (prompt step, decode steps, report with bytes and operations) on a
    model whose layers share a cache entry and route every token."""
    folder, _ = folders["mixed"]
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "foundry"), "bench", "--model",
                           folder, "--prompt-tokens", "20", "--new-tokens", "5", "--runs", "2",
                           "--batch-size", "3", "--out", str(tmp_path)],
                          capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    report = json.loads((tmp_path / "report.json").read_text())
    assert len(report["runs"]) == 2 and all(len(r) == 5 for r in report["runs"][0]["token_ids"])
    assert report["runs"][0]["token_ids"] == report["runs"][1]["token_ids"]
