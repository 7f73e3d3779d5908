"""Named configurations for measurements with random weights: the config.json
documents of the model sizes the benchmarks quote, so that `foundry bench
--config NAME --random-weights SEED` needs no model folder. These are data for
the command line and for bench.py; no part or kernel reads them."""
from __future__ import annotations

from typing import Dict


def _llama(layers, hidden, heads, kv_heads, head_dim, intermediate, vocab, factor, tied,
           theta=500000.0, eps=1e-5, original=8192, max_positions=131072) -> Dict:
    scaling = None if factor is None else {
        "rope_type": "llama3", "factor": float(factor), "low_freq_factor": 1.0,
        "high_freq_factor": 4.0, "original_max_position_embeddings": original}
    return {"architectures": ["LlamaForCausalLM"], "model_type": "llama",
            "num_hidden_layers": layers, "hidden_size": hidden, "num_attention_heads": heads,
            "num_key_value_heads": kv_heads, "head_dim": head_dim,
            "intermediate_size": intermediate, "vocab_size": vocab, "rms_norm_eps": eps,
            "rope_theta": theta, "rope_scaling": scaling, "tie_word_embeddings": tied,
            "max_position_embeddings": max_positions}


def _rupotar(layers, width, heads, kv_heads, dim, ff, vocab, window=1024, keep_first=4,
             experts=16, top=2, rank=64, taps=4, loop=None) -> Dict:
    """A Rupotar stack of real layer sizes: the three mixers in turn (attention,
    wkv, channel_delta), dense and routed feed-forwards alternating (an expert a
    quarter as wide as the dense one)."""
    stack = []
    for i in range(layers):
        kind = ("attention", "wkv", "channel_delta")[i % 3]
        if kind == "attention":
            mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim,
                     "scale": dim ** -0.5, "mask": {"size": window, "keep_first": keep_first}}
        elif kind == "wkv":
            mixer = {"heads": heads, "dim": dim, "decay_rank": rank}
        else:
            mixer = {"heads": heads, "kv_heads": heads, "dim": dim, "vdim": dim, "conv": taps,
                     "decay_rank": rank, "gate_rank": rank}
        mlp = {"kind": "dense", "ff": ff} if i % 2 == 0 else \
            {"kind": "moe", "expert": {"ff": ff // 4, "limit": 7.0},
             "router": {"experts": experts, "top": top}}
        stack.append({"type": kind, "mixer": mixer, "mlp": mlp})
    return {"architecture": "Rupotar", "vocab": vocab, "width": width,
            "embedding": {"scale": 1.0}, "norm": {"eps": 1e-5}, "layers": stack, "loop": loop}


def _vonulorn(layers, width, heads, kv_heads, dim, ff, vocab, kv_rank, q_rank, taps=4) -> Dict:
    """A Vonulorn stack of real layer sizes: the three mixers in turn (delta,
    differential attention, latent attention), every layer with a dense
    feed-forward. The differential attention has half the heads with two maps of
    at most 64 each and values twice that, so its scores and sums cost what `heads` plain
    heads of `dim` cost; the latent attention rotates half a head's size beside it."""
    stack = []
    for i in range(layers):
        kind = ("delta", "attention", "latent_attention")[i % 3]
        if kind == "delta":
            mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "conv": taps}
        elif kind == "attention":
            each = min(dim, 64)  # a map's key size; as many heads as keep the projections' sizes
            mixer = {"heads": heads * dim // (2 * each), "kv_heads": max(1, kv_heads * dim // (2 * each)),
                     "dim": each, "vdim": 2 * each, "scale": each ** -0.5, "softcap": 50.0,
                     "diff": 0.8, "q_temp": {"coef": 0.2, "every": 128}}
        else:
            mixer = {"heads": heads, "dim": dim, "rot_dim": dim // 2, "vdim": dim,
                     "kv_rank": kv_rank, "q_rank": q_rank, "scale": (dim + dim // 2) ** -0.5,
                     "rot": {"base": 10000.0, "dims": dim // 2}}
        stack.append({"type": kind, "mixer": mixer, "mlp": {"kind": "dense", "ff": ff}})
    return {"architecture": "Vonulorn", "vocab": vocab, "width": width, "norm": {"eps": 1e-5},
            "residual_mult": 0.7, "layers": stack}


def _vikarax(layers, width, heads, kv_heads, dim, ff, vocab, chunk=1024, state=128, taps=4,
             experts=16, top=2) -> Dict:
    """A Vikarax stack of real layer sizes: every layer the two mixers side by side
    (sigmoid attention inside chunks of `chunk` positions with half of each head
    rotated; a Mamba-2 layer of as many heads of the same size, eight groups of
    `state` rows), dense and routed feed-forwards alternating (an expert and the
    shared expert a quarter as wide as the dense one, four groups of experts of
    which two are kept)."""
    stack = []
    for i in range(layers):
        mixer = {"left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim,
                          "scale": dim ** -0.5, "mask": {"size": chunk},
                          "rot": {"dims": dim // 2, "base": 10000.0}},
                 "right": {"heads": heads, "vdim": dim, "state": state, "groups": kv_heads,
                           "conv": taps, "norm_groups": kv_heads},
                 "left_scale": 0.5, "right_scale": 0.5}
        mlp = {"kind": "dense", "ff": ff} if i % 2 == 0 else \
            {"kind": "moe", "expert": {"ff": ff // 4},
             "router": {"experts": experts, "top": top, "groups": {"count": 4, "keep": 2}},
             "shared": {"ff": ff // 4}}
        stack.append({"type": "parallel", "mixer": mixer, "mlp": mlp})
    return {"architecture": "Vikarax", "vocab": vocab, "width": width, "norm": {"eps": 1e-5},
            "logit_softcap": 30.0, "layers": stack}


def _kutepel(layers, width, heads, kv_heads, dim, ff, vocab, kv_rank, experts=16, top=2) -> Dict:
    """A Kutepel stack of real layer sizes: grouped attention with a sink and latent
    attention in turn, every third layer of the first kind reading the keys and values
    of the one before it; every layer with routed experts a quarter as wide as the dense
    feed-forward of the size (four groups of experts of which two are kept). The grouped
    heads are rotated whole, in the frequency bands of an eightfold stretch of 8,192
    positions; the latent attention rotates half a head's size beside it."""
    stack = []
    owners = []  # attention layers with keys and values of their own
    for i in range(layers):
        if i % 2 == 0:
            mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim,
                     "scale": dim ** -0.5,
                     "rot": {"base": 500000.0, "dims": dim,
                             "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}}
            if i % 6 == 4 and owners:
                mixer["kv_from"] = owners[-1]
            else:
                owners.append(i)
            kind = "attention"
        else:
            mixer = {"heads": heads, "dim": dim, "rot_dim": dim // 2, "vdim": dim,
                     "kv_rank": kv_rank, "scale": (dim + dim // 2) ** -0.5,
                     "rot": {"base": 10000.0, "dims": dim // 2}}
            kind = "latent_attention"
        mlp = {"kind": "moe", "expert": {"ff": ff // 4},
               "router": {"experts": experts, "top": top, "scale": 2.5,
                          "groups": {"count": 4, "keep": 2}}}
        stack.append({"type": kind, "mixer": mixer, "mlp": mlp})
    return {"architecture": "Kutepel", "vocab": vocab, "width": width, "norm": {"eps": 1e-5},
            "residual_mult": 0.7, "layers": stack}


PRESETS: Dict[str, Dict] = {
    "kutepel-1b-layers": _kutepel(6, 2048, 32, 8, 64, 8192, 32000, 256),
    "kutepel-3b-layers": _kutepel(6, 3072, 24, 8, 128, 8192, 32000, 512),
    "vikarax-1b-layers": _vikarax(6, 2048, 32, 8, 64, 8192, 32000),
    "vikarax-3b-layers": _vikarax(6, 3072, 24, 8, 128, 8192, 32000),
    "vonulorn-1b-layers": _vonulorn(6, 2048, 32, 8, 64, 8192, 32000, 256, 768),
    "vonulorn-3b-layers": _vonulorn(6, 3072, 24, 8, 128, 8192, 32000, 512, 1536),
    # six layers of the 1B and 3B layer sizes, as Rupotar and as Llama, for side-by-side timing
    "rupotar-1b-layers": _rupotar(6, 2048, 32, 8, 64, 8192, 32000),
    "rupotar-3b-layers": _rupotar(6, 3072, 24, 8, 128, 8192, 32000),
    "llama-1b-layers": _llama(6, 2048, 32, 8, 64, 8192, 32000, None, False),
    "llama-3b-layers": _llama(6, 3072, 24, 8, 128, 8192, 32000, None, False),
    "llama-3.2-1b": _llama(16, 2048, 32, 8, 64, 8192, 128256, 32.0, True),
    "llama-3.2-3b": _llama(28, 3072, 24, 8, 128, 8192, 128256, 32.0, True),
    "llama-3.1-8b": _llama(32, 4096, 32, 8, 128, 14336, 128256, 8.0, False),
    "tiny-a": _llama(2, 64, 4, 2, 16, 176, 256, None, True, theta=10000.0, max_positions=128),
    "tiny-b": _llama(3, 96, 6, 3, 32, 256, 384, 8.0, False, eps=1e-6, original=64,
                     max_positions=256),
}


def preset(name: str) -> Dict:
    try:
        return dict(PRESETS[name])
    except KeyError:
        raise ValueError(f"no configuration named {name!r}; known: {sorted(PRESETS)}") from None
