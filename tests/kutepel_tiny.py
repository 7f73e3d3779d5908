"""Small Kutepel configurations for the tests, and random weights for them.

The two differ from each other in every size and constant: widths, head counts and
groupings (as many key heads as heads, one key head for all, a grouping of three), key
sizes beside other value sizes, heads rotated whole and in part, with and without
frequency bands, scales, latent and rotated sizes, layers that read the keys and
values of an earlier layer (the one before, and one further back, twice), layers
without feed-forward, routers with groups of several experts, groups of one expert and
no groups, one chosen expert and several, the residual constant (also 1).
"""
import json
import os

import torch

CONFIGS = {
    "mixed": {
        "architecture": "Kutepel", "vocab": 190, "width": 96, "norm": {"eps": 1e-5},
        "residual_mult": 0.6,
        "layers": [
            {"type": "latent_attention",
             "mixer": {"heads": 3, "dim": 16, "rot_dim": 8, "vdim": 24, "kv_rank": 40, "scale": 0.2,
                       "rot": {"base": 10000.0, "dims": 8}},
             "mlp": {"kind": "moe", "expert": {"ff": 48},
                     "router": {"experts": 6, "top": 2, "scale": 1.5,
                                "groups": {"count": 3, "keep": 2}}}},
            {"type": "attention",
             "mixer": {"heads": 6, "kv_heads": 2, "dim": 16, "vdim": 24, "scale": 0.3,
                       "rot": {"base": 100.0, "dims": 12,
                               "scaling": {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 64}}},
             "mlp": None},
            {"type": "attention",
             "mixer": {"heads": 4, "kv_heads": 4, "dim": 32, "vdim": 32, "scale": 0.15,
                       "rot": {"base": 10000.0, "dims": 32}},
             "mlp": {"kind": "moe", "expert": {"ff": 40},
                     "router": {"experts": 5, "top": 1, "scale": 1.0}}},
            {"type": "attention",
             "mixer": {"heads": 2, "kv_heads": 2, "dim": 16, "vdim": 24, "scale": 0.25, "kv_from": 1,
                       "rot": {"base": 100.0, "dims": 12,
                               "scaling": {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 64}}},
             "mlp": {"kind": "moe", "expert": {"ff": 24},
                     "router": {"experts": 4, "top": 3, "scale": 0.7,
                                "groups": {"count": 4, "keep": 3}}}},
            {"type": "attention",
             "mixer": {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 24, "scale": 0.2, "kv_from": 1,
                       "rot": {"base": 100.0, "dims": 12,
                               "scaling": {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 64}}},
             "mlp": None},
        ],
    },
    "other": {
        "architecture": "Kutepel", "vocab": 130, "width": 64, "norm": {"eps": 3e-6},
        "residual_mult": 1.0,
        "layers": [
            {"type": "attention",
             "mixer": {"heads": 3, "kv_heads": 1, "dim": 24, "vdim": 8, "scale": 0.2,
                       "rot": {"base": 500000.0, "dims": 24,
                               "scaling": {"factor": 16.0, "low": 2.0, "high": 8.0, "original": 256}}},
             "mlp": {"kind": "moe", "expert": {"ff": 32},
                     "router": {"experts": 8, "top": 4, "scale": 2.5,
                                "groups": {"count": 2, "keep": 2}}}},
            {"type": "attention",
             "mixer": {"heads": 3, "kv_heads": 1, "dim": 24, "vdim": 8, "scale": 0.35, "kv_from": 0,
                       "rot": {"base": 500000.0, "dims": 24,
                               "scaling": {"factor": 16.0, "low": 2.0, "high": 8.0, "original": 256}}},
             "mlp": {"kind": "moe", "expert": {"ff": 16},
                     "router": {"experts": 3, "top": 2, "scale": 1.0,
                                "groups": {"count": 1, "keep": 1}}}},
            {"type": "latent_attention",
             "mixer": {"heads": 1, "dim": 32, "rot_dim": 16, "vdim": 16, "kv_rank": 64, "scale": 0.15,
                       "rot": {"base": 500.0, "dims": 16}},
             "mlp": {"kind": "moe", "expert": {"ff": 56},
                     "router": {"experts": 9, "top": 2, "scale": 3.0,
                                "groups": {"count": 3, "keep": 1}}}},
        ],
    },
}


def mixer_shapes(kind, m, W):
    """Tensor shapes of one mixer by the names under its prefix."""
    H, d, e = m["heads"], m["dim"], m["vdim"]
    if kind == "attention":
        G = m["kv_heads"]
        shapes = {"q": (H * d, W), "sink": (H,), "o": (W, H * e)}
        if m.get("kv_from") is None:
            shapes.update({"k": (G * d, W), "v": (G * e, W)})
        return shapes
    r, c = m["kv_rank"], m["rot_dim"]
    return {"q": (H * (d + c), W), "dkv": (r + c, W), "dkv.norm": (r,), "uk": (H * d, r),
            "uv": (H * e, r), "g": (H * e, W), "o": (W, H * e)}


def experts_shapes(mlp, W):
    ff, E = mlp["expert"]["ff"], mlp["router"]["experts"]
    shapes = {"router": (E, W), "correction": (E,)}
    for i in range(E):
        shapes.update({f"e{i}.gate": (ff, W), f"e{i}.up": (ff, W), f"e{i}.down": (W, ff)})
    return shapes


def tensor_shapes(cfg):
    W, V = cfg["width"], cfg["vocab"]
    shapes = {"embed": (V, W), "final.norm": (W,)}
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}"
        shapes[f"{p}.norm1"] = (W,)
        for name, shape in mixer_shapes(layer["type"], layer["mixer"], W).items():
            shapes[f"{p}.mix.{name}"] = shape
        if layer["mlp"]:
            for name, shape in experts_shapes(layer["mlp"], W).items():
                shapes[f"{p}.mlp.{name}"] = shape
    return shapes


def draw(key, shape, gen):
    """One bfloat16-representable float32 tensor in a range that lets its mechanism
    matter: sinks that take a real share of the sum, corrections that change the choice
    (some negative enough to make choice values negative), norm weights around one."""
    leaf = key.split(".")[-1]
    r = torch.randn(shape, generator=gen)
    if leaf in ("norm", "norm1"):
        t = 1.0 + 0.2 * r
    elif leaf == "sink":
        t = 1.0 + r
    elif leaf == "correction":
        t = 0.6 * r - 0.3
    elif leaf == "router":
        t = r / (shape[-1] ** 0.5) * 4.0
    elif leaf == "embed":
        t = 0.5 * r
    else:
        t = r / (shape[-1] ** 0.5) * 1.5
    return t.to(torch.bfloat16).to(torch.float32)


def random_weights(name, seed=0):
    gen = torch.Generator().manual_seed(seed)
    return {key: draw(key, shape, gen) for key, shape in tensor_shapes(CONFIGS[name]).items()}


def random_mixer(kind, m, W, prefix="a", seed=0):
    gen = torch.Generator().manual_seed(seed)
    return {f"{prefix}.{n}": draw(f"{prefix}.{n}", s, gen) for n, s in mixer_shapes(kind, m, W).items()}


def random_experts(mlp, W, prefix="a", seed=0):
    gen = torch.Generator().manual_seed(seed)
    return {f"{prefix}.{n}": draw(f"{prefix}.{n}", s, gen) for n, s in experts_shapes(mlp, W).items()}


def write_folder(folder, name, seed=0, doc=None, weights=None):
    """A model folder as the loader reads it: config.json + model.safetensors (bfloat16)."""
    from foundry_b200.weights.safetensors_io import SINGLE_FILE, save_file
    os.makedirs(folder, exist_ok=True)
    weights = random_weights(name, seed) if weights is None else weights
    save_file({k: v.to(torch.bfloat16) for k, v in weights.items()},
              os.path.join(folder, SINGLE_FILE), metadata={"format": "pt"})
    with open(os.path.join(folder, "config.json"), "w") as handle:
        json.dump(CONFIGS[name] if doc is None else doc, handle)
    return folder, weights
