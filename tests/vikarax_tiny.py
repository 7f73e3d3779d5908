"""Small Vikarax configurations for the tests, and random weights for them.

The two differ from each other in every size: widths, head counts and
groupings on both sides (one key/value head a query head in one, several in
the other; one state group for all heads in one, a group a head in the other),
key, value and state sizes (also sizes that are no multiple of 8), chunks
(shorter than a cache page, longer than one), rotated elements (a part of the
head, all of it), taps, norm groups (one, several), the sides' constants (also
1), experts, how many are chosen (also one), expert groups (three of which two
are kept, one), a shared expert or none, a layer without feed-forward, the
order of dense and routed layers, and the cap on the logits.
"""
import torch

CONFIGS = {
    "mixed": {
        "architecture": "Vikarax", "vocab": 150, "width": 80, "norm": {"eps": 1e-5},
        "logit_softcap": 8.0,
        "layers": [
            {"type": "parallel",
             "mixer": {"left": {"heads": 6, "kv_heads": 2, "dim": 24, "vdim": 40, "scale": 0.3,
                                "mask": {"size": 10}, "rot": {"dims": 8, "base": 500.0}},
                       "right": {"heads": 4, "vdim": 20, "state": 12, "groups": 1, "conv": 3,
                                 "norm_groups": 1},
                       "left_scale": 0.7, "right_scale": 1.3},
             "mlp": {"kind": "moe", "expert": {"ff": 24},
                     "router": {"experts": 6, "top": 3, "groups": {"count": 3, "keep": 2}},
                     "shared": {"ff": 40}}},
            {"type": "parallel",
             "mixer": {"left": {"heads": 2, "kv_heads": 1, "dim": 16, "vdim": 8, "scale": 0.5,
                                "mask": {"size": 10}, "rot": {"dims": 8, "base": 500.0}},
                       "right": {"heads": 2, "vdim": 24, "state": 40, "groups": 2, "conv": 4,
                                 "norm_groups": 3},
                       "left_scale": 1.2, "right_scale": 0.5},
             "mlp": None},
            {"type": "parallel",
             "mixer": {"left": {"heads": 6, "kv_heads": 2, "dim": 24, "vdim": 40, "scale": 0.3,
                                "mask": {"size": 10}, "rot": {"dims": 8, "base": 500.0}},
                       "right": {"heads": 4, "vdim": 20, "state": 12, "groups": 1, "conv": 3,
                                 "norm_groups": 1},
                       "left_scale": 0.7, "right_scale": 1.3},
             "mlp": {"kind": "dense", "ff": 104}},
        ],
    },
    "other": {
        "architecture": "Vikarax", "vocab": 97, "width": 64, "norm": {"eps": 1e-6},
        "logit_softcap": 30.0,
        "layers": [
            {"type": "parallel",
             "mixer": {"left": {"heads": 2, "kv_heads": 2, "dim": 32, "vdim": 16, "scale": 0.2,
                                "mask": {"size": 100}, "rot": {"dims": 32, "base": 10000.0}},
                       "right": {"heads": 4, "vdim": 16, "state": 32, "groups": 4, "conv": 2,
                                 "norm_groups": 4},
                       "left_scale": 1.0, "right_scale": 1.0},
             "mlp": {"kind": "dense", "ff": 72}},
            {"type": "parallel",
             "mixer": {"left": {"heads": 2, "kv_heads": 2, "dim": 32, "vdim": 16, "scale": 0.2,
                                "mask": {"size": 100}, "rot": {"dims": 32, "base": 10000.0}},
                       "right": {"heads": 4, "vdim": 16, "state": 32, "groups": 4, "conv": 2,
                                 "norm_groups": 4},
                       "left_scale": 1.0, "right_scale": 1.0},
             "mlp": {"kind": "moe", "expert": {"ff": 64},
                     "router": {"experts": 4, "top": 1, "groups": {"count": 1, "keep": 1}}}},
        ],
    },
}


def mixer_shapes(p, m, W):
    """The tensors of one parallel mixer under the prefix `p` (config entry `m`)."""
    a, s = m["left"], m["right"]
    H, G, d, e = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
    shapes = {f"{p}.left.q": (H * d, W), f"{p}.left.k": (G * d, W),
              f"{p}.left.v": (G * e, W), f"{p}.left.q.norm": (d,),
              f"{p}.left.k.norm": (d,), f"{p}.left.pb": (H,),
              f"{p}.left.g": (H, W), f"{p}.left.o": (W, H * e)}
    inner, GN = s["heads"] * s["vdim"], s["groups"] * s["state"]
    shapes.update({f"{p}.right.in": (2 * inner + 2 * GN + s["heads"], W),
                   f"{p}.right.conv": (inner + 2 * GN, s["conv"]),
                   f"{p}.right.conv.b": (inner + 2 * GN,),
                   f"{p}.right.dt_bias": (s["heads"],), f"{p}.right.A_log": (s["heads"],),
                   f"{p}.right.D": (s["heads"],), f"{p}.right.norm": (inner,),
                   f"{p}.right.o": (W, inner)})
    return shapes


def mlp_shapes(p, mlp, W):
    if mlp["kind"] == "dense":
        return {f"{p}.up": (mlp["ff"], W), f"{p}.down": (W, mlp["ff"])}
    ff, E = mlp["expert"]["ff"], mlp["router"]["experts"]
    shapes = {f"{p}.router": (E, W)}
    names = [(f"e{x}", ff) for x in range(E)]
    if mlp.get("shared"):
        names.append(("shared", mlp["shared"]["ff"]))
    for name, size in names:
        shapes.update({f"{p}.{name}.gate": (size, W), f"{p}.{name}.up": (size, W),
                       f"{p}.{name}.down": (W, size)})
    return shapes


def tensor_shapes(cfg):
    W, V = cfg["width"], cfg["vocab"]
    shapes = {"embed": (V, W), "head": (V, W), "final.norm": (W,), "final.norm.b": (W,)}
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}"
        norms = ["norm1", "norm1b"] + (["norm2", "norm2b"] if layer["mlp"] else [])
        for n in norms:
            shapes[f"{p}.{n}"] = shapes[f"{p}.{n}.b"] = (W,)
        shapes[f"{p}.dwa"] = (i + 2,)
        shapes.update(mixer_shapes(f"{p}.mix", layer["mixer"], W))
        if layer["mlp"]:
            shapes.update(mlp_shapes(f"{p}.mlp", layer["mlp"], W))
    return shapes


def draw(key, shape, gen):
    """One bfloat16-representable float32 tensor. Matrices are wide enough that a
    wrong key, state or expert moves the logits; norm weights lie around one; step
    sizes and decays in ranges where a state lasts for a few dozen tokens; the
    streams' weights around one half, of either sign."""
    leaf = key.split(".")[-1]
    r = torch.randn(shape, generator=gen)
    if key.endswith(".b") and ("norm" in key or "conv" in key) or leaf in ("pb",):
        t = 0.3 * r
    elif leaf == "dt_bias":
        t = -1.0 + 0.5 * r
    elif leaf in ("norm", "norm1", "norm1b", "norm2", "norm2b") and len(shape) == 1:
        t = 1.0 + 0.2 * r
    elif leaf == "A_log":
        t = -1.0 + 0.5 * r
    elif leaf == "D":
        t = 1.0 + 0.3 * r
    elif leaf == "conv":
        t = 0.5 * r
    elif leaf == "dwa":
        t = 0.5 + 0.4 * r
    elif leaf == "embed":
        t = 0.5 * r
    else:
        t = r / (shape[-1] ** 0.5) * 1.5
    return t.to(torch.bfloat16).to(torch.float32)


def random_weights(name, seed=0):
    """Every tensor of the configuration `name`, by file name."""
    gen = torch.Generator().manual_seed(seed)
    return {key: draw(key, shape, gen) for key, shape in tensor_shapes(CONFIGS[name]).items()}


def random_tensors(shapes, seed=0):
    gen = torch.Generator().manual_seed(seed)
    return {key: draw(key, shape, gen) for key, shape in shapes.items()}


def write_folder(folder, name, seed=0):
    """A model folder as the loader reads it: config.json + model.safetensors (bfloat16)."""
    import json
    import os
    from foundry_b200.weights.safetensors_io import SINGLE_FILE, save_file
    os.makedirs(folder, exist_ok=True)
    weights = random_weights(name, seed)
    save_file({k: v.to(torch.bfloat16) for k, v in weights.items()},
              os.path.join(folder, SINGLE_FILE), metadata={"format": "pt"})
    with open(os.path.join(folder, "config.json"), "w") as handle:
        json.dump(CONFIGS[name], handle)
    return folder, weights
