"""The Vikarax decoder as data: config.json -> `ModelSpec`.

A plain table lookup as embedding; layers with a layer norm in front of and
behind each part (`sandwich_norm_residual`) whose results are kept, so that
what goes on from layer i is a weighted sum over the embedding's output and
the results of layers 0 .. i (`depth`, tensor `l<i>.dwa`); as mixer two mixers
side by side on the same input (`parallel`): an attention with sigmoid
weights inside chunks (`chunked_sigmoid_attention`) and a Mamba-2 layer
(`state_space_duality`), each times a constant; behind it a dense feed-forward
with the square of relu, routed experts (sigmoid scores, groups of experts, a
shared expert) or nothing; a final layer norm, a separate output head and a
soft cap on the logits. Tensor names: `embed`, `head`, `final.norm[.b]`,
`l<i>.{norm1,norm1b,norm2,norm2b}[.b]`, `l<i>.mix.left.*`, `l<i>.mix.right.*`,
`l<i>.mlp.*`, `l<i>.dwa`.
"""
from __future__ import annotations

from ..config.registry import Architecture, register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec, default_schedule
from ..config.vikarax import ARCHITECTURE, MAX_POSITIONS, VikaraxConfig, VikaraxLayer

NAMES = {"mixer": "mix", "feed_forward": "mlp", "mixer_norm": "norm1", "mixer_post_norm": "norm1b",
         "feed_forward_norm": "norm2", "feed_forward_post_norm": "norm2b"}


def _mixer(config: VikaraxConfig, layer: VikaraxLayer) -> PartSpec:
    a, s = layer.left, layer.right
    left = PartSpec("chunked_sigmoid_attention", {
        "width": config.width, "heads": a.heads, "kv_heads": a.kv_heads, "dim": a.dim,
        "vdim": a.vdim, "scale": a.scale, "eps": config.norm_eps, "chunk": a.chunk,
        "rotary": a.rot_dims, "rotary_base": a.rot_base, "value_norm": True,
        "output_gate": True, "head_bias": True})
    right = PartSpec("state_space_duality", {
        "width": config.width, "heads": s.heads, "vdim": s.vdim, "state": s.state,
        "groups": s.groups, "taps": s.taps, "eps": config.norm_eps,
        "norm_groups": s.norm_groups})
    return PartSpec("parallel", {"left": left, "right": right, "left_scale": layer.left_scale,
                                 "right_scale": layer.right_scale, "names": ("left", "right")})


def _feed_forward(config: VikaraxConfig, layer: VikaraxLayer):
    mlp = layer.mlp
    if mlp is None:
        return None
    if mlp.kind == "dense":
        return PartSpec("dense_mlp", {"hidden_size": config.width, "intermediate_size": mlp.ff,
                                      "names": ("up", "down"), "suffix": "",
                                      "activation": "relu2"})
    return PartSpec("routed_experts", {
        "width": config.width, "ff": mlp.ff, "experts": mlp.experts, "top": mlp.top,
        "limit": float("inf"), "alpha": 1.0, "shift": 0.0, "score": "sigmoid",
        "groups": mlp.group_count, "keep": mlp.group_keep, "router_bias": False,
        "shared_ff": mlp.shared_ff})


def build_vikarax_spec(config: VikaraxConfig) -> ModelSpec:
    norm = PartSpec("layer_norm", {"size": config.width, "eps": config.norm_eps,
                                   "weight_suffix": "", "bias_suffix": ".b"})
    total = len(config.layers)
    layers = []
    for i, layer in enumerate(config.layers):
        ff = _feed_forward(config, layer)
        layers.append(LayerSpec(
            prefix=f"l{i}",
            block=PartSpec("sandwich_norm_residual", {"depth": i + 1, "depth_total": total,
                                                      "depth_name": "dwa"}),
            mixer=_mixer(config, layer), feed_forward=ff, mixer_norm=norm,
            feed_forward_norm=norm if ff is not None else None, names=NAMES,
            mixer_post_norm=norm, feed_forward_post_norm=norm if ff is not None else None))
    spec = ModelSpec(
        architecture=ARCHITECTURE, hidden_size=config.width, vocab_size=config.vocab,
        max_positions=MAX_POSITIONS, layers=tuple(layers), schedule=default_schedule(total),
        final_norm=norm, embedding_name="embed", final_norm_prefix="final.norm",
        output_head_name="head", logit_softcap=config.logit_softcap,
        # a layer without a feed-forward has no use for the norms around one; a file
        # that carries them all the same is still this model
        ignorable_tensors=tuple(f"l{i}.norm2{tail}" for i, layer in enumerate(config.layers)
                                if layer.mlp is None for tail in ("", ".b", "b", "b.b")))
    spec.validate()
    return spec


VIKARAX = register_architecture(Architecture(
    name=ARCHITECTURE, model_type="vikarax", parse_config=VikaraxConfig.parse,
    build_spec=build_vikarax_spec), replace=True)
