"""The Kutepel decoder as data: config.json -> `ModelSpec`.

A plain table lookup as embedding; layers in the order the configuration lists them,
each `h = norm1(x); x <- x + m * (mixer(h) + ff(h))` with a layer norm that has a
weight and no bias and one constant m for the whole model (`parallel_residual`); two
mixers (`rotary_sink_attention`, `latent_attention` with direct queries, no sink and
an output gate); routed experts with sigmoid scores, a correction of the choice,
groups, shares of the chosen scores' sum and a constant on the weights; a final layer
norm and the embedding table as the output head. A layer that names another's keys and
values runs on that layer's cache entry without writing it. Tensor names: `embed`,
`final.norm`, `l<i>.norm1`, `l<i>.mix.*`, `l<i>.mlp.{router,correction,e<j>.{gate,up,down}}`.
"""
from __future__ import annotations

from ..config.kutepel import ARCHITECTURE, MAX_POSITIONS, KutepelConfig, KutepelLayer
from ..config.registry import Architecture, register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from ..parts.rope import banded_frequencies

NAMES = {"mixer": "mix", "feed_forward": "mlp", "mixer_norm": "norm1"}
WEIGHT_SUM_FLOOR = 1e-20  # joins the sum of the chosen experts' scores under the division


def _mixer(config: KutepelConfig, layer: KutepelLayer) -> PartSpec:
    if layer.type == "attention":
        s = layer.rot_scaling
        scaling = {} if s is None else {"factor": s.factor, "low": s.low, "high": s.high,
                                        "original": s.original}
        freq = banded_frequencies(layer.rot_dims, layer.rot_base, **scaling)
        return PartSpec("rotary_sink_attention", {
            "width": config.width, "heads": layer.heads, "kv_heads": layer.kv_heads,
            "dim": layer.dim, "vdim": layer.vdim, "scale": layer.scale,
            "frequencies": tuple(float(f) for f in freq), "pairing": "interleaved",
            "sink": True, "own_kv": layer.kv_from is None})
    return PartSpec("latent_attention", {
        "width": config.width, "heads": layer.heads, "dim": layer.dim, "rot_dim": layer.rot_dim,
        "vdim": layer.vdim, "kv_rank": layer.kv_rank, "q_rank": 0, "scale": layer.scale,
        "eps": config.norm_eps, "rot_base": layer.rot_base, "rot_dims": layer.rot_dims,
        "sink": False, "output_gate": True})


def _feed_forward(config: KutepelConfig, layer: KutepelLayer):
    mlp = layer.mlp
    if mlp is None:
        return None
    return PartSpec("routed_experts", {
        "width": config.width, "ff": mlp.ff, "experts": mlp.experts, "top": mlp.top,
        "limit": float("inf"), "alpha": 1.0, "shift": 0.0, "score": "sigmoid",
        "groups": mlp.group_count, "keep": mlp.group_keep, "router_bias": False,
        "choice_correction": True, "correction_name": "correction", "normalise": True,
        "sum_floor": WEIGHT_SUM_FLOOR, "weight_scale": mlp.scale})


def build_kutepel_spec(config: KutepelConfig) -> ModelSpec:
    norm = PartSpec("layer_norm", {"size": config.width, "eps": config.norm_eps,
                                   "weight_suffix": "", "bias_suffix": None})
    block = PartSpec("parallel_residual", {"residual_scale": config.residual_mult})
    layers, schedule = [], []
    for i, layer in enumerate(config.layers):
        layers.append(LayerSpec(prefix=f"l{i}", block=block, mixer=_mixer(config, layer),
                                feed_forward=_feed_forward(config, layer), mixer_norm=norm,
                                feed_forward_norm=None, names=NAMES))
        source = layer.kv_from
        schedule.append(ScheduleEntry(layer=i, cache=i) if source is None else
                        ScheduleEntry(layer=i, cache=source, writes_cache=False))
    spec = ModelSpec(
        architecture=ARCHITECTURE, hidden_size=config.width, vocab_size=config.vocab,
        max_positions=MAX_POSITIONS, layers=tuple(layers), schedule=tuple(schedule),
        final_norm=norm, embedding_name="embed", final_norm_prefix="final.norm",
        output_head_name=None)
    spec.validate()
    return spec


KUTEPEL = register_architecture(Architecture(
    name=ARCHITECTURE, model_type="kutepel", parse_config=KutepelConfig.parse,
    build_spec=build_kutepel_spec), replace=True)
