"""Typed configuration of the Kutepel decoder, read from config.json.

A Kutepel model is a list of layers. Every layer has ONE norm (a layer norm with a
weight and no bias) whose output both of its parts read: a mixer (`attention`:
grouped heads with rotated queries and keys and a learnt sink per head, which may
read the keys and values of an earlier layer; `latent_attention`: attention through
a cached low-rank latent with one rotated key part for all heads and a sigmoid gate
on the heads' outputs) and routed experts (or no feed-forward). The two results join
the stream as one sum times a constant. Keys:

    architecture: "Kutepel", vocab, width, norm.eps, residual_mult,
    layers[i]: {type, mixer: {...}, mlp: null | {kind: "moe", expert: {ff},
                router: {experts, top, scale, groups: {count, keep}}}}
    attention:        heads, kv_heads, dim, vdim, scale, rot: {base, dims,
                      scaling: {factor, low, high, original}}, kv_from
    latent_attention: heads, dim, rot_dim, vdim, kv_rank, scale, rot: {base, dims}

Absent `rot.scaling`, `kv_from`, `router.groups` and `mlp` mean none.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, Mapping, Optional, Tuple

from . import errors
from .fields import need as _need, positive as _positive
from .files import decode_json

ARCHITECTURE = "Kutepel"
MIXER_TYPES = ("attention", "latent_attention")
# No key bounds the positions; 2^24 keeps every position exact in 32-bit floats.
MAX_POSITIONS = 1 << 24


@dataclass(frozen=True)
class RotScaling:
    factor: float
    low: float
    high: float
    original: float

    def to_json(self) -> dict:
        original = int(self.original) if float(self.original).is_integer() else self.original
        return {"factor": self.factor, "low": self.low, "high": self.high, "original": original}


@dataclass(frozen=True)
class KutepelExperts:
    ff: int
    experts: int
    top: int
    scale: float
    group_count: int = 1
    group_keep: int = 1
    has_groups: bool = True  # whether config.json spelt the groups out

    def to_json(self) -> dict:
        router: Dict[str, Any] = {"experts": self.experts, "top": self.top, "scale": self.scale}
        if self.has_groups:
            router["groups"] = {"count": self.group_count, "keep": self.group_keep}
        return {"kind": "moe", "expert": {"ff": self.ff}, "router": router}


@dataclass(frozen=True)
class KutepelLayer:
    type: str
    heads: int
    dim: int
    vdim: int
    scale: float
    rot_base: float
    rot_dims: int
    kv_heads: int = 0                       # attention
    rot_scaling: Optional[RotScaling] = None  # attention
    kv_from: Optional[int] = None           # attention: the layer whose keys and values it reads
    rot_dim: int = 0                        # latent_attention
    kv_rank: int = 0                        # latent_attention
    mlp: Optional[KutepelExperts] = None

    def to_json(self) -> dict:
        rot: Dict[str, Any] = {"base": self.rot_base, "dims": self.rot_dims}
        m: Dict[str, Any] = {"heads": self.heads, "dim": self.dim, "vdim": self.vdim,
                             "scale": self.scale, "rot": rot}
        if self.type == "attention":
            m["kv_heads"] = self.kv_heads
            if self.rot_scaling is not None:
                rot["scaling"] = self.rot_scaling.to_json()
            if self.kv_from is not None:
                m["kv_from"] = self.kv_from
        else:
            m.update(rot_dim=self.rot_dim, kv_rank=self.kv_rank)
        return {"type": self.type, "mixer": m,
                "mlp": None if self.mlp is None else self.mlp.to_json()}


@dataclass(frozen=True)
class KutepelConfig:
    vocab: int
    width: int
    norm_eps: float
    residual_mult: float
    layers: Tuple[KutepelLayer, ...]
    extra: Mapping[str, Any] = field(default_factory=dict, compare=False)

    @property
    def vocab_size(self) -> int:  # the name other parts of the library ask for
        return self.vocab

    @classmethod
    def parse(cls, source) -> "KutepelConfig":
        doc = decode_json(source)
        if doc.get("architecture") != ARCHITECTURE:
            raise errors.ModelType(f"architecture is {doc.get('architecture')!r}, "
                                   f"expected {ARCHITECTURE!r}")
        layers_doc = _need(doc, "layers", list, "config")
        if not layers_doc:
            raise errors.ConfigJson("config: no layers")
        known = {"architecture", "vocab", "width", "norm", "residual_mult", "layers"}
        layers = tuple(_parse_layer(e, f"layers[{i}]") for i, e in enumerate(layers_doc))
        for i, layer in enumerate(layers):
            _check_shared_keys(layers, i)
        return cls(
            vocab=_positive(doc, "vocab", "config"), width=_positive(doc, "width", "config"),
            norm_eps=_need(_need(doc, "norm", dict, "config"), "eps", float, "norm"),
            residual_mult=_need(doc, "residual_mult", float, "config"), layers=layers,
            extra={k: v for k, v in doc.items() if k not in known})

    def to_json(self) -> dict:
        return {"architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width,
                "norm": {"eps": self.norm_eps}, "residual_mult": self.residual_mult,
                "layers": [layer.to_json() for layer in self.layers]}


def _check_shared_keys(layers, i: int) -> None:
    """A layer that reads another's keys and values names an EARLIER attention layer
    that has projections of its own and the same head counts, sizes and rotation."""
    layer = layers[i]
    j = layer.kv_from
    if j is None:
        return
    where = f"layers[{i}].mixer.kv_from"
    if not 0 <= j < i:
        raise errors.ConfigJson(f"{where} = {j}: it must name an earlier layer")
    source = layers[j]
    if source.type != "attention" or source.kv_from is not None:
        raise errors.ConfigJson(f"{where} = {j}: layer {j} has no keys and values of its own")
    same = ("kv_heads", "dim", "vdim", "rot_base", "rot_dims", "rot_scaling")
    differs = [n for n in same if getattr(source, n) != getattr(layer, n)]
    if layer.heads % source.kv_heads or differs:
        raise errors.ConfigJson(f"{where} = {j}: the two layers differ in {differs or 'heads'}")


def _parse_rot(m, w: str, limit: int, what: str):
    rot = _need(m, "rot", dict, w)
    base = _need(rot, "base", float, f"{w}.rot")
    dims = _need(rot, "dims", int, f"{w}.rot")
    if dims < 0 or dims % 2 or dims > limit:
        raise errors.ConfigJson(f"{w}: rot.dims {dims} must be even and at most {what} {limit}")
    if base <= 0.0:
        raise errors.ConfigJson(f"{w}: rot.base {base} must be positive")
    scaling = None
    s = rot.get("scaling")
    if s is not None:
        if not isinstance(s, dict):
            raise errors.ConfigJson(f"{w}.rot.scaling is not an object")
        ws = f"{w}.rot.scaling"
        scaling = RotScaling(factor=_need(s, "factor", float, ws), low=_need(s, "low", float, ws),
                             high=_need(s, "high", float, ws),
                             original=_need(s, "original", float, ws))
        if scaling.factor <= 0 or scaling.low <= 0 or scaling.high <= 0 or scaling.original <= 0:
            raise errors.ConfigJson(f"{ws}: factor, low, high and original must be positive")
    return base, dims, scaling


def _parse_experts(mlp, where: str) -> KutepelExperts:
    if not isinstance(mlp, dict):
        raise errors.ConfigJson(f"{where} is not an object")
    kind = _need(mlp, "kind", str, where)
    if kind != "moe":
        raise errors.UnsupportedOption(f"{where}.kind {kind!r}; known: moe")
    router = _need(mlp, "router", dict, where)
    wr = f"{where}.router"
    groups = router.get("groups")
    count = keep = 1
    if groups is not None:
        if not isinstance(groups, dict):
            raise errors.ConfigJson(f"{wr}.groups is not an object")
        count, keep = _positive(groups, "count", f"{wr}.groups"), _positive(groups, "keep", f"{wr}.groups")
    out = KutepelExperts(ff=_positive(_need(mlp, "expert", dict, where), "ff", f"{where}.expert"),
                         experts=_positive(router, "experts", wr), top=_positive(router, "top", wr),
                         scale=_need(router, "scale", float, wr), group_count=count,
                         group_keep=keep, has_groups=groups is not None)
    if out.experts % count or keep > count or keep * (out.experts // count) < out.top:
        raise errors.ConfigJson(f"{wr}: {out.experts} experts in {count} groups, {keep} kept, "
                                f"{out.top} chosen")
    return out


def _parse_layer(entry, where: str) -> KutepelLayer:
    if not isinstance(entry, dict):
        raise errors.ConfigJson(f"{where} is not an object")
    kind = _need(entry, "type", str, where)
    if kind not in MIXER_TYPES:
        raise errors.UnsupportedOption(f"{where}: mixer type {kind!r}; known: {MIXER_TYPES}")
    m = _need(entry, "mixer", dict, where)
    w = f"{where}.mixer"
    fields: Dict[str, Any] = dict(type=kind, heads=_positive(m, "heads", w),
                                  dim=_positive(m, "dim", w), vdim=_positive(m, "vdim", w),
                                  scale=_need(m, "scale", float, w))
    if kind == "attention":
        fields["kv_heads"] = _positive(m, "kv_heads", w)
        if fields["heads"] % fields["kv_heads"]:
            raise errors.HeadRatio(f"{w}: {fields['heads']} heads over {fields['kv_heads']} kv heads")
        base, dims, scaling = _parse_rot(m, w, fields["dim"], "dim")
        fields.update(rot_base=base, rot_dims=dims, rot_scaling=scaling)
        if m.get("kv_from") is not None:
            fields["kv_from"] = _need(m, "kv_from", int, w)
    else:
        fields.update(rot_dim=_positive(m, "rot_dim", w), kv_rank=_positive(m, "kv_rank", w))
        base, dims, scaling = _parse_rot(m, w, fields["rot_dim"], "rot_dim")
        if scaling is not None:
            raise errors.UnsupportedOption(f"{w}.rot.scaling: the latent attention's rotation "
                                           f"has no frequency scaling")
        fields.update(rot_base=base, rot_dims=dims)
    if entry.get("mlp") is not None:
        fields["mlp"] = _parse_experts(entry["mlp"], f"{where}.mlp")
    return KutepelLayer(**fields)
