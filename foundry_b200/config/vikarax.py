"""Typed configuration of the Vikarax decoder, read from config.json.

A Vikarax model is a list of layers whose mixer is two mixers side by side on
the same input (`parallel`: an attention with sigmoid weights inside chunks on
the left, a Mamba-2 layer on the right, each side times a constant), a dense,
routed or absent feed-forward behind it, layer norms on both sides of every
part, a weighted sum over all earlier streams behind every layer, and a soft
cap on the logits. Keys:

    architecture: "Vikarax", vocab, width, norm.eps, logit_softcap,
    layers[i]: {type: "parallel",
                mixer: {left: {heads, kv_heads, dim, vdim, scale, mask: {size},
                               rot: {dims, base}},
                        right: {heads, vdim, state, groups, conv, norm_groups},
                        left_scale, right_scale},
                mlp: null | {kind: "dense", ff} |
                     {kind: "moe", expert: {ff}, router: {experts, top,
                      groups: {count, keep}}, shared: {ff}}}

A `mask` or `rot` that is absent means no chunks (every earlier key is
visible) or no rotation; absent `groups` mean one group; an absent `shared`
no shared expert; an absent `logit_softcap` no cap.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, Mapping, Optional, Tuple

from . import errors
from .fields import need as _need, positive as _positive
from .files import decode_json

ARCHITECTURE = "Vikarax"
MIXER_TYPES = ("parallel",)
# No key bounds the positions (angles are computed from the position in double
# precision); 2^24 keeps every position exactly representable in 32-bit floats.
MAX_POSITIONS = 1 << 24


@dataclass(frozen=True)
class VikaraxAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    chunk: Optional[int] = None      # mask.size
    rot_dims: int = 0                # rot.dims
    rot_base: float = 10000.0        # rot.base

    def to_json(self) -> dict:
        doc: Dict[str, Any] = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim,
                               "vdim": self.vdim, "scale": self.scale}
        if self.chunk is not None:
            doc["mask"] = {"size": self.chunk}
        if self.rot_dims:
            doc["rot"] = {"dims": self.rot_dims, "base": self.rot_base}
        return doc


@dataclass(frozen=True)
class VikaraxStateSpace:
    heads: int
    vdim: int
    state: int
    groups: int
    taps: int          # conv
    norm_groups: int

    def to_json(self) -> dict:
        return {"heads": self.heads, "vdim": self.vdim, "state": self.state, "groups": self.groups,
                "conv": self.taps, "norm_groups": self.norm_groups}


@dataclass(frozen=True)
class VikaraxMlp:
    kind: str  # "dense" | "moe"
    ff: int
    experts: int = 0
    top: int = 0
    group_count: int = 1
    group_keep: int = 1
    shared_ff: int = 0  # 0: no shared expert

    def to_json(self) -> dict:
        if self.kind == "dense":
            return {"kind": "dense", "ff": self.ff}
        doc: Dict[str, Any] = {"kind": "moe", "expert": {"ff": self.ff},
                               "router": {"experts": self.experts, "top": self.top,
                                          "groups": {"count": self.group_count,
                                                     "keep": self.group_keep}}}
        if self.shared_ff:
            doc["shared"] = {"ff": self.shared_ff}
        return doc


@dataclass(frozen=True)
class VikaraxLayer:
    type: str
    left: VikaraxAttention
    right: VikaraxStateSpace
    left_scale: float
    right_scale: float
    mlp: Optional[VikaraxMlp] = None

    def to_json(self) -> dict:
        return {"type": self.type,
                "mixer": {"left": self.left.to_json(), "right": self.right.to_json(),
                          "left_scale": self.left_scale, "right_scale": self.right_scale},
                "mlp": self.mlp.to_json() if self.mlp else None}


@dataclass(frozen=True)
class VikaraxConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[VikaraxLayer, ...]
    logit_softcap: Optional[float] = None
    extra: Mapping[str, Any] = field(default_factory=dict, compare=False)

    @property
    def vocab_size(self) -> int:  # the name other parts of the library ask for
        return self.vocab

    @classmethod
    def parse(cls, source) -> "VikaraxConfig":
        doc = decode_json(source)
        if doc.get("architecture") != ARCHITECTURE:
            raise errors.ModelType(f"architecture is {doc.get('architecture')!r}, "
                                   f"expected {ARCHITECTURE!r}")
        layers_doc = _need(doc, "layers", list, "config")
        if not layers_doc:
            raise errors.ConfigJson("config: no layers")
        cap = None
        if doc.get("logit_softcap") is not None:
            cap = _need(doc, "logit_softcap", float, "config")
            if cap <= 0:
                raise errors.ConfigJson(f"config: logit_softcap = {cap} must be positive")
        known = {"architecture", "vocab", "width", "norm", "layers", "logit_softcap"}
        return cls(
            vocab=_positive(doc, "vocab", "config"), width=_positive(doc, "width", "config"),
            norm_eps=_need(_need(doc, "norm", dict, "config"), "eps", float, "norm"),
            layers=tuple(_parse_layer(e, f"layers[{i}]") for i, e in enumerate(layers_doc)),
            logit_softcap=cap, extra={k: v for k, v in doc.items() if k not in known})

    def to_json(self) -> dict:
        doc = {"architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width,
               "norm": {"eps": self.norm_eps}, "layers": [l.to_json() for l in self.layers]}
        if self.logit_softcap is not None:
            doc["logit_softcap"] = self.logit_softcap
        return doc


def _optional(doc, key, where):
    value = doc.get(key)
    if value is not None and not isinstance(value, dict):
        raise errors.ConfigJson(f"{where}.{key} is not an object")
    return value


def _parse_attention(m, where: str) -> VikaraxAttention:
    heads, kv_heads = _positive(m, "heads", where), _positive(m, "kv_heads", where)
    if heads % kv_heads:
        raise errors.HeadRatio(f"{where}: {heads} heads over {kv_heads} kv heads")
    dim = _positive(m, "dim", where)
    fields: Dict[str, Any] = dict(heads=heads, kv_heads=kv_heads, dim=dim,
                                  vdim=_positive(m, "vdim", where),
                                  scale=_need(m, "scale", float, where))
    mask = _optional(m, "mask", where)
    if mask is not None and mask.get("size") is not None:
        fields["chunk"] = _positive(mask, "size", f"{where}.mask")
    rot = _optional(m, "rot", where)
    if rot is not None and rot.get("dims"):
        dims = _positive(rot, "dims", f"{where}.rot")
        if dims % 2 or dims > dim:
            raise errors.ConfigJson(f"{where}.rot: {dims} rotated elements in heads of {dim}")
        fields["rot_dims"] = dims
        fields["rot_base"] = _need(rot, "base", float, f"{where}.rot")
    return VikaraxAttention(**fields)


def _parse_state_space(m, where: str) -> VikaraxStateSpace:
    heads, groups = _positive(m, "heads", where), _positive(m, "groups", where)
    if heads % groups:
        raise errors.ConfigJson(f"{where}: {heads} heads over {groups} groups")
    vdim = _positive(m, "vdim", where)
    norm_groups = _positive(m, "norm_groups", where) if m.get("norm_groups") is not None else 1
    if (heads * vdim) % norm_groups:
        raise errors.ConfigJson(f"{where}: {heads * vdim} channels over {norm_groups} norm groups")
    return VikaraxStateSpace(heads=heads, vdim=vdim, state=_positive(m, "state", where),
                             groups=groups, taps=_positive(m, "conv", where),
                             norm_groups=norm_groups)


def _parse_mlp(mlp, where: str) -> Optional[VikaraxMlp]:
    if mlp is None:
        return None
    if not isinstance(mlp, dict):
        raise errors.ConfigJson(f"{where} is not an object")
    kind = _need(mlp, "kind", str, where)
    if kind == "dense":
        return VikaraxMlp("dense", _positive(mlp, "ff", where))
    if kind != "moe":
        raise errors.UnsupportedOption(f"{where}.kind {kind!r}; known: dense, moe")
    ex = _need(mlp, "expert", dict, where)
    ro = _need(mlp, "router", dict, where)
    experts, top = _positive(ro, "experts", f"{where}.router"), _positive(ro, "top", f"{where}.router")
    count = keep = 1
    groups = _optional(ro, "groups", f"{where}.router")
    if groups is not None:
        count = _positive(groups, "count", f"{where}.router.groups")
        keep = _positive(groups, "keep", f"{where}.router.groups")
    if experts % count or keep > count:
        raise errors.ConfigJson(f"{where}.router: {experts} experts in {count} groups, {keep} kept")
    if top > keep * (experts // count):
        raise errors.ConfigJson(f"{where}.router: {top} experts out of {keep} groups of "
                                f"{experts // count}")
    shared = _optional(mlp, "shared", where)
    return VikaraxMlp("moe", _positive(ex, "ff", f"{where}.expert"), experts, top, count, keep,
                      _positive(shared, "ff", f"{where}.shared") if shared is not None else 0)


def _parse_layer(entry, where: str) -> VikaraxLayer:
    if not isinstance(entry, dict):
        raise errors.ConfigJson(f"{where} is not an object")
    kind = _need(entry, "type", str, where)
    if kind not in MIXER_TYPES:
        raise errors.UnsupportedOption(f"{where}: mixer type {kind!r}; known: {MIXER_TYPES}")
    m = _need(entry, "mixer", dict, where)
    w = f"{where}.mixer"
    return VikaraxLayer(
        type=kind, left=_parse_attention(_need(m, "left", dict, w), f"{w}.left"),
        right=_parse_state_space(_need(m, "right", dict, w), f"{w}.right"),
        left_scale=_need(m, "left_scale", float, w) if m.get("left_scale") is not None else 1.0,
        right_scale=_need(m, "right_scale", float, w) if m.get("right_scale") is not None else 1.0,
        mlp=_parse_mlp(entry.get("mlp"), f"{where}.mlp"))
