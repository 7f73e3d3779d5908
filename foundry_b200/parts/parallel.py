"""Two mixers side by side on the same input, as one mixer.

    y = left_scale * left(h) + right_scale * right(h)

Both read the same normalised input, so their input projections are ONE
product (the rows of the two weights stacked), and their output projections
are one product too: each side writes its inner rows, times its scale, into
its columns of one buffer, which meets the two output weights side by side,

    y = [left_scale * a_left | right_scale * a_right] [Wo_left | Wo_right]^T

(the scales multiply 32-bit values before they are rounded, not the weights).
A side is any mixer that offers `input_weight()`, `output_weight()`,
`inner_size` and `between(ctx, projections, cache_view, out, out_scale)`. The
cache entry of the run holds what each side asks for: pages, a state row, or
both (`JointRequest`). The sides' tensors lie under `<prefix>.<left name>` and
`<prefix>.<right name>`.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..cache.store import JointRequest, JointView, KVRequest, StateRequest
from ..config.spec import PartSpec
from ..weights.loader import ExpectedTensor
from .base import MIXERS, Fetch, Part, register_mixer
from .products import product_f32


@register_mixer("parallel")
class ParallelMixer(Part):
    replay_safe = True

    def __init__(self, left: PartSpec, right: PartSpec, left_scale: float = 1.0,
                 right_scale: float = 1.0, names=("left", "right"), *, dtype: torch.dtype,
                 device: torch.device):
        self.sides = [MIXERS.build(left, dtype=dtype, device=device),
                      MIXERS.build(right, dtype=dtype, device=device)]
        for side in self.sides:
            for need in ("input_weight", "output_weight", "between", "inner_size"):
                if not hasattr(side, need):
                    raise ValueError(f"{type(side).__name__} cannot stand beside another mixer: "
                                     f"it lacks `{need}`")
        self.scales = (float(left_scale), float(right_scale))
        self.names = tuple(names)
        self.replay_safe = all(getattr(s, "replay_safe", False) for s in self.sides)
        self.dtype, self.device = dtype, device
        self.w_in = self.w_out = None

    def expected_tensors(self, prefix: str) -> Dict[str, ExpectedTensor]:
        out: Dict[str, ExpectedTensor] = {}
        for side, name in zip(self.sides, self.names):
            out.update(side.expected_tensors(f"{prefix}.{name}"))
        return out

    def load(self, prefix: str, fetch: Fetch) -> None:
        for side, name in zip(self.sides, self.names):
            side.load(f"{prefix}.{name}", fetch)
        self.w_in = torch.cat([s.input_weight() for s in self.sides], 0).contiguous()
        self.w_out = torch.cat([s.output_weight() for s in self.sides], 1).contiguous()
        self.rows = [s.input_weight().shape[0] for s in self.sides]

    def cache_request(self):
        wants = [s.cache_request() for s in self.sides]
        kv = [w for w in wants if isinstance(w, KVRequest)]
        st = [w for w in wants if isinstance(w, StateRequest)]
        if len(kv) > 1 or len(st) > 1 or len(kv) + len(st) != sum(w is not None for w in wants):
            raise ValueError("the two sides of a parallel mixer ask for storage that one cache "
                             "entry cannot hold")
        if kv and st:
            return JointRequest(kv[0], st[0])
        return kv[0] if kv else st[0] if st else None

    def first_weight(self):
        return self.w_in

    def context_flops(self, token_counts, starts) -> float:
        return sum(s.context_flops(token_counts, starts) for s in self.sides
                   if hasattr(s, "context_flops"))

    def _view_for(self, side, cache):
        if not isinstance(cache, JointView):
            return cache
        return cache.kv if isinstance(side.cache_request(), KVRequest) else cache.state

    def forward(self, ctx, x, cache):
        T = x.shape[0]
        p = product_f32(x, self.w_in)
        inner = [s.inner_size for s in self.sides]
        both = torch.empty((T, sum(inner)), dtype=x.dtype, device=x.device)
        at_p = at_o = 0
        for side, rows, n, scale in zip(self.sides, self.rows, inner, self.scales):
            side.between(ctx, p[:, at_p:at_p + rows], self._view_for(side, cache),
                         both[:, at_o:at_o + n], scale)
            at_p += rows
            at_o += n
        return product_f32(both, self.w_out)
