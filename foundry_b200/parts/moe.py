"""A feed-forward of routed experts.

    z = W_router h (+ b)   (32-bit). Two scoring rules:
    "softmax_chosen": the `top` experts with the largest z are chosen (the lower index
        among equals) and weighted by the softmax over the chosen z only
    "sigmoid": s = sigmoid(z); the choice goes by c = s (+ a learnt correction per expert,
        `choice_correction`, which never enters a weight); the experts form `groups` equal
        groups of neighbours, a group's score is the sum of its two largest c, only experts
        of the `keep` best groups can be chosen; the `top` largest c are chosen and weighted
        by s itself or (`normalise`) by s / (the chosen experts' sum of s + `sum_floor`),
        times `weight_scale`
    expert:  g = min(W_gate h, limit);  u = clamp(W_up h, -limit, limit)
             y = W_down (g * sigmoid(alpha g) * (u + shift))
             (limit = infinity, alpha = 1, shift = 0:  W_down (silu(g) * u))
    out = sum over the chosen experts of weight * y  (+ shared(h), an expert of the plain
          SiLU form that every token uses, where `shared_ff` gives it a size)

The experts' tensors are `<prefix>.e<i>.gate|up|down`, the router's
`<prefix>.router`, (with `router_bias`) `<prefix>.router.b` and (with
`choice_correction`) `<prefix>.<correction_name>`, the shared
expert's `<prefix>.shared.gate|up|down`; the routed ones are stacked at load
time so that a kernel reaches any expert by index. Every constant is a parameter.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..kernels import ops
from ..weights.loader import ExpectedTensor
from .base import Fetch, Part, register_feed_forward
from .linear import matmul_nt
from .mlp import SwiGLU
from .products import product_f32


@register_feed_forward("routed_experts")
class RoutedExperts(Part):
    replay_safe = True
    accepts_addend = True  # forward(ctx, x, addend=rows): the rows join the experts' sum

    def __init__(self, width: int, ff: int, experts: int, top: int, limit: float = float("inf"),
                 alpha: float = 1.702, shift: float = 1.0, score: str = "softmax_chosen",
                 groups: int = 1, keep: int = 1, router_bias: bool = True, shared_ff: int = 0,
                 shared_name: str = "shared", choice_correction: bool = False,
                 correction_name: str = "correction", normalise: bool = False,
                 sum_floor: float = 0.0, weight_scale: float = 1.0, *, dtype: torch.dtype,
                 device: torch.device):
        if not 1 <= top <= min(experts, 32) or experts > 256:
            raise ValueError(f"{top} of {experts} experts: the router takes up to 256 experts and "
                             f"chooses up to 32")
        if score not in ops.MOE_SCORES:
            raise ValueError(f"scoring rule {score!r}; known: {sorted(ops.MOE_SCORES)}")
        if groups < 1 or experts % groups or not 1 <= keep <= groups or \
                keep * (experts // groups) < top or (groups > 1 and score != "sigmoid"):
            raise ValueError(f"{experts} experts in {groups} groups, {keep} kept, {top} chosen "
                             f"(groups need the sigmoid scores)")
        self.width, self.ff, self.experts, self.top = width, ff, experts, top
        self.limit, self.alpha, self.shift = float(limit), float(alpha), float(shift)
        self.score, self.groups, self.keep = score, int(groups), int(keep)
        self.has_router_bias = bool(router_bias)
        if (choice_correction or normalise or weight_scale != 1.0) and score != "sigmoid":
            raise ValueError("a correction of the choice, shares of the chosen scores' sum and "
                             "a constant on the weights need the sigmoid scores")
        self.has_correction, self.correction_name = bool(choice_correction), correction_name
        self.normalise, self.sum_floor = bool(normalise), float(sum_floor)
        self.weight_scale = float(weight_scale)
        self.correction = None
        self.dtype, self.device = dtype, device
        self.router_bias = None
        self.shared_name = shared_name
        self.shared = None
        if shared_ff:
            self.shared = SwiGLU(width, int(shared_ff), dtype=dtype, device=device,
                                 names=("gate", "up", "down"), suffix="", activation="silu")

    def expected_tensors(self, prefix: str) -> Dict[str, ExpectedTensor]:
        out = {f"{prefix}.router": ExpectedTensor((self.experts, self.width))}
        if self.has_router_bias:
            out[f"{prefix}.router.b"] = ExpectedTensor((self.experts,))
        if self.has_correction:
            out[f"{prefix}.{self.correction_name}"] = ExpectedTensor((self.experts,))
        if self.shared is not None:
            out.update(self.shared.expected_tensors(f"{prefix}.{self.shared_name}"))
        for e in range(self.experts):
            out[f"{prefix}.e{e}.gate"] = ExpectedTensor((self.ff, self.width))
            out[f"{prefix}.e{e}.up"] = ExpectedTensor((self.ff, self.width))
            out[f"{prefix}.e{e}.down"] = ExpectedTensor((self.width, self.ff))
        return out

    def load(self, prefix: str, fetch: Fetch) -> None:
        self.router = fetch(f"{prefix}.router").contiguous()
        if self.has_router_bias:
            self.router_bias = fetch(f"{prefix}.router.b").to(torch.float32).contiguous()
        if self.has_correction:
            self.correction = fetch(f"{prefix}.{self.correction_name}").to(
                torch.float32).contiguous()
        if self.shared is not None:
            self.shared.load(f"{prefix}.{self.shared_name}", fetch)
        # [E, 2 ff, W]: an expert's gate rows, then its up rows;  [E, W, ff]
        self.gate_up = torch.stack([torch.cat([fetch(f"{prefix}.e{e}.gate"),
                                               fetch(f"{prefix}.e{e}.up")], 0)
                                    for e in range(self.experts)], 0).contiguous()
        self.down = torch.stack([fetch(f"{prefix}.e{e}.down") for e in range(self.experts)],
                                0).contiguous()

    def first_weight(self):
        return self.router

    def forward(self, ctx, x, addend=None):
        """`addend` (float32 [T, width]): rows that join the sum where the chosen experts'
        rows are combined (the result of a part that ran beside this one)."""
        T = x.shape[0]
        z = product_f32(x, self.router)
        chosen = torch.empty((T, self.top), dtype=torch.int32, device=x.device)
        weights = torch.empty((T, self.top), dtype=torch.float32, device=x.device)
        rule = dict(score=self.score, groups=self.groups, keep=self.keep,
                    correction=self.correction, normalise=self.normalise,
                    sum_floor=self.sum_floor, weight_scale=self.weight_scale)
        grouped = ops.moe_grouped_fits(self.width) and ops.moe_grouped_fits(self.ff)
        if grouped:  # the choice, and the pairs sorted by expert
            order = ops.moe_route_sorted(z, self.router_bias, self.top, chosen, weights, **rule)
        else:
            ops.moe_route(z, self.router_bias, self.top, chosen, weights, **rule)
        # the shared expert's rows join the sum where the chosen experts' rows are combined
        shared = addend
        if self.shared is not None:
            shared = product_f32(self.shared.hidden(ops.plain(x)), self.shared.down.weight)
            if addend is not None:
                ops.add_into(shared, addend)
        out = torch.empty((T, self.width), dtype=torch.float32, device=x.device)
        if not grouped:
            # sizes the grouped kernels do not take: every token streams its own experts
            return ops.moe_experts_rows(x, self.gate_up, self.down, chosen, weights, out,
                                        self.limit, self.alpha, self.shift, addend=shared)
        if T >= self.LIBRARY_ROWS and ops.moe_grouped_tc_fits(x, self.width, self.ff):
            # many tokens: every expert's rows in one tcgen05 launch a product
            # (the activation is the first product's epilogue)
            act = ops.gemm_tc_grouped(ops.moe_gather(ops.plain(x), order), self.gate_up, order,
                                      glu=(self.limit, self.alpha, self.shift))
            y = ops.gemm_tc_grouped(act, self.down, order)
        elif T >= self.LIBRARY_ROWS and getattr(ctx, "cu_tokens_host", None) is not None:
            y = self._per_expert_products(ops.moe_gather(x, order), order)
        elif ops.moe_grouped_mma_fits(x, self.width, self.ff):
            act = ops.moe_grouped_mma(x, self.gate_up, order, True, self.limit, self.alpha,
                                      by_token=True, shift=self.shift)
            y = ops.moe_grouped_mma(act, self.down, order, False)
        else:
            act = ops.moe_grouped(x, self.gate_up, order, True, self.limit, self.alpha,
                                  by_token=True, shift=self.shift)
            y = ops.moe_grouped(act, self.down, order, False)
        return ops.moe_combine(y, order, weights, out, addend=shared)

    # From this many tokens on the experts' products run on the tcgen05 products: as one
    # grouped launch a product where the sizes allow it; else, in a step that is launched
    # plainly (its context has the host copies; such a step is never captured), expert by
    # expert through the dense products, which needs the experts' counts on the host.
    LIBRARY_ROWS = 128

    def _per_expert_products(self, rows, order):
        starts = order.starts.tolist()  # waits for the routing
        pairs, dev = order.pairs, rows.device
        gate_up = torch.empty((pairs, 2 * self.ff), dtype=torch.float32, device=dev)
        for e in range(self.experts):
            a, b = starts[e], starts[e + 1]
            if b > a:
                matmul_nt(rows[a:b], self.gate_up[e], gate_up[a:b])
        act = torch.empty((pairs, self.ff), dtype=rows.dtype, device=dev)
        ops.moe_glu(gate_up, act, order, self.limit, self.alpha, self.shift)
        y = torch.empty((pairs, self.width), dtype=torch.float32, device=dev)
        for e in range(self.experts):
            a, b = starts[e], starts[e + 1]
            if b > a:
                matmul_nt(act[a:b], self.down[e], y[a:b])
        return y
