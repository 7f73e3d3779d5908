"""Mixers that carry a matrix state per head from token to token.

`gated_delta_channel`: the gated delta rule with a decay per key channel.

    q = Wq h, k = Wk h  (kv_heads x dim),  v = Wv h  (heads x vdim); head a uses q/k head
    a // (heads / kv_heads). Each passes a causal convolution over time per channel
    (`taps` weights a channel, the newest input under the last weight, nothing but zeros in
    front of a sequence's first token) and SiLU;
    q and k become unit vectors per head, x / sqrt(sum x^2 + 1e-6), q also times dim^-1/2.
    beta = sigmoid(Wb h) per head;  g = exp(-exp(A_log[a]) softplus(Wa2 (Wa1 h) + dt_bias))
    per head and key channel.
    S <- diag(g) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
    out = Wo [ o / rms(o) * norm * sigmoid(Wg2 (Wg1 h)) ]   (norm [vdim], shared by heads)

`gated_delta`: the same rule with ONE decay per head and full-rank gates.

    q, k, v, convolutions, SiLU and unit vectors as above;  beta = sigmoid(Wb h);
    g = exp(-exp(A_log[a]) softplus(Wa h + dt_bias))  one number per head (Wa [heads, W]);
    S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
    out = Wo [ o / rms(o) * norm * silu(Wg h) ]      (Wg [heads * vdim, W])

`wkv_time_mix`: RWKV-style time mixing.

    with h' the previous token's h (zeros at the start): m_s = h + (h' - h) mu_s for
    s in r, k, v, g, w;  r = Wr m_r, k = Wk m_k, v = Wv m_v (heads x dim);
    gate = silu(Wg m_g);  w = exp(-exp(Ww2 tanh(Ww1 m_w) + w0)) per head and key channel
    o = (S + diag(u) k v^T)^T r;  S <- diag(w) S + k v^T
    out = Wo [ o / rms(o per head) * norm * gate ]          (norm [heads * dim])

`state_space_duality`: the Mamba-2 layer.

    W_in h = [z: inner | x: inner | B: groups x state | C: groups x state | dt: heads],
    inner = heads x vdim;  x, B, C together pass a causal convolution per channel (`taps`
    weights and a bias, the newest input under the last weight, zeros in front of the
    sequence) and SiLU;  dt <- softplus(dt + dt_bias), no clamp;  per head a (group
    a // (heads / groups)):
    S <- exp(-exp(A_log[a]) dt) S + dt B x^T   (S [state, vdim]);  y = S^T C + D[a] x
    out = Wo [ rms_parts(y * silu(z)) * norm ]   (the gate first; the row normalised in
    `norm_groups` equal parts, each by its own root mean square)

The state S is float32 and, with the inputs that the next step needs from this
one (the convolution's last taps - 1 inputs; the last h), one float32 row per
sequence in the cache's state storage. Decays, step sizes, gates, unit norms
and the recurrence itself are 32-bit; the projections run in the element type
of the run with 32-bit sums and hand their results over unrounded.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..cache.store import StateRequest, StateView
from ..kernels import ops
from ..weights.loader import ExpectedTensor
from .base import Fetch, Part, register_mixer
from .products import product_f32, product_to_residual


def _f32(t: torch.Tensor) -> torch.Tensor:
    return t.to(torch.float32).contiguous()


@register_mixer("gated_delta_channel")
class GatedDeltaChannel(Part):
    replay_safe = True

    def __init__(self, width: int, heads: int, kv_heads: int, dim: int, vdim: int, taps: int,
                 eps: float, decay_rank: int, gate_rank: int, unit_eps: float = 1e-6, *,
                 dtype: torch.dtype, device: torch.device):
        if kv_heads <= 0 or heads % kv_heads:
            raise ValueError(f"{heads} heads are not a multiple of {kv_heads} key heads")
        if dim > 512:
            raise ValueError(f"{dim} key channels a head: the recurrence kernel holds at most 512")
        self.width, self.heads, self.kv_heads, self.dim, self.vdim = width, heads, kv_heads, dim, vdim
        self.taps, self.eps, self.unit_eps = int(taps), float(eps), float(unit_eps)
        self.decay_rank, self.gate_rank = decay_rank, gate_rank
        self.dtype, self.device = dtype, device
        self.channels = 2 * kv_heads * dim + heads * vdim
        self.fields = [("tail", (self.taps - 1) * self.channels), ("S", heads * dim * vdim)]

    def _shapes(self):
        W, H, G, d, v = self.width, self.heads, self.kv_heads, self.dim, self.vdim
        return {"q": (G * d, W), "q.conv": (G * d, self.taps), "k": (G * d, W),
                "k.conv": (G * d, self.taps), "v": (H * v, W), "v.conv": (H * v, self.taps),
                "b": (H, W), "A_log": (H,), "norm": (v,), "a1": (self.decay_rank, W),
                "a2": (H * d, self.decay_rank), "dt_bias": (H * d,), "g1": (self.gate_rank, W),
                "g2": (H * v, self.gate_rank), "o": (W, H * v)}

    def expected_tensors(self, prefix: str) -> Dict[str, ExpectedTensor]:
        return {f"{prefix}.{n}": ExpectedTensor(s) for n, s in self._shapes().items()}

    def load(self, prefix: str, fetch: Fetch) -> None:
        f = lambda n: fetch(f"{prefix}.{n}")
        # every projection of h in one product: q | k | v | beta | decay low rank | gate low rank
        self.w_in = torch.cat([f("q"), f("k"), f("v"), f("b"), f("a1"), f("g1")], 0).contiguous()
        self.conv = _f32(torch.cat([f("q.conv"), f("k.conv"), f("v.conv")], 0))
        self.a2, self.g2, self.o = f("a2").contiguous(), f("g2").contiguous(), f("o").contiguous()
        self.A_log, self.dt_bias, self.norm = _f32(f("A_log")), _f32(f("dt_bias")), _f32(f("norm"))

    def cache_request(self) -> StateRequest:
        return StateRequest((sum(n for _, n in self.fields),), torch.float32)

    def first_weight(self):
        return self.w_in

    def forward(self, ctx, x, cache: StateView):
        T = x.shape[0]
        H, G, d, v, C = self.heads, self.kv_heads, self.dim, self.vdim, self.channels
        f32 = dict(dtype=torch.float32, device=x.device)
        state = ops.StateRows(cache.rows, self.fields)
        p = product_f32(x, self.w_in)
        qkv = torch.empty((T, C), **f32)
        if not ops.conv_silu_unit(ctx, p, self.conv, state, "tail", qkv, C, n_unit=2 * G, dim=d,
                                  n_scaled=G, extra=d ** -0.5, unit_eps=self.unit_eps):
            ops.state_tail_update(ctx, p, state, "tail", self.taps - 1, C)
        low = torch.empty((T, self.decay_rank + self.gate_rank), dtype=x.dtype, device=x.device)
        ops.unary_cast(p[:, C + H:], low)
        decay = product_f32(low[:, :self.decay_rank], self.a2)
        gate = product_f32(low[:, self.decay_rank:], self.g2)
        ops.decay_gate(decay, d, self.dt_bias, self.A_log)
        o = torch.empty((T, H * v), **f32)
        ops.state_scan(ctx, ops.SCAN_DELTA, qkv, qkv[:, G * d:], qkv[:, 2 * G * d:], decay, state,
                       "S", o, H, H // G, d, v, beta=p[:, C:])
        y = torch.empty((T, H * v), dtype=x.dtype, device=x.device)
        ops.head_norm_gate(o, self.norm, False, gate, "sigmoid", self.eps, y, H, v)
        return product_f32(y, self.o)


@register_mixer("gated_delta")
class GatedDelta(Part):
    """The gated delta rule with a decay per head (see the module's notes). The
    output gate's activation and the constant inside the unit vectors' root are
    parameters."""
    replay_safe = True
    accepts_row_scaled = True  # the first product applies a deferred norm's row scale

    def __init__(self, width: int, heads: int, kv_heads: int, dim: int, vdim: int, taps: int,
                 eps: float, unit_eps: float = 1e-6, gate: str = "silu", *,
                 dtype: torch.dtype, device: torch.device):
        if kv_heads <= 0 or heads % kv_heads:
            raise ValueError(f"{heads} heads are not a multiple of {kv_heads} key heads")
        if dim > 512:
            raise ValueError(f"{dim} key channels a head: the recurrence kernel holds at most 512")
        if gate not in ("silu", "sigmoid"):
            raise ValueError(f"output gate {gate!r}; known: silu, sigmoid")
        self.width, self.heads, self.kv_heads, self.dim, self.vdim = width, heads, kv_heads, dim, vdim
        self.taps, self.eps, self.unit_eps, self.gate = int(taps), float(eps), float(unit_eps), gate
        self.dtype, self.device = dtype, device
        self.channels = 2 * kv_heads * dim + heads * vdim
        self.fields = [("tail", (self.taps - 1) * self.channels), ("S", heads * dim * vdim)]

    def _shapes(self):
        W, H, G, d, v = self.width, self.heads, self.kv_heads, self.dim, self.vdim
        return {"q": (G * d, W), "q.conv": (G * d, self.taps), "k": (G * d, W),
                "k.conv": (G * d, self.taps), "v": (H * v, W), "v.conv": (H * v, self.taps),
                "b": (H, W), "A_log": (H,), "norm": (v,), "a": (H, W), "dt_bias": (H,),
                "g": (H * v, W), "o": (W, H * v)}

    def expected_tensors(self, prefix: str) -> Dict[str, ExpectedTensor]:
        return {f"{prefix}.{n}": ExpectedTensor(s) for n, s in self._shapes().items()}

    def load(self, prefix: str, fetch: Fetch) -> None:
        f = lambda n: fetch(f"{prefix}.{n}")
        # every projection of h in one product: q | k | v | gate | beta | decay
        self.w_in = torch.cat([f("q"), f("k"), f("v"), f("g"), f("b"), f("a")], 0).contiguous()
        self.conv = _f32(torch.cat([f("q.conv"), f("k.conv"), f("v.conv")], 0))
        self.o = f("o").contiguous()
        self.A_log, self.dt_bias, self.norm = _f32(f("A_log")), _f32(f("dt_bias")), _f32(f("norm"))

    def cache_request(self) -> StateRequest:
        return StateRequest((sum(n for _, n in self.fields),), torch.float32)

    def first_weight(self):
        return self.w_in

    def forward(self, ctx, x, cache: StateView):
        T = x.shape[0]
        H, G, d, v, C = self.heads, self.kv_heads, self.dim, self.vdim, self.channels
        f32 = dict(dtype=torch.float32, device=x.device)
        state = ops.StateRows(cache.rows, self.fields)
        p = product_f32(x, self.w_in)  # [T, C | H v | H | H]
        qkv = torch.empty((T, C), **f32)
        if not ops.conv_silu_unit(ctx, p, self.conv, state, "tail", qkv, C, n_unit=2 * G, dim=d,
                                  n_scaled=G, extra=d ** -0.5, unit_eps=self.unit_eps):
            ops.state_tail_update(ctx, p, state, "tail", self.taps - 1, C)
        at = C + H * v
        decay = torch.empty((T, H), **f32)
        ops.decay_gate(p[:, at + H:at + 2 * H], 1, self.dt_bias, self.A_log, out=decay)
        o = torch.empty((T, H * v), **f32)
        ops.state_scan(ctx, ops.SCAN_DELTA, qkv, qkv[:, G * d:], qkv[:, 2 * G * d:], decay, state,
                       "S", o, H, H // G, d, v, beta=p[:, at:at + H], decay_per_head=True)
        y = torch.empty((T, H * v), dtype=x.dtype, device=x.device)
        ops.head_norm_gate(o, self.norm, False, p[:, C:at], self.gate, self.eps, y, H, v)
        return product_to_residual(ctx, y, self.o)


@register_mixer("wkv_time_mix")
class WkvTimeMix(Part):
    replay_safe = True
    MIXES = ("r", "k", "v", "g", "w")

    def __init__(self, width: int, heads: int, dim: int, eps: float, decay_rank: int, *,
                 dtype: torch.dtype, device: torch.device):
        if dim > 512:
            raise ValueError(f"{dim} key channels a head: the recurrence kernel holds at most 512")
        self.width, self.heads, self.dim, self.eps = width, heads, dim, float(eps)
        self.decay_rank = decay_rank
        self.dtype, self.device = dtype, device
        self.fields = [("prev", width), ("S", heads * dim * dim)]

    def _shapes(self):
        W, n = self.width, self.heads * self.dim
        shapes = {f"mu.{s}": (W,) for s in self.MIXES}
        shapes.update({"r": (n, W), "k": (n, W), "v": (n, W), "g": (n, W),
                       "w1": (self.decay_rank, W), "w2": (n, self.decay_rank), "w0": (n,),
                       "u": (self.heads, self.dim), "norm": (n,), "o": (W, n)})
        return shapes

    def expected_tensors(self, prefix: str) -> Dict[str, ExpectedTensor]:
        return {f"{prefix}.{n}": ExpectedTensor(s) for n, s in self._shapes().items()}

    def load(self, prefix: str, fetch: Fetch) -> None:
        f = lambda n: fetch(f"{prefix}.{n}")
        self.mu = _f32(torch.stack([f(f"mu.{s}") for s in self.MIXES], 0))
        self.r, self.k, self.v, self.g = (f(n).contiguous() for n in ("r", "k", "v", "g"))
        self.w1, self.w2, self.o = f("w1").contiguous(), f("w2").contiguous(), f("o").contiguous()
        self.w0, self.u, self.norm = _f32(f("w0")), _f32(f("u")), _f32(f("norm"))

    def cache_request(self) -> StateRequest:
        return StateRequest((sum(n for _, n in self.fields),), torch.float32)

    def first_weight(self):
        return self.r

    def forward(self, ctx, x, cache: StateView):
        T, W = x.shape
        H, d = self.heads, self.dim
        state = ops.StateRows(cache.rows, self.fields)
        mixes = torch.empty((len(self.MIXES), T, W), dtype=x.dtype, device=x.device)
        if not ops.token_shift_mix(ctx, x, state, "prev", self.mu, mixes):
            ops.state_tail_update(ctx, x, state, "prev", 1, W)
        r, k, v, g = (product_f32(mixes[i], w) for i, w in
                      enumerate((self.r, self.k, self.v, self.g)))
        low = torch.empty((T, self.decay_rank), dtype=x.dtype, device=x.device)
        ops.unary_cast(product_f32(mixes[4], self.w1), low, "tanh")
        decay = product_f32(low, self.w2)
        ops.decay_gate(decay, d, self.w0, None)
        o = torch.empty((T, H * d), dtype=torch.float32, device=x.device)
        ops.state_scan(ctx, ops.SCAN_WKV, r, k, v, decay, state, "S", o, H, 1, d, d, bonus=self.u)
        y = torch.empty((T, H * d), dtype=x.dtype, device=x.device)
        ops.head_norm_gate(o, self.norm, True, g, "silu", self.eps, y, H, d)
        return product_f32(y, self.o)


@register_mixer("state_space_duality")
class StateSpaceDuality(Part):
    """The Mamba-2 layer (see the module's notes). Tensor names under the prefix:
    `in`, `conv`, `conv.b`, `dt_bias`, `A_log`, `D`, `norm`, `o`."""
    replay_safe = True

    def __init__(self, width: int, heads: int, vdim: int, state: int, groups: int, taps: int,
                 eps: float, norm_groups: int = 1, *, dtype: torch.dtype, device: torch.device):
        if groups <= 0 or heads % groups:
            raise ValueError(f"{heads} heads are not a multiple of {groups} groups")
        if state > 512:
            raise ValueError(f"a state of {state} rows a head: the recurrence kernel holds at most 512")
        inner = heads * vdim
        if norm_groups <= 0 or inner % norm_groups:
            raise ValueError(f"{inner} inner channels are not a multiple of {norm_groups} norm groups")
        self.width, self.heads, self.vdim, self.state, self.groups = width, heads, vdim, state, groups
        self.taps, self.eps, self.norm_groups = int(taps), float(eps), int(norm_groups)
        self.inner = inner
        self.channels = inner + 2 * groups * state   # what passes the convolution
        self.rows_in = 2 * inner + 2 * groups * state + heads
        self.dtype, self.device = dtype, device
        self.fields = [("tail", (self.taps - 1) * self.channels), ("S", heads * state * vdim)]

    def _shapes(self):
        return {"in": (self.rows_in, self.width), "conv": (self.channels, self.taps),
                "conv.b": (self.channels,), "dt_bias": (self.heads,), "A_log": (self.heads,),
                "D": (self.heads,), "norm": (self.inner,), "o": (self.width, self.inner)}

    def expected_tensors(self, prefix: str) -> Dict[str, ExpectedTensor]:
        return {f"{prefix}.{n}": ExpectedTensor(s) for n, s in self._shapes().items()}

    def load(self, prefix: str, fetch: Fetch) -> None:
        f = lambda n: fetch(f"{prefix}.{n}")
        self.w_in, self.o = f("in").contiguous(), f("o").contiguous()
        self.conv, self.conv_bias = _f32(f("conv")), _f32(f("conv.b"))
        self.dt_bias, self.A_log, self.skip = _f32(f("dt_bias")), _f32(f("A_log")), _f32(f("D"))
        self.norm = _f32(f("norm"))

    def cache_request(self) -> StateRequest:
        return StateRequest((max(1, sum(n for _, n in self.fields)),), torch.float32)

    def first_weight(self):
        return self.w_in

    # the same three pieces as the attention beside which it may stand (parts/parallel.py)
    def input_weight(self) -> torch.Tensor:
        return self.w_in

    def output_weight(self) -> torch.Tensor:
        return self.o

    @property
    def inner_size(self) -> int:
        return self.inner

    def between(self, ctx, p: torch.Tensor, cache: StateView, out: torch.Tensor,
                out_scale: float = 1.0) -> torch.Tensor:
        """From the input projection `p` (float32 rows [z | x | B | C | dt]) to the gated,
        normalised rows in `out` (rows may lie further apart), times `out_scale`."""
        T = p.shape[0]
        H, G, N, v, C, inner = self.heads, self.groups, self.state, self.vdim, self.channels, \
            self.inner
        f32 = dict(dtype=torch.float32, device=p.device)
        state = ops.StateRows(cache.rows, self.fields)
        xbc = torch.empty((T, C), **f32)
        if not ops.conv_silu_unit(ctx, p[:, inner:], self.conv, state, "tail", xbc, C,
                                  bias=self.conv_bias):
            ops.state_tail_update(ctx, p[:, inner:], state, "tail", self.taps - 1, C)
        decay, steps = torch.empty((T, H), **f32), torch.empty((T, H), **f32)
        ops.decay_gate(p[:, inner + C:inner + C + H], 1, self.dt_bias, self.A_log, out=decay,
                       steps=steps)
        y = torch.empty((T, inner), **f32)
        ops.state_scan(ctx, ops.SCAN_SSD, xbc[:, inner + G * N:], xbc[:, inner:], xbc, decay, state,
                       "S", y, H, H // G, N, v, beta=steps, bonus=self.skip, decay_per_head=True)
        ops.head_norm_gate(y, self.norm, True, p[:, :inner], "silu", self.eps, out,
                           self.norm_groups, inner // self.norm_groups, gate_first=True,
                           out_scale=out_scale)
        return out

    def forward(self, ctx, x, cache: StateView):
        y = torch.empty((x.shape[0], self.inner), dtype=x.dtype, device=x.device)
        self.between(ctx, product_f32(x, self.w_in), cache, y)
        return product_f32(y, self.o)
