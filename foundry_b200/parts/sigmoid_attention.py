"""Grouped-query attention with sigmoid weights inside chunks, as a mixer.

    q = Wq h, k = Wk h, v = Wv h, gate = Wg h   (one product), no biases
    q, k per head:  x / sqrt(mean(x^2) + eps) * w   (w [dim], shared by the heads), then
        rotated on the first `rotary` elements: element i with element i + rotary/2 by the
        angle p * base^(-2i / rotary) at position p
    v per head:  x / sqrt(mean(x^2) + eps)  (no weight; cached so)          [value_norm]
    s_ij = (q_i . k_j) * scale + bias_h
    j visible to i iff j <= i and floor(i / chunk) == floor(j / chunk)      [chunk; None: j <= i]
    o_i = sigmoid(gate_i,h) * sum_j sigmoid(s_ij) v_j                       [output_gate]
    out = Wo [heads' outputs side by side]

The weights of the keys are not normalised over the keys. Keys have `dim`
elements a head, values `vdim`; query head a reads key head a // (heads /
kv_heads). Every constant is a parameter; the tensor names under the mixer's
prefix are `q k v g o`, `q.norm k.norm` and `pb` (the bias per head).

The cache keeps every key of the sequence; the kernels walk the query's own
chunk only.
"""
from __future__ import annotations

from typing import Dict, Optional

import numpy as np
import torch

from ..cache.store import KVRequest, KVView
from ..kernels import ops
from ..weights.loader import ExpectedTensor
from .base import Fetch, Part, register_mixer
from .linear import Linear
from .products import product_f32


@register_mixer("chunked_sigmoid_attention")
class ChunkedSigmoidAttention(Part):
    replay_safe = True

    def __init__(self, width: int, heads: int, kv_heads: int, dim: int, vdim: int, scale: float,
                 eps: float, chunk: Optional[int] = None, rotary: int = 0,
                 rotary_base: float = 10000.0, value_norm: bool = True, output_gate: bool = True,
                 head_bias: bool = True, *, dtype: torch.dtype, device: torch.device):
        if kv_heads <= 0 or heads % kv_heads:
            raise ValueError(f"{heads} heads are not a multiple of {kv_heads} key-value heads")
        if not 1 <= vdim <= 256 or dim < 1:
            raise ValueError(f"key size {dim}, value size {vdim}: values of at most 256")
        if rotary < 0 or rotary % 2 or rotary > dim:
            raise ValueError(f"{rotary} rotated elements in heads of {dim}")
        self.width, self.heads, self.kv_heads, self.dim, self.vdim = width, heads, kv_heads, dim, vdim
        self.scale, self.eps = float(scale), float(eps)
        self.chunk = int(chunk) if chunk else 0
        self.rotary, self.rotary_base = int(rotary), float(rotary_base)
        self.value_norm, self.output_gate, self.head_bias = bool(value_norm), bool(output_gate), \
            bool(head_bias)
        self.dtype, self.device = dtype, device
        self.nq, self.nk, self.nv = heads * dim, kv_heads * dim, kv_heads * vdim
        outs = [("q", self.nq), ("k", self.nk), ("v", self.nv)]
        if self.output_gate:
            outs.append(("g", heads))
        self.qkvg = Linear(width, outs, dtype=dtype, device=device, suffix="")
        self.o = Linear(heads * vdim, [("o", width)], dtype=dtype, device=device, suffix="")
        self.q_norm = self.k_norm = self.bias = self.freq = None

    def expected_tensors(self, prefix: str) -> Dict[str, ExpectedTensor]:
        out = {**self.qkvg.expected_tensors(prefix), **self.o.expected_tensors(prefix),
               f"{prefix}.q.norm": ExpectedTensor((self.dim,)),
               f"{prefix}.k.norm": ExpectedTensor((self.dim,))}
        if self.head_bias:
            out[f"{prefix}.pb"] = ExpectedTensor((self.heads,))
        return out

    def load(self, prefix: str, fetch: Fetch) -> None:
        self.qkvg.load(prefix, fetch)
        self.o.load(prefix, fetch)
        self.q_norm = fetch(f"{prefix}.q.norm").to(torch.float32).contiguous()
        self.k_norm = fetch(f"{prefix}.k.norm").to(torch.float32).contiguous()
        if self.head_bias:
            self.bias = fetch(f"{prefix}.pb").to(torch.float32).contiguous()
        if self.rotary:
            f = np.power(np.float64(self.rotary_base),
                         -2.0 * np.arange(self.rotary // 2, dtype=np.float64) / self.rotary)
            self.freq = torch.from_numpy(f).to(self.q_norm.device)

    def cache_request(self) -> KVRequest:
        return KVRequest(self.kv_heads, self.dim, None, self.vdim)

    def first_weight(self):
        return self.qkvg.weight

    def context_flops(self, token_counts, starts) -> float:
        pairs = 0.0
        for n, start in zip(token_counts, starts):
            for p in range(start, start + n):
                pairs += (p % self.chunk if self.chunk else p) + 1
        return 2.0 * self.heads * (self.dim + self.vdim) * pairs

    # A mixer that can stand beside another one on the same input (parts/parallel.py)
    # offers its input projection's weight, the work between its two products, and its
    # output projection's weight.
    def input_weight(self) -> torch.Tensor:
        return self.qkvg.weight

    def output_weight(self) -> torch.Tensor:
        return self.o.weight

    @property
    def inner_size(self) -> int:
        return self.heads * self.vdim

    def between(self, ctx, p: torch.Tensor, cache: KVView, out: torch.Tensor,
                out_scale: float = 1.0) -> torch.Tensor:
        """From the projections `p` (float32 rows [q | k | v | gate]) to the heads'
        gated outputs side by side in `out` (rows may lie further apart), times
        `out_scale`."""
        T = p.shape[0]
        table = ctx.page_table(cache.group)
        q = torch.empty((T, self.nq), dtype=out.dtype, device=p.device)
        ops.head_norm_rope_cache_write(p, q, self.q_norm, self.k_norm, self.eps, self.value_norm,
                                       self.freq, ctx.positions, ctx.seq_of_token, table, cache.k,
                                       cache.v, self.heads, self.kv_heads, self.dim, self.vdim,
                                       write_cache=cache.writes)
        at = self.nq + self.nk + self.nv
        gate = p[:, at:at + self.heads] if self.output_gate else None
        ops.attention_sigmoid(ctx, q, out, table, cache.k, cache.v, self.heads, self.kv_heads,
                              self.dim, self.vdim, self.scale, self.chunk, self.bias, gate,
                              out_scale=out_scale)
        return out

    def forward(self, ctx, x, cache: KVView):
        attn = torch.empty((x.shape[0], self.inner_size), dtype=x.dtype, device=x.device)
        self.between(ctx, product_f32(x, self.qkvg.weight), cache, attn)
        return product_f32(attn, self.o.weight)
