"""Grouped-query attention with rotated queries and keys, a constant score scale and a
learnt sink per head, as a mixer.

    q = Wq h (H x dim), k = Wk h (G x dim), v = Wv h (G x vdim)   (one product), no biases
    q, k: the first `rot_dims` elements of every head turned by the token's position p,
          element 2i with 2i + 1 ("interleaved") or i with i + rot_dims / 2 ("half"),
          by p * f_i; the frequencies f are a parameter (float64; any scaling of them is
          another vector)
    s_ij = (q_i . k_j) * scale;   j visible to i iff j <= i
    p_ij = exp(s_ij) / (exp(sink_h) + sum_j exp(s_ij))     the sink has no key and no value
    out = Wo [heads' outputs side by side]

Query head a reads key-value head a // (H / G). Keys have `dim` elements a head,
values `vdim`. With `own_kv = False` the mixer has no key and value projections: it
reads the cache entry that another run of the schedule wrote (keys as they were rotated
there), with its own queries, sink and output projection. Tensor names under the
mixer's prefix: `q k v o sink`.

Kernels. The general path, any sizes and both element types: one product for q | k | v
(float32 out), one kernel that rotates (the angle a 64-bit product) and writes the cache
rows, the CUDA-core attention with the sink. In bfloat16, with keys and values of one
size that the tensor-core attentions have, the mixer runs as the plain grouped attention
does: rotation and cache write in the projection's epilogue (the angle a 32-bit
product), the tcgen05 attention for prompts and the split-range `mma.sync` attention for
single tokens, both with the sink's term as the start of the running sum.
"""
from __future__ import annotations

from typing import Dict, Optional, Sequence

import numpy as np
import torch

from ..cache.store import KVRequest, KVView
from ..kernels import ops
from ..weights.loader import ExpectedTensor
from .attention import rotated_projection
from .base import Fetch, Part, register_mixer
from .products import product_f32, product_to_residual


@register_mixer("rotary_sink_attention")
class RotarySinkAttention(Part):
    replay_safe = True

    def __init__(self, width: int, heads: int, kv_heads: int, dim: int, vdim: int, scale: float,
                 frequencies: Optional[Sequence[float]] = None, pairing: str = "interleaved",
                 sink: bool = True, own_kv: bool = True, *, dtype: torch.dtype,
                 device: torch.device):
        if kv_heads <= 0 or heads % kv_heads:
            raise ValueError(f"{heads} heads are not a multiple of {kv_heads} key-value heads")
        if not 1 <= dim <= 256 or not 1 <= vdim <= 256:
            raise ValueError(f"key size {dim} and value size {vdim} must be at most 256")
        freq = np.asarray(() if frequencies is None else frequencies, dtype=np.float64)
        if 2 * freq.size > dim:
            raise ValueError(f"{2 * freq.size} rotated elements of heads of {dim}")
        if pairing not in ops.PAIRINGS:
            raise ValueError(f"rotation pairing {pairing!r}; known: {sorted(ops.PAIRINGS)}")
        self.width, self.heads, self.kv_heads, self.dim, self.vdim = width, heads, kv_heads, dim, vdim
        self.scale, self.sink, self.own_kv, self.pairing = float(scale), bool(sink), bool(own_kv), pairing
        self.dtype, self.device = dtype, device
        self.nq, self.nk, self.nv = heads * dim, kv_heads * dim, kv_heads * vdim
        self.freq = torch.from_numpy(freq.copy()).to(device) if freq.size else None
        # for the projections that rotate in their epilogue (bfloat16 steps)
        self.inv_freq = torch.from_numpy(freq.astype(np.float32)).to(device)
        self.angles_key = ("rotary angles", freq.astype(np.float32).tobytes())
        self.w_in = self.w_o = self.sink_logits = None

    def _shapes(self):
        shapes = {"q": (self.nq, self.width), "o": (self.width, self.heads * self.vdim)}
        if self.own_kv:
            shapes.update(k=(self.nk, self.width), v=(self.nv, self.width))
        if self.sink:
            shapes["sink"] = (self.heads,)
        return shapes

    def expected_tensors(self, prefix: str) -> Dict[str, ExpectedTensor]:
        return {f"{prefix}.{n}": ExpectedTensor(s) for n, s in self._shapes().items()}

    def load(self, prefix: str, fetch: Fetch) -> None:
        names = ("q", "k", "v") if self.own_kv else ("q",)
        self.w_in = torch.cat([fetch(f"{prefix}.{n}") for n in names], 0).contiguous()
        self.w_o = fetch(f"{prefix}.o").contiguous()
        self.sink_logits = (fetch(f"{prefix}.sink").to(torch.float32).contiguous()
                            if self.sink else None)

    def cache_request(self) -> KVRequest:
        return KVRequest(self.kv_heads, self.dim, None, self.vdim)

    def first_weight(self):
        return self.w_in

    def context_flops(self, token_counts, starts) -> float:
        pairs = sum(0.5 * n * (2 * start + n + 1) for n, start in zip(token_counts, starts))
        return 2.0 * self.heads * (self.dim + self.vdim) * pairs

    def _as_plain_heads(self, x, cache: KVView) -> bool:
        """Whether the step runs on the kernels of the plain grouped attention."""
        return (x.dtype == torch.bfloat16 and self.dim == self.vdim
                and self.dim in ops.FAST_HEAD_DIMS and self.heads // self.kv_heads <= 16
                and cache.k.stride() == cache.v.stride() and self.pairing == "interleaved")

    def forward(self, ctx, x, cache: KVView):
        T = x.shape[0]
        H, G, d, e = self.heads, self.kv_heads, self.dim, self.vdim
        table = ctx.page_table(cache.group)
        writes = self.own_kv and cache.writes
        if self.own_kv and self._as_plain_heads(x, cache):
            q = rotated_projection(ctx, x, self.w_in, self.inv_freq, 2 * self.inv_freq.numel(),
                                   self.pairing, self.angles_key, cache, H, G, d)
            attn = torch.empty((T, H * e), dtype=x.dtype, device=x.device)
            ops.attention(ctx, q, attn, table, cache.k, cache.v, H, G, d, self.scale,
                          then_reads=self.w_o, sink_logits=self.sink_logits)
            return product_to_residual(ctx, attn, self.w_o)
        rows = product_f32(x, self.w_in)  # [T, q | k | v] or [T, q]
        q = torch.empty((T, self.nq), dtype=x.dtype, device=x.device)
        ops.head_norm_rope_cache_write(rows, q, None, None, 1.0, False, self.freq, ctx.positions,
                                       ctx.seq_of_token, table, cache.k, cache.v, H,
                                       G if self.own_kv else 0, d, e, write_cache=writes,
                                       qk_norm=False, pairing=self.pairing)
        attn = torch.empty((T, H * e), dtype=x.dtype, device=x.device)
        if self._as_plain_heads(x, cache):  # a reader of another run's keys and values
            ops.attention(ctx, q, attn, table, cache.k, cache.v, H, G, d, self.scale,
                          then_reads=self.w_o, sink_logits=self.sink_logits)
        else:
            ops.attention_sink(ctx, q, attn, table, cache.k, cache.v, H, G, d, e, self.scale,
                               sink_logits=self.sink_logits)
        return product_to_residual(ctx, attn, self.w_o)
