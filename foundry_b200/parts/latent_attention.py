"""Attention through a low-rank latent of keys and values, as a mixer.

    c_q = rmsnorm(Wdq h) * wq;   q = Wuq c_q   (heads x [dim plain | rot_dim rotated])
    Wdkv h = [kv_rank rows | rot_dim rows]:  c = rmsnorm(first) * wkv  is the latent,
    the last rot_dim rows, rotated, are ONE key part shared by all heads
    per head:  k_plain = Wuk c,  v = Wuv c
    s = (q_plain . k_plain + q_rot . k_rot) * scale;  causal;
    p = exp(s) / (exp(sink_h) + sum exp(s))     a learned score per head joins the sum once
    out = Wo [heads' sum p v]

Options: `q_rank = 0`, the queries come straight from the input, q = Wq h (tensor `q`;
no `dq`, `dq.norm`, `uq`); `sink = False`, the ordinary softmax; `output_gate`, the heads'
outputs side by side are multiplied, element by element, with sigmoid(Wg h) (tensor `g`;
the gate reads the mixer's input) in front of Wo.

The rotation turns neighbouring pairs (2i, 2i + 1) of the first `rot_dims`
elements of the rotated part by position * base^(-2i / rot_dims).

Only the latent and the rotated key part are cached: one row of kv_rank +
rot_dim elements per token, whatever the head count. The key and value
expansions are folded into the query and the output,

    q_plain . (Wuk_h c) = (Wuk_h^T q_plain) . c,    sum p (Wuv_h c) = Wuv_h (sum p c),

so a step, whatever it brings, is an attention of all heads over the one
cached row per token (key size kv_rank + rot_dim, the value its first kv_rank
elements) between two small per-head products.

A prompt step in which every sequence begins at its first token sees only its
own rows. In bfloat16, at head sizes the tensor-core kernel has, it expands
them instead (one product for k_plain | v of all heads) and runs the heads as
ordinary attention with keys of dim + rot_dim and values of vdim, which costs a
third of the operations of the folded form; the cache rows are written all the same.
"""
from __future__ import annotations

from typing import Dict, Optional

import numpy as np
import torch

from ..cache.store import KVRequest, KVView
from ..kernels import ops
from ..weights.loader import ExpectedTensor
from .base import Fetch, Part, register_mixer
from .linear import matmul_nt
from .products import product_f32, product_to_residual


@register_mixer("latent_attention")
class LatentAttention(Part):
    replay_safe = True
    accepts_row_scaled = True  # the first product applies a deferred norm's row scale

    def __init__(self, width: int, heads: int, dim: int, rot_dim: int, vdim: int, kv_rank: int,
                 q_rank: int, scale: float, eps: float, rot_base: float,
                 rot_dims: Optional[int] = None, sink: bool = True, output_gate: bool = False,
                 *, dtype: torch.dtype, device: torch.device):
        rot_dims = rot_dim if rot_dims is None else int(rot_dims)
        if rot_dims % 2 or not 0 <= rot_dims <= rot_dim:
            raise ValueError(f"{rot_dims} rotated elements of a part of {rot_dim}")
        if kv_rank + rot_dim > 1024 or kv_rank > 768:
            raise ValueError(f"latent rows of {kv_rank} + {rot_dim}: the attention kernel takes "
                             f"rows of at most 1024 with at most 768 latent elements")
        self.width, self.heads, self.dim, self.rot_dim, self.vdim = width, heads, dim, rot_dim, vdim
        self.kv_rank, self.q_rank = kv_rank, int(q_rank or 0)
        self.output_gate = bool(output_gate)
        self.scale, self.eps, self.sink = float(scale), float(eps), bool(sink)
        self.rot_dims, self.rot_base = rot_dims, float(rot_base)
        self.dtype, self.device = dtype, device
        self.row = kv_rank + rot_dim
        freq = np.power(np.float64(rot_base), -2.0 * np.arange(max(1, rot_dims // 2)) / max(1, rot_dims))
        self.freq = torch.from_numpy(freq.astype(np.float64)).to(device)

    def _shapes(self):
        W, H = self.width, self.heads
        shapes = {"dkv": (self.row, W), "dkv.norm": (self.kv_rank,),
                  "uk": (H * self.dim, self.kv_rank), "uv": (H * self.vdim, self.kv_rank),
                  "o": (W, H * self.vdim)}
        if self.q_rank:
            shapes.update({"dq": (self.q_rank, W), "dq.norm": (self.q_rank,),
                           "uq": (H * (self.dim + self.rot_dim), self.q_rank)})
        else:
            shapes["q"] = (H * (self.dim + self.rot_dim), W)
        if self.output_gate:
            shapes["g"] = (H * self.vdim, W)
        if self.sink:
            shapes["sink"] = (H,)
        return shapes

    def expected_tensors(self, prefix: str) -> Dict[str, ExpectedTensor]:
        return {f"{prefix}.{n}": ExpectedTensor(s) for n, s in self._shapes().items()}

    def load(self, prefix: str, fetch: Fetch) -> None:
        f = lambda n: fetch(f"{prefix}.{n}")
        H, d, e, r = self.heads, self.dim, self.vdim, self.kv_rank
        # one product for everything that reads the mixer's input: the query latent (or
        # the queries themselves), the gate, the key-value latent with the rotated key part
        first = [f("dq")] if self.q_rank else [f("q")]
        self.down = torch.cat(first + [f("dkv")] + ([f("g")] if self.output_gate else []),
                              0).contiguous()
        self.uq = f("uq").contiguous() if self.q_rank else None
        self.o = f("o").contiguous()
        # per head: [r, d] so that (plain query) x this^T is the query against the latent
        self.uk_t = f("uk").view(H, d, r).transpose(1, 2).contiguous()
        self.uv = f("uv").view(H, e, r).contiguous()
        # per head [k_plain rows | v rows]: one product expands a step's latent rows
        self.expand = torch.cat([f("uk").view(H, d, r), self.uv], 1).reshape(H * (d + e), r).contiguous()
        self.q_norm = f("dq.norm").to(torch.float32).contiguous() if self.q_rank else None
        self.kv_norm = f("dkv.norm").to(torch.float32).contiguous()
        self.sink_logits = f("sink").to(torch.float32).contiguous() if self.sink else None

    def cache_request(self) -> KVRequest:
        return KVRequest(1, self.row, None, 0)  # values are a part of the key rows

    def first_weight(self):
        return self.down

    def context_flops(self, token_counts, starts) -> float:
        pairs = sum(0.5 * n * (2 * start + n + 1) for n, start in zip(token_counts, starts))
        return 2.0 * self.heads * (self.row + self.kv_rank) * pairs

    def forward(self, ctx, x, cache: KVView):
        T = x.shape[0]
        H, d, c, e, r = self.heads, self.dim, self.rot_dim, self.vdim, self.kv_rank
        act = dict(dtype=x.dtype, device=x.device)
        table = ctx.page_table(cache.group)
        # [T, q_rank (or the queries, H (d + c)) | kv_rank | rot_dim | the gate, H e]
        down = product_f32(x, self.down)
        n_first = self.q_rank or H * (d + c)
        gate = down[:, n_first + self.row:] if self.output_gate else None
        cq = torch.empty((T, self.q_rank), **act)
        expanded = (getattr(ctx, "fresh", False) and r % 8 == 0 and c % 8 == 0 and d % 8 == 0
                    and e % 8 == 0 and ops.attention_maps_fits(ctx, cq, d + c, e, 1))
        rows = torch.empty((T, self.row), **act) if expanded else None
        if self.q_rank:
            ops.latent_rows(down, cq, self.q_norm, self.kv_norm, self.eps, self.freq,
                            self.rot_dims, ctx.positions, ctx.seq_of_token, table, cache.k, r, c,
                            write_cache=cache.writes, rows_out=rows)
            q = product_f32(cq, self.uq)  # [T, H (d + c)]
        else:  # no query latent: the kernel norms and caches the key-value side only
            ops.latent_rows(down[:, n_first:], cq, self.kv_norm, self.kv_norm, self.eps,
                            self.freq, self.rot_dims, ctx.positions, ctx.seq_of_token, table,
                            cache.k, r, c, write_cache=cache.writes, rows_out=rows)
            q = down[:, :n_first]
        if expanded:
            q_full = torch.empty((T, H, d + c), **act)
            ops.split_rotate(q, None, q_full, d, self.freq, self.rot_dims, ctx.positions,
                             ctx.seq_of_token, H, d, c)
            kv = torch.empty((T, H, d + e), **act)
            matmul_nt(rows[:, :r], self.expand, kv.view(T, H * (d + e)))
            out = torch.empty((T, H * e), **act)
            ops.attention_maps_rows(ctx, q_full.view(T, H * (d + c)), out, kv[:, :, :d],
                                    rows[:, r:], kv[:, :, d:], H, d + c, e, self.scale,
                                    sink_logits=self.sink_logits)
            if gate is not None:
                ops.sigmoid_gate(out, gate)
            return product_to_residual(ctx, out, self.o)
        q_plain = torch.empty((T, H * d), **act)
        q_wide = torch.empty((T, H, self.row), **act)
        ops.split_rotate(q, q_plain, q_wide, r, self.freq, self.rot_dims, ctx.positions,
                         ctx.seq_of_token, H, d, c)
        ops.head_products(q_plain.view(T, H, d), self.uk_t, q_wide[:, :, :r])
        mixed = torch.empty((T, H * r), **act)
        if ops.attention_folded_fits(q_wide, self.row, r):
            # all heads as the rows of tensor-core tiles over the shared latent rows
            ops.attention_folded(ctx, q_wide.view(T, H * self.row), mixed, table, cache.k, H,
                                 self.row, r, self.scale, sink_logits=self.sink_logits)
        else:
            ops.attention_sink(ctx, q_wide.view(T, H * self.row), mixed, table, cache.k, cache.k, H,
                               1, self.row, r, self.scale, sink_logits=self.sink_logits,
                               values_in_keys=True)
        out = torch.empty((T, H, e), **act)
        ops.head_products(mixed.view(T, H, r), self.uv, out)
        if gate is not None:
            ops.sigmoid_gate(out.view(T, H * e), gate)
        return product_to_residual(ctx, out.view(T, H * e), self.o)
