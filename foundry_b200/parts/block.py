"""The arrangement of a layer's parts.

`pre_norm_residual` is the reference's decoder layer
(src/models/llama/model.rs:254-278):

    h = x + mixer(norm1(x));  x' = h + feed_forward(norm2(h))

The residual stream is float32 and each sum is made in the kernel that also
normalises for the next part, so a block receives the previous block's output
still un-added (`delta`) and returns its own the same way. In single-token
steps that kernel is the projection in front of the norm: the block offers the
norm's `sink` to the part in front through `ctx.residual_sink`, and a part
that used it returns an `ops.NormPending`, which the norm turns into the
`ops.RowScaled` input of the part behind it.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..config.spec import LayerSpec
from ..weights.loader import ExpectedTensor
from .base import (FEED_FORWARDS, MIXERS, NORMS, Fetch, Part, first_weight_of,
                   register_block)


@register_block("pre_norm_residual")
class PreNormResidualBlock(Part):
    replay_safe = True  # forward reads nothing of the step on the host

    def __init__(self, layer: LayerSpec, *, dtype: torch.dtype, device: torch.device):
        ctx = dict(dtype=dtype, device=device)
        self.prefix = layer.prefix
        self.names = dict(layer.names)
        self.mixer = MIXERS.build(layer.mixer, **ctx)
        self.feed_forward = FEED_FORWARDS.build(layer.feed_forward, **ctx)
        self.mixer_norm = NORMS.build(layer.mixer_norm, **ctx)
        self.feed_forward_norm = NORMS.build(layer.feed_forward_norm, **ctx)

    def _named(self):
        p, n = self.prefix, self.names
        return ((self.mixer_norm, f"{p}.{n['mixer_norm']}"),
                (self.mixer, f"{p}.{n['mixer']}"),
                (self.feed_forward_norm, f"{p}.{n['feed_forward_norm']}"),
                (self.feed_forward, f"{p}.{n['feed_forward']}"))

    def expected_tensors(self, prefix: str = "") -> Dict[str, ExpectedTensor]:
        out: Dict[str, ExpectedTensor] = {}
        for part, name in self._named():
            out.update(part.expected_tensors(name))
        return out

    def load(self, prefix: str, fetch: Fetch) -> None:
        for part, name in self._named():
            part.load(name, fetch)

    def cache_request(self):
        return self.mixer.cache_request()

    def first_weight(self):
        return first_weight_of(self.mixer)

    def input_sink(self, resid: torch.Tensor):
        """The sink of this block's first norm, if its mixer takes the norm's
        output without its row scale; for whatever runs in front of the block."""
        return _sink_for(self.mixer_norm, self.mixer, resid)

    def forward(self, ctx, resid: torch.Tensor, delta, cache):
        after_block = getattr(ctx, "reads_after_part", None)  # what follows this block
        sink_after_block = getattr(ctx, "residual_sink", None)
        normed = self.mixer_norm.add_norm(resid, delta)
        ctx.reads_after_part = first_weight_of(self.feed_forward)
        ctx.residual_sink = _sink_for(self.feed_forward_norm, self.feed_forward, resid)
        mixed = self.mixer.forward(ctx, normed, cache)
        normed = self.feed_forward_norm.add_norm(resid, mixed)
        ctx.reads_after_part = after_block
        ctx.residual_sink = sink_after_block
        return self.feed_forward.forward(ctx, normed)


def _sink_for(norm, consumer, resid: torch.Tensor):
    """`norm.sink(resid)` where the norm offers one and `consumer` takes the
    norm's output as an `ops.RowScaled`; else None."""
    offer = getattr(norm, "sink", None)
    if not callable(offer) or not getattr(consumer, "accepts_row_scaled", False):
        return None
    return offer(resid)


@register_block("sandwich_norm_residual")
class SandwichNormBlock(Part):
    """A norm in front of AND behind each part:

        x <- x + post1(mixer(pre1(x)));  x <- x + post2(feed_forward(pre2(x)))

    the second line only where the layer has a feed-forward. A part's output
    leaves as an `ops.NormedDelta` (its post-norm still to be applied) and the
    norm that runs next makes `x += post(y)` and its own normalisation in one
    pass over the row, so the block, like `pre_norm_residual`, returns its last
    output un-added. The residual stream and all statistics are 32-bit.

    With `depth` = n > 0 the block is the n-th of `depth_total` whose results are
    kept, and what leaves it is a weighted sum over all streams so far:

        X_n = the block's result;  x <- sum_j w[j] X_j, j = 0 .. n

    X_0 being the stream as the embedding left it and w the tensor
    `<prefix>.<depth_name>` of n + 1 numbers. The sum is work of the norm that
    runs next, too: the block's output leaves as an `ops.DepthMix`."""
    replay_safe = True

    def __init__(self, layer: LayerSpec, depth: int = 0, depth_total: int = 0,
                 depth_name: str = "dwa", *, dtype: torch.dtype, device: torch.device):
        ctx = dict(dtype=dtype, device=device)
        if layer.mixer_post_norm is None:
            raise ValueError("sandwich_norm_residual needs a norm behind the mixer")
        if depth < 0 or (depth > 0 and depth > depth_total):
            raise ValueError(f"block {depth} of {depth_total} kept streams")
        self.depth, self.depth_total, self.depth_name = int(depth), int(depth_total), depth_name
        self.needs_embedding_output = self.depth > 0
        self.depth_weights = None
        self.prefix = layer.prefix
        self.names = dict(layer.names)
        self.mixer = MIXERS.build(layer.mixer, **ctx)
        self.mixer_norm = NORMS.build(layer.mixer_norm, **ctx)
        self.mixer_post_norm = NORMS.build(layer.mixer_post_norm, **ctx)
        self.feed_forward = self.feed_forward_norm = self.feed_forward_post_norm = None
        if layer.feed_forward is not None:
            if layer.feed_forward_norm is None or layer.feed_forward_post_norm is None:
                raise ValueError("sandwich_norm_residual needs both norms of the feed-forward")
            self.feed_forward = FEED_FORWARDS.build(layer.feed_forward, **ctx)
            self.feed_forward_norm = NORMS.build(layer.feed_forward_norm, **ctx)
            self.feed_forward_post_norm = NORMS.build(layer.feed_forward_post_norm, **ctx)

    def _named(self):
        p, n = self.prefix, self.names
        named = [(self.mixer_norm, f"{p}.{n['mixer_norm']}"), (self.mixer, f"{p}.{n['mixer']}"),
                 (self.mixer_post_norm, f"{p}.{n['mixer_post_norm']}")]
        if self.feed_forward is not None:
            named += [(self.feed_forward_norm, f"{p}.{n['feed_forward_norm']}"),
                      (self.feed_forward, f"{p}.{n['feed_forward']}"),
                      (self.feed_forward_post_norm, f"{p}.{n['feed_forward_post_norm']}")]
        return named

    def parts(self):
        """Every part of the block (for whoever asks them all something)."""
        return [part for part, _ in self._named()]

    def expected_tensors(self, prefix: str = "") -> Dict[str, ExpectedTensor]:
        out: Dict[str, ExpectedTensor] = {}
        for part, name in self._named():
            out.update(part.expected_tensors(name))
        if self.depth:
            out[f"{self.prefix}.{self.depth_name}"] = ExpectedTensor((self.depth + 1,))
        return out

    def load(self, prefix: str, fetch: Fetch) -> None:
        for part, name in self._named():
            part.load(name, fetch)
        if self.depth:
            self.depth_weights = fetch(f"{self.prefix}.{self.depth_name}").to(
                torch.float32).contiguous()

    def cache_request(self):
        return self.mixer.cache_request()

    def first_weight(self):
        return first_weight_of(self.mixer)

    def forward(self, ctx, resid: torch.Tensor, delta, cache):
        ctx.reads_after_part = None
        ctx.residual_sink = None  # these norms are not the kind a projection can take over
        normed = self.mixer_norm.add_norm(resid, delta)
        mixed = _as_rows(self.mixer.forward(ctx, normed, cache))
        pending = self.mixer_post_norm.pending(mixed)
        if self.feed_forward is not None:
            normed = self.feed_forward_norm.add_norm(resid, pending)
            pending = self.feed_forward_post_norm.pending(
                _as_rows(self.feed_forward.forward(ctx, normed)))
        if not self.depth:
            return pending
        from ..kernels import ops
        kept = ctx.shared.get(KEPT_STREAMS)
        if kept is None or kept.shape[0] < self.depth_total or kept.shape[1:] != resid.shape:
            kept = ctx.shared[KEPT_STREAMS] = torch.empty(
                (self.depth_total, *resid.shape), dtype=torch.float32, device=resid.device)
        return ops.DepthMix(pending, ctx.shared[EMBEDDING_OUTPUT], kept, self.depth_weights,
                            self.depth)


# keys of `ctx.shared`: the stream as the embedding left it (the model puts it there for
# blocks that say `needs_embedding_output`), and the blocks' kept results [depth, T, W]
EMBEDDING_OUTPUT = "embedding_output"
KEPT_STREAMS = "kept_streams"


def _as_rows(y):
    """A part's output as one tensor (split-K planes are summed in 32-bit)."""
    from ..kernels import ops
    return y.sum(torch.float32) if isinstance(y, ops.Planes) else y


@register_block("scaled_pre_norm_residual")
class ScaledPreNormBlock(Part):
    """The pre-norm arrangement with a constant on every part's output:

        x <- x + m * mixer(norm1(x));  x <- x + m * feed_forward(norm2(x))

    the second line only where the layer has a feed-forward. The products are
    not scaled: a part's output leaves as an `ops.ScaledDelta` and the norm
    that runs next makes `x += m * y` in 32-bit in its own pass over the row."""
    replay_safe = True

    def __init__(self, layer: LayerSpec, residual_scale: float = 1.0, *, dtype: torch.dtype,
                 device: torch.device):
        ctx = dict(dtype=dtype, device=device)
        self.prefix = layer.prefix
        self.names = dict(layer.names)
        self.residual_scale = float(residual_scale)
        self.mixer = MIXERS.build(layer.mixer, **ctx)
        self.mixer_norm = NORMS.build(layer.mixer_norm, **ctx)
        self.feed_forward = self.feed_forward_norm = None
        if layer.feed_forward is not None:
            if layer.feed_forward_norm is None:
                raise ValueError("scaled_pre_norm_residual: a feed-forward needs its norm")
            self.feed_forward = FEED_FORWARDS.build(layer.feed_forward, **ctx)
            self.feed_forward_norm = NORMS.build(layer.feed_forward_norm, **ctx)

    def _named(self):
        p, n = self.prefix, self.names
        named = [(self.mixer_norm, f"{p}.{n['mixer_norm']}"), (self.mixer, f"{p}.{n['mixer']}")]
        if self.feed_forward is not None:
            named += [(self.feed_forward_norm, f"{p}.{n['feed_forward_norm']}"),
                      (self.feed_forward, f"{p}.{n['feed_forward']}")]
        return named

    def parts(self):
        return [part for part, _ in self._named()]

    def expected_tensors(self, prefix: str = "") -> Dict[str, ExpectedTensor]:
        out: Dict[str, ExpectedTensor] = {}
        for part, name in self._named():
            out.update(part.expected_tensors(name))
        return out

    def load(self, prefix: str, fetch: Fetch) -> None:
        for part, name in self._named():
            part.load(name, fetch)

    def cache_request(self):
        return self.mixer.cache_request()

    def first_weight(self):
        return first_weight_of(self.mixer)

    def input_sink(self, resid: torch.Tensor):
        """The sink of this block's first norm, if its mixer takes the norm's
        output without its row scale; for whatever runs in front of the block."""
        return _sink_for(self.mixer_norm, self.mixer, resid)

    def _scaled(self, sink):
        """The sink with this block's constant: the product that uses it adds m times its result."""
        if sink is not None:
            sink.scale = self.residual_scale
        return sink

    def _leaves(self, y):
        """A part's output on its way to the residual: already summed by the part's last
        product (`ops.NormPending`), or still to be added times the constant."""
        from ..kernels import ops
        return y if isinstance(y, ops.NormPending) else ops.ScaledDelta(y, self.residual_scale)

    def forward(self, ctx, resid: torch.Tensor, delta, cache):
        after_block = getattr(ctx, "reads_after_part", None)
        sink_after_block = self._scaled(getattr(ctx, "residual_sink", None))
        normed = self.mixer_norm.add_norm(resid, delta)
        if self.feed_forward is None:
            ctx.reads_after_part, ctx.residual_sink = after_block, sink_after_block
            return self._leaves(self.mixer.forward(ctx, normed, cache))
        ctx.reads_after_part = first_weight_of(self.feed_forward)
        ctx.residual_sink = self._scaled(_sink_for(self.feed_forward_norm, self.feed_forward, resid))
        mixed = self._leaves(self.mixer.forward(ctx, normed, cache))
        normed = self.feed_forward_norm.add_norm(resid, mixed)
        ctx.reads_after_part, ctx.residual_sink = after_block, sink_after_block
        return self._leaves(self.feed_forward.forward(ctx, normed))


@register_block("parallel_residual")
class ParallelResidualBlock(Part):
    """One norm whose output both parts read, their results joining the stream as one sum:

        h = norm(x);  x <- x + m * (mixer(h) + feed_forward(h))

    (without a feed-forward: x <- x + m * mixer(h)). The sum of the two results is
    made in 32-bit where the second of them is finished: a feed-forward that says
    `accepts_addend = True` takes the mixer's rows as `addend` and adds them where it
    writes its own (the routed experts' combine does); otherwise a kernel adds them.
    The block's output leaves as an `ops.ScaledDelta`, and the norm that runs next
    makes `x += m * y` in its own pass over the row."""
    replay_safe = True

    def __init__(self, layer: LayerSpec, residual_scale: float = 1.0, *, dtype: torch.dtype,
                 device: torch.device):
        ctx = dict(dtype=dtype, device=device)
        self.prefix = layer.prefix
        self.names = dict(layer.names)
        self.residual_scale = float(residual_scale)
        self.mixer = MIXERS.build(layer.mixer, **ctx)
        self.mixer_norm = NORMS.build(layer.mixer_norm, **ctx)
        self.feed_forward = None
        if layer.feed_forward is not None:
            self.feed_forward = FEED_FORWARDS.build(layer.feed_forward, **ctx)

    def _named(self):
        p, n = self.prefix, self.names
        named = [(self.mixer_norm, f"{p}.{n['mixer_norm']}"), (self.mixer, f"{p}.{n['mixer']}")]
        if self.feed_forward is not None:
            named.append((self.feed_forward, f"{p}.{n['feed_forward']}"))
        return named

    def parts(self):
        return [part for part, _ in self._named()]

    def expected_tensors(self, prefix: str = "") -> Dict[str, ExpectedTensor]:
        out: Dict[str, ExpectedTensor] = {}
        for part, name in self._named():
            out.update(part.expected_tensors(name))
        return out

    def load(self, prefix: str, fetch: Fetch) -> None:
        for part, name in self._named():
            part.load(name, fetch)

    def cache_request(self):
        return self.mixer.cache_request()

    def first_weight(self):
        return first_weight_of(self.mixer)

    def forward(self, ctx, resid: torch.Tensor, delta, cache):
        from ..kernels import ops
        after_block = getattr(ctx, "reads_after_part", None)
        # the sum of two parts is not one product's epilogue: no norm is handed forward
        ctx.residual_sink = None
        normed = self.mixer_norm.add_norm(resid, delta)
        if self.feed_forward is None:
            ctx.reads_after_part = after_block
            return ops.ScaledDelta(_as_float_rows(self.mixer.forward(ctx, normed, cache)),
                                   self.residual_scale)
        ctx.reads_after_part = first_weight_of(self.feed_forward)
        mixed = _as_float_rows(self.mixer.forward(ctx, normed, cache))
        ctx.reads_after_part = after_block
        if getattr(self.feed_forward, "accepts_addend", False):
            both = self.feed_forward.forward(ctx, normed, addend=mixed)
        else:
            both = ops.add_into(_as_float_rows(self.feed_forward.forward(ctx, normed)), mixed)
        return ops.ScaledDelta(both, self.residual_scale)


def _as_float_rows(y):
    """A part's output as one float32 tensor (planes summed; 16-bit rows widened)."""
    from ..kernels import ops
    y = _as_rows(y)
    if y.dtype != torch.float32:
        wide = torch.empty(y.shape, dtype=torch.float32, device=y.device)
        y = ops.cast(y, wide)
    return y
