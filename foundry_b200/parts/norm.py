"""RMS normalisation, fused with the residual sum that precedes it.

y = x * 1/sqrt(mean(x^2) + eps) * w, the statistics in 32-bit
(src/nn/norm.rs:31-51: square, sum, * 1/H, + eps, sqrt, reciprocal). The
reference rounds x*r to 16 bits before the weight multiply; here the product
is rounded once, at the end. The weight is held in float32 (exact for a
bfloat16 file; a 32-bit file stays as stored).
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..kernels import ops
from ..weights.loader import ExpectedTensor
from .base import Fetch, Part, register_norm


@register_norm("rms_norm")
class RMSNorm(Part):
    replay_safe = True  # forward reads nothing of the step on the host

    def __init__(self, size: int, eps: float, weight_suffix: str = ".weight", *,
                 dtype: torch.dtype, device: torch.device):
        self.size, self.eps = size, float(eps)
        self.weight_suffix = weight_suffix  # the tensor is `<prefix><weight_suffix>`
        self.dtype, self.device = dtype, device
        self.weight: Optional[torch.Tensor] = None

    def expected_tensors(self, prefix: str) -> Dict[str, ExpectedTensor]:
        return {f"{prefix}{self.weight_suffix}": ExpectedTensor((self.size,))}

    def load(self, prefix: str, fetch: Fetch) -> None:
        self.weight = fetch(f"{prefix}{self.weight_suffix}").to(torch.float32).contiguous()

    def sink(self, resid: torch.Tensor) -> Optional[ops.ResidualSink]:
        """What the projection in front of this norm needs to make the sum and
        prepare the norm itself (bfloat16 steps only)."""
        if self.dtype != torch.bfloat16 or self.weight is None:
            return None
        return ops.ResidualSink(resid, self.weight, self.eps)

    def add_norm(self, resid: torch.Tensor, delta, out: Optional[torch.Tensor] = None):
        """resid += delta (a tensor, split-K `ops.Planes`, an `ops.ScaledDelta`, or None); returns
        norm(resid) in the activation dtype. A delta that a projection made
        with this norm's `sink` comes back as an `ops.RowScaled`."""
        if isinstance(delta, ops.NormPending):
            return ops.add_rmsnorm(resid, delta, self.weight, self.eps, None)
        if out is None:
            out = torch.empty(resid.shape, dtype=self.dtype, device=resid.device)
        scale = 1.0
        if isinstance(delta, ops.ScaledDelta):  # resid += scale * values
            delta, scale = delta.values, delta.scale
        return ops.add_rmsnorm(resid, delta, self.weight, self.eps, out, delta_scale=scale)


@register_norm("layer_norm")
class LayerNorm(Part):
    """(x - mean) / sqrt(mean((x - mean)^2) + eps) * w + b with 32-bit statistics
    (csrc/layernorm.cu). The tensors are `<prefix><weight_suffix>` and
    `<prefix><bias_suffix>`; `bias_suffix = None` is the norm without a bias. Beside normalising a part's input (`add_norm`) it
    may stand behind a part: `pending(y)` says that LN(y) is still to join the
    residual, and the next `add_norm` (or `NormedDelta.settle`) makes that sum in
    the same pass."""
    replay_safe = True

    def __init__(self, size: int, eps: float, weight_suffix: str = ".weight",
                 bias_suffix: Optional[str] = ".bias", *, dtype: torch.dtype,
                 device: torch.device):
        self.size, self.eps = size, float(eps)
        self.weight_suffix, self.bias_suffix = weight_suffix, bias_suffix
        self.dtype, self.device = dtype, device
        self.weight: Optional[torch.Tensor] = None
        self.bias: Optional[torch.Tensor] = None

    def expected_tensors(self, prefix: str) -> Dict[str, ExpectedTensor]:
        out = {f"{prefix}{self.weight_suffix}": ExpectedTensor((self.size,))}
        if self.bias_suffix is not None:
            out[f"{prefix}{self.bias_suffix}"] = ExpectedTensor((self.size,))
        return out

    def load(self, prefix: str, fetch: Fetch) -> None:
        self.weight = fetch(f"{prefix}{self.weight_suffix}").to(torch.float32).contiguous()
        if self.bias_suffix is not None:
            self.bias = fetch(f"{prefix}{self.bias_suffix}").to(torch.float32).contiguous()

    def pending(self, values: torch.Tensor) -> ops.NormedDelta:
        if self.bias is None:
            raise ValueError("a layer norm without a bias cannot stand behind a part")
        return ops.NormedDelta(values, self.weight, self.bias, self.eps)

    def add_norm(self, resid: torch.Tensor, delta, out: Optional[torch.Tensor] = None):
        """resid += delta (None, a tensor, split-K planes, an `ops.ScaledDelta` that joins
        times its constant, an `ops.NormedDelta` whose norm is applied on the way, or an
        `ops.DepthMix`, which also replaces the stream by its weighted sum); returns
        LN(resid) in the activation dtype."""
        mix = None
        if isinstance(delta, ops.DepthMix):  # the stream is a weighted sum over kept streams
            mix, delta = delta, delta.pending
            if delta is not None and delta.eps != self.eps:
                mix, delta = None, mix.settle(resid)
        scale = 1.0
        if isinstance(delta, ops.ScaledDelta):  # resid += scale * values
            delta, scale = delta.values, delta.scale
        if isinstance(delta, ops.Planes):
            delta = delta.sum(torch.float32)
        if delta is not None and not isinstance(delta, ops.NormedDelta):
            delta = ops.NormedDelta(delta, None, None, self.eps, scale)  # a plain sum
        if delta is not None and delta.eps != self.eps:  # one pass takes one eps
            delta = delta.settle(resid)
        if out is None:
            out = torch.empty(resid.shape, dtype=self.dtype, device=resid.device)
        return ops.ln_add_ln(resid, delta, self.weight, self.bias, self.eps, out, mix=mix)
