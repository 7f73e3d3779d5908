"""Gated feed-forward: down(act(gate(x)) * up(x)), no biases. With act = SiLU
it is the reference's SwiGLU (src/models/llama/mlp.rs:49-58; SiLU is
x / (1 + exp(-x)) in 32-bit, src/nn/activation.rs:18-27); `activation =
"gelu_tanh"` makes it 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))).
gate and up are one fused product. `dense_mlp` is the form without a gate.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..kernels import ops
from ..weights.loader import ExpectedTensor
from .base import Fetch, Part, register_feed_forward
from .linear import Linear, matmul_nt


@register_feed_forward("swiglu")
class SwiGLU(Part):
    replay_safe = True  # forward reads nothing of the step on the host
    accepts_row_scaled = True  # the gate/up product applies a deferred norm's row scale

    def __init__(self, hidden_size: int, intermediate_size: int, *, dtype: torch.dtype,
                 device: torch.device, names=("gate_proj", "up_proj", "down_proj"),
                 suffix: str = ".weight", activation: str = "silu"):
        if activation not in ops.GLU_ACTIVATIONS:
            raise ValueError(f"activation {activation!r}; known: {sorted(ops.GLU_ACTIVATIONS)}")
        self.activation = activation
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size
        self.dtype, self.device = dtype, device
        self.names, self.suffix = tuple(names), suffix  # the three projections in the files
        self.gate_up: torch.Tensor = None  # [2I, H]: row 2i is gate i, row 2i+1 is up i
        self.down = Linear(intermediate_size, [(self.names[2], hidden_size)], dtype=dtype,
                           device=device, suffix=suffix)

    def expected_tensors(self, prefix: str) -> Dict[str, ExpectedTensor]:
        shape = (self.intermediate_size, self.hidden_size)
        return {f"{prefix}.{self.names[0]}{self.suffix}": ExpectedTensor(shape),
                f"{prefix}.{self.names[1]}{self.suffix}": ExpectedTensor(shape),
                **self.down.expected_tensors(prefix)}

    def load(self, prefix: str, fetch: Fetch) -> None:
        gate = fetch(f"{prefix}.{self.names[0]}{self.suffix}")
        up = fetch(f"{prefix}.{self.names[1]}{self.suffix}")
        if gate.dtype != up.dtype:
            raise ops.KernelError(f"{prefix}: gate and up projections are stored in different dtypes")
        # rows interleaved so that a product tile holds matching gate / up pairs
        self.gate_up = torch.stack([gate, up], 1).reshape(2 * self.intermediate_size,
                                                          self.hidden_size).contiguous()
        self.down.load(prefix, fetch)

    def first_weight(self):
        return self.gate_up

    def hidden(self, x) -> torch.Tensor:
        """act(gate(x)) * up(x) in the activation type: what the down projection reads."""
        hidden = torch.empty((x.shape[0], self.intermediate_size), dtype=x.dtype, device=x.device)
        if x.dtype == torch.bfloat16 and self.gate_up.dtype == torch.bfloat16:
            ops.gemm_bf16_silu_mul(x, self.gate_up, hidden,  # activation in the epilogue
                                   then_reads=self.down.weight, act=self.activation)
        else:
            ops.silu_mul(matmul_nt(ops.plain(x), self.gate_up), hidden, interleaved=True,
                         act=self.activation)
        return hidden

    def forward(self, ctx, x):
        hidden = self.hidden(x)
        return self.down.forward(hidden, allow_planes=True,
                                 then_reads=getattr(ctx, "reads_after_part", None),
                                 residual=getattr(ctx, "residual_sink", None))


UNARY_ACTIVATIONS = ("relu2",)


@register_feed_forward("dense_mlp")
class DenseMLP(Part):
    """The feed-forward without a gate: down(act(up(x))), no biases; `activation =
    "relu2"` is the square of relu, max(z, 0)^2. The up product is accumulated in
    32-bit and the activation is taken of those values before they are rounded
    for the down product."""
    replay_safe = True

    def __init__(self, hidden_size: int, intermediate_size: int, *, dtype: torch.dtype,
                 device: torch.device, names=("up", "down"), suffix: str = "",
                 activation: str = "relu2"):
        if activation not in UNARY_ACTIVATIONS:
            raise ValueError(f"activation {activation!r}; known: {UNARY_ACTIVATIONS}")
        self.activation = activation
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size
        self.dtype, self.device = dtype, device
        self.up = Linear(hidden_size, [(names[0], intermediate_size)], dtype=dtype, device=device,
                         suffix=suffix)
        self.down = Linear(intermediate_size, [(names[1], hidden_size)], dtype=dtype,
                           device=device, suffix=suffix)

    def expected_tensors(self, prefix: str) -> Dict[str, ExpectedTensor]:
        return {**self.up.expected_tensors(prefix), **self.down.expected_tensors(prefix)}

    def load(self, prefix: str, fetch: Fetch) -> None:
        self.up.load(prefix, fetch)
        self.down.load(prefix, fetch)

    def first_weight(self):
        return self.up.weight

    def forward(self, ctx, x):
        x = ops.plain(x)
        hidden = torch.empty((x.shape[0], self.intermediate_size), dtype=x.dtype, device=x.device)
        ops.gemm_bf16_unary(x, self.up.weight, hidden, self.activation,
                            then_reads=self.down.weight)
        return self.down.forward(hidden, allow_planes=True,
                                 then_reads=getattr(ctx, "reads_after_part", None))
