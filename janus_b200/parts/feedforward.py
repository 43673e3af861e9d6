"""Dense SwiGLU feed-forward: down( silu(gate(x)) * up(x) ), added into the
residual stream (crates/janus-engine/src/model/block.rs:383-455; SiLU as
x/(1+exp(-x)), crates/janus-engine/src/compute/shaders/activations.wgsl:20-35)."""
from __future__ import annotations

import torch

from .base import FeedForward, register_part
from .linear import GatedLinear, Linear


class SwiGLUFeedForward(FeedForward):
    """`pad_width`: widths that are no multiple of 8 run on zero-padded operands in bfloat16 instead of being refused."""

    def __init__(self, hidden_size: int, intermediate_size: int, pad_width: bool = False,
                 dtype: torch.dtype = torch.bfloat16, device: torch.device = torch.device("cuda")):
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size
        self.dtype, self.device = dtype, device
        self.gate_up = GatedLinear(hidden_size, intermediate_size, dtype, device, pad_width=pad_width)
        self.down = Linear(intermediate_size, hidden_size, dtype, device, name="down", pad_width=pad_width)

    def weight_shapes(self):
        return {"gate": ((self.intermediate_size, self.hidden_size), "normal"),
                "up": ((self.intermediate_size, self.hidden_size), "normal"),
                "down": ((self.hidden_size, self.intermediate_size), "normal")}

    def load(self, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor) -> None:
        self.gate_up.load(gate, up)
        self.down.load([down])

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx) -> None:
        act = ctx.workspace.get("ffn_act", (x.shape[0], self.intermediate_size), self.dtype)
        self.gate_up.forward(x, act, ctx)
        self.down.forward_add(act, residual)


class ClampedGLUFeedForward(FeedForward):
    """down( g * sigmoid(alpha g) * (u + 1) ) with g = min(gate(x), limit) and u = clamp(up(x), -limit, limit),
    added into the residual stream.  The gated product is the SwiGLU one with another activation in the same
    epilogue (`GatedLinear` with a limit)."""

    def __init__(self, hidden_size: int, intermediate_size: int, limit: float, alpha: float = 1.702,
                 dtype: torch.dtype = torch.bfloat16, device: torch.device = torch.device("cuda")):
        if not limit > 0.0:
            raise ValueError(f"the clamp's limit must be positive, got {limit}")
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size
        self.limit, self.alpha = float(limit), float(alpha)
        self.dtype, self.device = dtype, device
        # widths that are no multiple of 8 run on zero-padded operands
        self.gate_up = GatedLinear(hidden_size, intermediate_size, dtype, device, limit=self.limit, alpha=self.alpha,
                                   pad_width=True)
        self.down = Linear(intermediate_size, hidden_size, dtype, device, name="down", pad_width=True)

    def weight_shapes(self):
        return {"gate": ((self.intermediate_size, self.hidden_size), "normal"),
                "up": ((self.intermediate_size, self.hidden_size), "normal"),
                "down": ((self.hidden_size, self.intermediate_size), "normal")}

    def load(self, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor) -> None:
        self.gate_up.load(gate, up)
        self.down.load([down])

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx) -> None:
        act = ctx.workspace.get("ffn_act", (x.shape[0], self.intermediate_size), self.dtype)
        self.gate_up.forward(x, act, ctx)
        self.down.forward_add(act, residual)


class GeluGLUFeedForward(FeedForward):
    """down( gelu_tanh(gate(x)) * up(x) ), gelu_tanh(z) = 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))), added into
    the residual stream.  The gated product is the SwiGLU one with another activation in the same epilogue."""

    def __init__(self, hidden_size: int, intermediate_size: int,
                 dtype: torch.dtype = torch.bfloat16, device: torch.device = torch.device("cuda")):
        from ..kernels import ops
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size
        self.dtype, self.device = dtype, device
        self.gate_up = GatedLinear(hidden_size, intermediate_size, dtype, device, limit=ops.GELU_TANH_GATE,
                                   pad_width=True)
        self.down = Linear(intermediate_size, hidden_size, dtype, device, name="down", pad_width=True)

    def weight_shapes(self):
        return {"gate": ((self.intermediate_size, self.hidden_size), "normal"),
                "up": ((self.intermediate_size, self.hidden_size), "normal"),
                "down": ((self.hidden_size, self.intermediate_size), "normal")}

    def load(self, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor) -> None:
        self.gate_up.load(gate, up)
        self.down.load([down])

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx) -> None:
        act = ctx.workspace.get("ffn_act", (x.shape[0], self.intermediate_size), self.dtype)
        self.gate_up.forward(x, act, ctx)
        self.down.forward_add(act, residual)


register_part("feed_forward", "swiglu", SwiGLUFeedForward)
register_part("feed_forward", "gelu_glu", GeluGLUFeedForward)
register_part("feed_forward", "clamped_glu", ClampedGLUFeedForward)
