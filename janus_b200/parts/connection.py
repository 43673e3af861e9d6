"""Hyper-connections: a layer keeps S copies x_1 .. x_S of the residual stream per token
instead of one.  A sublayer reads u = sum_s a[s] x_s (normed before it enters the sublayer)
and, once it has produced y, every stream is rewritten from the old ones at once:
x_t <- sum_s M[s, t] x_s + b[t] y, with M indexed [from, to].  With S = 1, a = b = M = 1 this is the
plain residual sum.  The weights a, b, M are float32 on the device whatever the engine dtype;
the sums are made in float32.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..kernels import ops
from .base import Connection, register_part


class HyperConnection(Connection):
    def __init__(self, streams: int, width: int, dtype: torch.dtype = torch.float32,
                 device: torch.device = torch.device("cuda")):
        if streams < 1:
            raise ValueError(f"a connection needs at least one stream, got {streams}")
        self.streams, self.width = int(streams), int(width)
        self.dtype, self.device = dtype, device
        self.a: Optional[torch.Tensor] = None
        self.b: Optional[torch.Tensor] = None
        self.mix: Optional[torch.Tensor] = None

    def weight_shapes(self):
        return {"into": ((self.streams,), "ones"), "out": ((self.streams,), "ones"),
                "mix": ((self.streams, self.streams), "eye")}

    def load(self, into: torch.Tensor, out: torch.Tensor, mix: torch.Tensor) -> None:
        S = self.streams
        for name, t, shape in (("into", into, (S,)), ("out", out, (S,)), ("mix", mix, (S, S))):
            if tuple(t.shape) != shape:
                raise ValueError(f"connection weight '{name}' of shape {tuple(t.shape)} does not fit {shape}")
        self.a = into.to(device=self.device, dtype=torch.float32).contiguous()
        self.b = out.to(device=self.device, dtype=torch.float32).contiguous()
        self.mix = mix.to(device=self.device, dtype=torch.float32).contiguous()

    def read(self, residual: torch.Tensor, norm, out: torch.Tensor, clear: Optional[torch.Tensor] = None,
             clear2: Optional[torch.Tensor] = None) -> None:
        """out = norm(sum_s a[s] x_s); `clear` ([T, width] float32, the sublayer's target) is zeroed on the way, and
        `clear2` (a scratch tensor that the sublayer wants zeroed) too."""
        norm.forward_streams(residual, self.streams, self.a, out, clear=clear, clear2=clear2)

    def write(self, residual: torch.Tensor, y: torch.Tensor) -> None:
        ops.streams_mix(residual, y, self.mix, self.b, self.streams)

    def write_then_read(self, residual: torch.Tensor, y: torch.Tensor, then: "HyperConnection", norm,
                        out: torch.Tensor, clear2: Optional[torch.Tensor] = None) -> None:
        """This sublayer's write and the next sublayer's read (`then`, with its norm) in one launch; y is
        left zeroed for the next sublayer to add into."""
        gamma, eps = getattr(norm, "gamma", None), getattr(norm, "eps", None)
        if isinstance(then, HyperConnection) and then.streams == self.streams and gamma is not None and eps is not None:
            ops.streams_mix_rmsnorm(residual, y, self.mix, self.b, then.a, self.streams, gamma, eps, out, clear2)
        else:
            self.write(residual, y)
            then.read(residual, norm, out, clear=y, clear2=clear2)


register_part("connection", "hyper_connection", HyperConnection)


class LayerScale(Connection):
    """One residual stream; what a sublayer produced is multiplied feature by feature by a weight before it joins:
    x <- x + scale * y.  The sublayer reads norm(x).  The sum is made in float32; a sublayer's write and the next
    sublayer's read are one launch where the norm can do both (`join`)."""

    def __init__(self, width: int, dtype: torch.dtype = torch.float32, device: torch.device = torch.device("cuda")):
        self.width = int(width)
        self.dtype, self.device = dtype, device
        self.scale: Optional[torch.Tensor] = None

    def weight_shapes(self):
        return {"scale": ((self.width,), "ones")}

    def load(self, scale: torch.Tensor) -> None:
        if tuple(scale.shape) != (self.width,):
            raise ValueError(f"layer scale of shape {tuple(scale.shape)} does not fit ({self.width},)")
        self.scale = scale.to(device=self.device, dtype=torch.float32).contiguous()

    def read(self, residual: torch.Tensor, norm, out: torch.Tensor, clear: Optional[torch.Tensor] = None,
             clear2: Optional[torch.Tensor] = None) -> None:
        if clear2 is not None and not hasattr(norm, "join"):
            ops.zero_f32(clear2)
            clear2 = None
        if clear is not None and clear.numel() % 4:
            clear.zero_()
            clear = None
        if clear2 is not None:
            norm.forward(residual, out, clear=clear, clear2=clear2)
        else:
            norm.forward(residual, out, clear=clear)

    def write(self, residual: torch.Tensor, y: torch.Tensor) -> None:
        ops.join_norm(residual, ya=y, scale=self.scale)

    def write_then_read(self, residual: torch.Tensor, y: torch.Tensor, then: "Connection", norm,
                        out: torch.Tensor, clear2: Optional[torch.Tensor] = None) -> None:
        """This sublayer's write and the next sublayer's read in one launch; y is left zeroed."""
        if isinstance(then, LayerScale) and hasattr(norm, "join"):
            norm.join(residual, y, self.scale, out, clear2=clear2)
        else:
            self.write(residual, y)
            then.read(residual, norm, out, clear=None, clear2=clear2)      # y is zero already


register_part("connection", "layer_scale", LayerScale)
