"""RMSNorm: y = x / sqrt(mean(x^2) + eps) * gamma, statistics in float32
(crates/janus-engine/src/compute/shaders/activations.wgsl:81-133).  The weight
keeps the dtype it was stored in (the reference keeps 1-D tensors in f32,
crates/janus-engine/src/compute/engine.rs:448-470)."""
from __future__ import annotations

from typing import Optional

import torch

from ..kernels import ops
from .base import Norm, register_part


class RMSNorm(Norm):
    def __init__(self, width: int, eps: float, dtype: torch.dtype, device: torch.device):
        self.width, self.eps = int(width), float(eps)
        self.dtype, self.device = dtype, device
        self.gamma: Optional[torch.Tensor] = None

    def weight_shapes(self):
        return {"gamma": ((self.width,), "ones")}

    def load(self, gamma: torch.Tensor) -> None:
        if tuple(gamma.shape) != (self.width,):
            raise ValueError(f"norm weight of shape {tuple(gamma.shape)} does not fit ({self.width},)")
        if self.dtype == torch.float32:
            gamma = gamma.to(torch.float32)
        self.gamma = gamma.to(self.device).contiguous()

    def forward(self, x: torch.Tensor, out: torch.Tensor, row_index: Optional[torch.Tensor] = None,
                clear: Optional[torch.Tensor] = None) -> None:
        """`clear`: a float32 scratch tensor of the part that runs next, set to zero by the same launch."""
        ops.rmsnorm(x, self.gamma, self.eps, out, row_index, clear)

    def add_normed(self, y: Optional[torch.Tensor], residual: torch.Tensor, mult: float,
                   x_out: Optional[torch.Tensor] = None, clear: Optional[torch.Tensor] = None,
                   clear2: Optional[torch.Tensor] = None) -> None:
        """residual += mult * norm(y), y <- 0, x_out = residual in its dtype (y None: only that), one launch."""
        ops.sublayer_norm_add(y, self.gamma, self.eps, mult, residual, x_out, clear, clear2)

    def forward_streams(self, x: torch.Tensor, streams: int, weights: Optional[torch.Tensor], out: torch.Tensor,
                        row_index: Optional[torch.Tensor] = None, clear: Optional[torch.Tensor] = None,
                        clear2: Optional[torch.Tensor] = None) -> None:
        """The norm of the weighted sum of `streams` residual streams, summed and normed in one launch."""
        ops.streams_rmsnorm(x, streams, weights, self.gamma, self.eps, out, row_index, clear, clear2)


register_part("norm", "rms_norm", RMSNorm)


class LayerNorm(Norm):
    """y = (x - mean(x)) / sqrt(mean((x - mean(x))^2) + eps) * gamma: a layer norm with a weight and no bias,
    statistics in float32 (the mean first, then the mean of the squared deviations)."""

    CENTER = True

    def __init__(self, width: int, eps: float, dtype: torch.dtype, device: torch.device):
        self.width, self.eps = int(width), float(eps)
        self.dtype, self.device = dtype, device
        self.gamma: Optional[torch.Tensor] = None

    def weight_shapes(self):
        return {"gamma": ((self.width,), "ones")}

    def load(self, gamma: torch.Tensor) -> None:
        if tuple(gamma.shape) != (self.width,):
            raise ValueError(f"norm weight of shape {tuple(gamma.shape)} does not fit ({self.width},)")
        self.gamma = gamma.to(device=self.device, dtype=torch.float32).contiguous()

    def forward(self, x: torch.Tensor, out: torch.Tensor, row_index: Optional[torch.Tensor] = None,
                clear: Optional[torch.Tensor] = None, clear2: Optional[torch.Tensor] = None) -> None:
        ops.join_norm(x, gamma=self.gamma, eps=self.eps, center=self.CENTER, x_out=out, row_index=row_index,
                      clear=clear, clear2=clear2)

    def join(self, residual: torch.Tensor, y: torch.Tensor, scale: Optional[torch.Tensor], out: torch.Tensor,
             clear2: Optional[torch.Tensor] = None) -> None:
        """residual += scale * y (per feature; None: y itself), y <- 0, out = norm(residual), in one launch."""
        ops.join_norm(residual, ya=y, scale=scale, gamma=self.gamma, eps=self.eps, center=self.CENTER, x_out=out,
                      clear2=clear2)


register_part("norm", "layer_norm", LayerNorm)
