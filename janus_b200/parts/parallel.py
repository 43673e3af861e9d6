"""Two mixers side by side that read the same input: the sublayer's output is a multiple of the sum of their
outputs, each first divided by its root mean square over the model width (eps inside the root) and multiplied by a
weight of its own:  y = mult (a / rms(a) * wa + b / rms(b) * wb), mult = 1/2 for the mean of the two.  With
`branch_norm` off the branches join as they are, each with a factor of its own:  y = left_mult a + right_mult b,
and the mixer has no tensors besides its branches'.

The branches are registered mixers named by `PartSpec`s (parameters `left` and `right`, their tensors under the
parameter names `left.<name>` and `right.<name>`); at most one of them may keep keys and values and at most one a
state of fixed size, so that a place of the cache serves both.  Each adds its output into a zeroed float32 buffer of
its own; one launch norms, weighs and adds both into the sublayer's output and leaves the buffers zeroed.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..kernels import ops
from .base import Mixer, PartSpec, make_part, register_part, split_cache_spec


class ParallelMixers(Mixer):
    def __init__(self, hidden_size: int, left: PartSpec, right: PartSpec, eps: float, mult: float = 0.5,
                 branch_norm: bool = True, left_mult: Optional[float] = None, right_mult: Optional[float] = None,
                 dtype: torch.dtype = torch.bfloat16, device: torch.device = torch.device("cuda")):
        self.hidden_size, self.eps, self.mult = int(hidden_size), float(eps), float(mult)
        self.branch_norm = bool(branch_norm)
        self.left_mult = self.mult if left_mult is None else float(left_mult)
        self.right_mult = self.mult if right_mult is None else float(right_mult)
        self.dtype, self.device = dtype, device
        self.branches = {"left": make_part("mixer", left, dtype, device),
                         "right": make_part("mixer", right, dtype, device)}
        specs = [split_cache_spec(b.cache_spec()) for b in self.branches.values()]
        if sum(kv is not None for kv, _ in specs) > 1 or sum(st is not None for _, st in specs) > 1:
            raise ValueError("of two mixers side by side at most one may keep keys and values and at most one a state")
        self.w = {"left": None, "right": None}

    def cache_spec(self):
        items = []
        for b in self.branches.values():
            items += [s for s in split_cache_spec(b.cache_spec()) if s is not None]
        return None if not items else items[0] if len(items) == 1 else tuple(items)

    def limit_positions(self, n: int) -> None:
        for b in self.branches.values():
            limit = getattr(b, "limit_positions", None)
            if limit is not None:
                limit(n)

    def weight_shapes(self):
        shapes = {}
        if self.branch_norm:
            shapes = {"left_out": ((self.hidden_size,), "ones"), "right_out": ((self.hidden_size,), "ones")}
        for side, b in self.branches.items():
            shapes.update({f"{side}.{name}": v for name, v in b.weight_shapes().items()})
        return shapes

    def load(self, left_out: Optional[torch.Tensor] = None, right_out: Optional[torch.Tensor] = None,
             **tensors: torch.Tensor) -> None:
        for side, t in (("left", left_out), ("right", right_out)):
            if self.branch_norm:
                if t is None or tuple(t.shape) != (self.hidden_size,):
                    raise ValueError(f"branch weight of shape {None if t is None else tuple(t.shape)} does not fit "
                                     f"({self.hidden_size},)")
                self.w[side] = t.to(device=self.device, dtype=torch.float32).contiguous()
            elif t is not None:
                raise TypeError("mixers side by side without branch norms take no branch weights")
            self.branches[side].load(**{n[len(side) + 1:]: v for n, v in tensors.items() if n.startswith(side + ".")})

    def _buffers(self, ctx, tokens: int) -> torch.Tensor:
        return ctx.workspace.get("parallel_branches", (2, tokens, self.hidden_size), torch.float32)

    def scratch_to_clear(self, ctx, tokens: int, writes_cache: bool = True) -> Optional[torch.Tensor]:
        """The branches' buffers: the launch before this mixer zeroes them in passing."""
        buf = self._buffers(ctx, tokens)
        return buf if buf.numel() % 4 == 0 else None

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx, cache_view, writes_cache: bool = True,
                scratch_cleared: bool = False) -> None:
        buf = self._buffers(ctx, x.shape[0])
        if not scratch_cleared:
            buf.zero_()
        for i, b in enumerate(self.branches.values()):
            b.forward(x, buf[i], ctx, cache_view, writes_cache)
        ops.join_norm(residual, ya=buf[0], yb=buf[1], wa=self.w["left"], wb=self.w["right"], mult=self.left_mult,
                      mult_b=self.right_mult, eps=self.eps)


register_part("mixer", "parallel", ParallelMixers)
