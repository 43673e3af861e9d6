"""The gated delta rule, a mixer with a matrix state of fixed size per head.

With h the mixer's input: q = Wq h and k = Wk h (kv_heads x dim), v = Wv h (heads x vdim), no biases; head i uses q/k
head floor(i / (heads / kv_heads)).  Each of q, k, v passes a short causal convolution over time per channel (weight
[channels, taps] whose last column meets the current token, zeros before a sequence's start) and SiLU.  q and k are
then made unit vectors per head, x / sqrt(sum(x^2) + 1e-6), and q is multiplied by dim^-1/2.  beta = sigmoid(Wb h)
and the decay g = exp(-exp(A_log) softplus(Wa h + dt_bias)) are one number per head and token.  Per head the state S
(dim x vdim, float32, zero at a sequence's start) follows S <- g S; w = beta (v - S^T k); S <- S + k w^T, and the
head's output is o = S^T q, read after the token's own write.  Each head's o is divided by its root mean square over
vdim (eps inside the root), multiplied by a weight of size vdim that the heads share and by silu(Wg h), and the
concatenated heads are projected by Wo.

The six projections are one stacked product whose float32 accumulators the convolution, the recurrence and the gate
read; the recurrence's state and the convolution's last taps - 1 inputs live side by side in one block of the cache's
fixed-size state area per sequence slot, so prompts, portions of prompts and single tokens all run the same kernels
from whatever the steps before left.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..kernels import ops
from .base import Mixer, StateSpec, register_part
from .linear import Linear

UNIT_EPS = 1e-6      # inside the root of the unit norms of q and k


class GatedDeltaRule(Mixer):
    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, dim: int, vdim: int, conv_taps: int,
                 eps: float, dtype: torch.dtype = torch.bfloat16, device: torch.device = torch.device("cuda")):
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} heads are not a multiple of {num_kv_heads} query/key heads")
        if not 1 <= dim <= 256:
            raise ValueError(f"a key size of {dim} is not supported by the recurrence kernel (1 to 256)")
        if conv_taps < 1:
            raise ValueError(f"the convolution needs at least one tap, got {conv_taps}")
        self.hidden_size, self.nh, self.nkv = int(hidden_size), int(num_heads), int(num_kv_heads)
        self.dim, self.vdim, self.taps, self.eps = int(dim), int(vdim), int(conv_taps), float(eps)
        self.dtype, self.device = dtype, device
        self.qk_width, self.v_width = self.nkv * self.dim, self.nh * self.vdim
        self.channels = 2 * self.qk_width + self.v_width            # what the convolution sees: q, k, v
        self.gate_col = self.channels
        self.b_col = self.gate_col + self.v_width
        self.a_col = self.b_col + self.nh
        self.width = self.a_col + self.nh                           # q, k, v, g, b, a
        self.proj = Linear(hidden_size, self.width, dtype, device, name="qkvgba", pad_width=True)
        self.o = Linear(self.v_width, hidden_size, dtype, device, name="o", pad_width=True)
        # one block of state per slot: the recurrence's [heads, dim, vdim], then the convolution's [taps - 1, channels]
        self.scan_floats = self.nh * self.dim * self.vdim
        self.state_floats = self.scan_floats + (self.taps - 1) * self.channels
        self.conv_w = self.a_log = self.dt_bias = self.norm_weight = None

    def cache_spec(self) -> StateSpec:
        return StateSpec((self.state_floats,))

    def weight_shapes(self):
        H = self.hidden_size
        return {"q": ((self.qk_width, H), "normal"), "k": ((self.qk_width, H), "normal"),
                "v": ((self.v_width, H), "normal"), "g": ((self.v_width, H), "normal"), "b": ((self.nh, H), "normal"),
                "a": ((self.nh, H), "normal"), "q_conv": ((self.qk_width, self.taps), "normal"),
                "k_conv": ((self.qk_width, self.taps), "normal"), "v_conv": ((self.v_width, self.taps), "normal"),
                "A_log": ((self.nh,), "normal"), "dt_bias": ((self.nh,), "normal"), "norm": ((self.vdim,), "ones"),
                "o": ((H, self.v_width), "normal")}

    def load(self, q, k, v, g, b, a, q_conv, k_conv, v_conv, A_log, dt_bias, norm, o) -> None:
        self.proj.load([q, k, v, g, b, a])
        self.o.load([o])

        def f32(name, t, shape):
            if tuple(t.shape) != shape:
                raise ValueError(f"'{name}' of shape {tuple(t.shape)} does not fit {shape}")
            return t.to(device=self.device, dtype=torch.float32).contiguous()

        conv = torch.cat([t.to(torch.float32) for t in (q_conv, k_conv, v_conv)], dim=0)
        self.conv_w = f32("conv", conv, (self.channels, self.taps))
        self.a_log, self.dt_bias = f32("A_log", A_log, (self.nh,)), f32("dt_bias", dt_bias, (self.nh,))
        self.norm_weight = f32("norm", norm, (self.vdim,))

    def scratch_to_clear(self, ctx, tokens: int, writes_cache: bool = True) -> Optional[torch.Tensor]:
        """The projection's float32 buffer, if this step's product adds slices of K into it (decode-sized steps):
        the launch before this mixer clears it in passing."""
        if not self.proj.meets_by_adds(tokens, torch.float32):
            return None
        buf = ctx.workspace.get("delta_proj", (tokens, self.width), torch.float32)
        return buf if buf.numel() % 4 == 0 else None

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx, cache_view, writes_cache: bool = True,
                scratch_cleared: bool = False) -> None:
        if not writes_cache:
            raise ValueError("a delta-rule mixer cannot read another place's state: its state is its own")
        T = x.shape[0]
        ws = ctx.workspace
        state = cache_view.state                                      # float32 [slots, state_floats]
        proj = ws.get("delta_proj", (T, self.width), torch.float32)
        self.proj.forward(x, proj, y_is_zero=scratch_cleared)
        conv = ws.get("delta_conv", (T, self.channels), torch.float32)
        ops.causal_conv_silu(proj, 0, self.channels, self.conv_w, None, self.taps, state, self.scan_floats,
                             ctx.token_seq, ctx.q_start, ctx.seq_slot, conv, ctx.n_seqs, single_tokens=ctx.is_decode)
        o = ws.get("delta_o", (T, self.v_width), torch.float32)
        ops.delta_rule(conv, 0, self.qk_width, 2 * self.qk_width, proj, self.b_col, self.a_col, self.a_log,
                       self.dt_bias, UNIT_EPS, o, state, 0, ctx.q_start, ctx.seq_slot, ctx.n_seqs, self.nh, self.nkv,
                       self.dim, self.vdim)
        gated = ws.get("delta_gated", (T, self.v_width), self.dtype)
        ops.head_norm_gate(o, proj[:, self.gate_col: self.gate_col + self.v_width], self.norm_weight, self.eps, gated,
                           self.nh, self.vdim)
        self.o.forward_add(gated, residual)


register_part("mixer", "gated_delta_rule", GatedDeltaRule)
