"""Linear attention with a matrix state per head whose gates depend on the token: two mixers that share one recurrence
kernel (`ops.gated_linear_scan`), S_t = diag(a_t) S_(t-1) + b_t k_t v_t^T, o_t = S_t^T q_t.

`gated_linear_attention` (a decay per key channel).  With h the mixer's input: q = Wq h * dim^-1/2, k = Wk h
(heads x dim), v = Wv h (heads x vdim); the decays a_t = sigmoid(z)^(1/tau) with z = A2 (A1 h) + bias, a low-rank
projection laid out heads x dim; b_t = 1.  Each head's o is divided by its root mean square over vdim (eps inside the
root) and multiplied by a weight of size vdim that the heads share; the concatenated heads are multiplied by
silu(Wg h) and projected by Wo.

`matrix_memory` (the matrix memory of xLSTM, exponential gates).  q, k, v as above.  Per head and token a log input
gate i = cap tanh((Wi h + bi) / cap) and a log forget gate f = logsigmoid(cap tanh((Wf h + bf) / cap)); with a running
maximum m_t = max(f + m_(t-1), i) that starts at 0:  a_t = exp(f + m_(t-1) - m_t), b_t = exp(i - m_t); a normalizer
n_t = a_t n_(t-1) + b_t k_t walks along, and the head's output is S_t^T q / (max(|n_t . q|, exp(-m_t)) + 1e-6).  Each
head's o is divided by its root mean square (eps inside the root); the concatenated heads are multiplied by a weight
of all heads' size and by sigmoid(Wg h), and projected by Wo.

The projections are one stacked product whose float32 accumulators the gates, the recurrence and the output gate
read; everything that enters the state is float32.  The state (and the normalizer and the running maxima) lives in
the cache's fixed-size state area, one block per sequence slot, zero when a slot is taken, so prompts, portions of
prompts and single tokens all run the same kernels from whatever the steps before left.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..kernels import ops
from .base import Mixer, StateSpec, register_part
from .linear import Linear


def _f32(name: str, t: torch.Tensor, shape, device) -> torch.Tensor:
    if tuple(t.shape) != tuple(shape):
        raise ValueError(f"'{name}' of shape {tuple(t.shape)} does not fit {tuple(shape)}")
    return t.to(device=device, dtype=torch.float32).contiguous()


class _GatedLinearBase(Mixer):
    """What the two mixers share: sizes, the stacked projection, the output product and the scratch to clear."""

    PROJ = "gated_linear_proj"

    def __init__(self, hidden_size: int, num_heads: int, dim: int, vdim: int, eps: float, extra_rows: int,
                 dtype: torch.dtype, device: torch.device, name: str):
        if not 1 <= dim <= 256:
            raise ValueError(f"a key size of {dim} is not supported by the recurrence kernel (1 to 256)")
        self.hidden_size, self.nh, self.dim, self.vdim = int(hidden_size), int(num_heads), int(dim), int(vdim)
        self.eps = float(eps)
        self.dtype, self.device = dtype, device
        self.qk_width, self.v_width = self.nh * self.dim, self.nh * self.vdim
        self.k_col, self.v_col = self.qk_width, 2 * self.qk_width
        self.gate_col = self.v_col + self.v_width
        self.extra_col = self.gate_col + self.v_width
        self.width = self.extra_col + int(extra_rows)               # q, k, v, g, then the gates' own rows
        self.proj = Linear(hidden_size, self.width, dtype, device, name=name, pad_width=True)
        self.o = Linear(self.v_width, hidden_size, dtype, device, name="o", pad_width=True)
        self.q_scale = float(self.dim) ** -0.5

    def scratch_to_clear(self, ctx, tokens: int, writes_cache: bool = True) -> Optional[torch.Tensor]:
        """The projections' float32 buffer, if this step's product adds slices of K into it (decode-sized steps):
        the launch before this mixer clears it in passing."""
        if not self.proj.meets_by_adds(tokens, torch.float32):
            return None
        buf = ctx.workspace.get(self.PROJ, (tokens, self.width), torch.float32)
        return buf if buf.numel() % 4 == 0 else None


class GatedLinearAttention(_GatedLinearBase):
    PROJ = "gla_proj"

    def __init__(self, hidden_size: int, num_heads: int, dim: int, vdim: int, rank: int, tau: float, eps: float,
                 dtype: torch.dtype = torch.bfloat16, device: torch.device = torch.device("cuda")):
        if rank < 1 or not tau > 0.0:
            raise ValueError(f"the decay's projection has rank {rank} and temperature {tau}")
        super().__init__(hidden_size, num_heads, dim, vdim, eps, rank, dtype, device, "qkvga")
        self.rank, self.tau = int(rank), float(tau)
        self.a2t = self.a2_bias = self.norm_weight = None

    def cache_spec(self) -> StateSpec:
        return StateSpec((self.nh * self.dim * self.vdim,))

    def weight_shapes(self):
        H = self.hidden_size
        return {"q": ((self.qk_width, H), "normal"), "k": ((self.qk_width, H), "normal"),
                "v": ((self.v_width, H), "normal"), "g": ((self.v_width, H), "normal"),
                "a1": ((self.rank, H), "normal"), "a2": ((self.qk_width, self.rank), "normal"),
                "a2_bias": ((self.qk_width,), "normal"), "norm": ((self.vdim,), "ones"),
                "o": ((H, self.v_width), "normal")}

    def load(self, q, k, v, g, a1, a2, a2_bias, norm, o) -> None:
        self.proj.load([q, k, v, g, a1])
        self.o.load([o])
        self.a2t = _f32("a2", a2, (self.qk_width, self.rank), self.device).t().contiguous()
        self.a2_bias = _f32("a2_bias", a2_bias, (self.qk_width,), self.device)
        self.norm_weight = _f32("norm", norm, (self.vdim,), self.device)

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx, cache_view, writes_cache: bool = True,
                scratch_cleared: bool = False) -> None:
        if not writes_cache:
            raise ValueError("a gated linear attention mixer cannot read another place's state: its state is its own")
        T = x.shape[0]
        ws = ctx.workspace
        proj = ws.get(self.PROJ, (T, self.width), torch.float32)
        self.proj.forward(x, proj, y_is_zero=scratch_cleared)
        decays = ws.get("gla_decays", (T, self.qk_width), torch.float32)
        ops.gla_decay(proj, self.extra_col, self.rank, self.a2t, self.a2_bias, self.tau, decays)
        o = ws.get("gla_o", (T, self.v_width), torch.float32)
        ops.gated_linear_scan(proj, 0, self.k_col, self.v_col, self.q_scale, decays, o, cache_view.state, ctx.q_start,
                              ctx.seq_slot, ctx.n_seqs, self.nh, self.dim, self.vdim, ctx.max_q_len, ws)
        gated = ws.get("gla_gated", (T, self.v_width), self.dtype)
        ops.head_norm_gate(o, proj[:, self.gate_col: self.gate_col + self.v_width], self.norm_weight, self.eps, gated,
                           self.nh, self.vdim)
        self.o.forward_add(gated, residual)


class MatrixMemory(_GatedLinearBase):
    PROJ = "matrix_memory_proj"

    def __init__(self, hidden_size: int, num_heads: int, dim: int, vdim: int, gate_cap: float, eps: float,
                 dtype: torch.dtype = torch.bfloat16, device: torch.device = torch.device("cuda")):
        if not gate_cap > 0.0:
            raise ValueError(f"the gates' cap must be positive, got {gate_cap}")
        super().__init__(hidden_size, num_heads, dim, vdim, eps, 2 * num_heads, dtype, device, "qkvgif")
        self.cap = float(gate_cap)
        # one block of state per slot: per head [dim, vdim] of S then [dim] of n; then the heads' running maxima
        self.m_off = self.nh * self.dim * (self.vdim + 1)
        self.bias_i = self.bias_f = self.norm_weight = None

    def cache_spec(self) -> StateSpec:
        return StateSpec((self.m_off + self.nh,))

    def weight_shapes(self):
        H = self.hidden_size
        return {"q": ((self.qk_width, H), "normal"), "k": ((self.qk_width, H), "normal"),
                "v": ((self.v_width, H), "normal"), "g": ((self.v_width, H), "normal"),
                "i": ((self.nh, H), "normal"), "f": ((self.nh, H), "normal"), "i_bias": ((self.nh,), "normal"),
                "f_bias": ((self.nh,), "normal"), "norm": ((self.v_width,), "ones"),
                "o": ((H, self.v_width), "normal")}

    def load(self, q, k, v, g, i, f, i_bias, f_bias, norm, o) -> None:
        self.proj.load([q, k, v, g, i, f])
        self.o.load([o])
        self.bias_i = _f32("i_bias", i_bias, (self.nh,), self.device)
        self.bias_f = _f32("f_bias", f_bias, (self.nh,), self.device)
        self.norm_weight = _f32("norm", norm, (self.v_width,), self.device)

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx, cache_view, writes_cache: bool = True,
                scratch_cleared: bool = False) -> None:
        if not writes_cache:
            raise ValueError("a matrix memory mixer cannot read another place's state: its state is its own")
        T = x.shape[0]
        ws = ctx.workspace
        state = cache_view.state
        proj = ws.get(self.PROJ, (T, self.width), torch.float32)
        self.proj.forward(x, proj, y_is_zero=scratch_cleared)
        gates = ws.get("matrix_memory_gates", (T, self.nh, 4), torch.float32)
        ops.exp_gates(proj, self.extra_col, self.extra_col + self.nh, self.bias_i, self.bias_f, self.cap, gates, state,
                      self.m_off, ctx.q_start, ctx.seq_slot, ctx.n_seqs, self.nh)
        o = ws.get("matrix_memory_o", (T, self.v_width), torch.float32)
        divisors = ws.get("matrix_memory_divisors", (T, self.nh), torch.float32)
        ops.gated_linear_scan(proj, 0, self.k_col, self.v_col, self.q_scale, gates, o, state, ctx.q_start, ctx.seq_slot,
                              ctx.n_seqs, self.nh, self.dim, self.vdim, ctx.max_q_len, ws, divisors=divisors)
        gated = ws.get("matrix_memory_gated", (T, self.v_width), self.dtype)
        ops.head_norm_gate(o, proj[:, self.gate_col: self.gate_col + self.v_width], self.norm_weight, self.eps, gated,
                           self.nh, self.vdim, sigmoid=True, denom=divisors)
        self.o.forward_add(gated, residual)


register_part("mixer", "gated_linear_attention", GatedLinearAttention)
register_part("mixer", "matrix_memory", MatrixMemory)
