"""Grouped-query softmax attention with capped scores, a chunked mask and an output gate, over the paged cache.

With h the mixer's input: q = Wq h (heads x dim), k = Wk h (kv_heads x dim), v = Wv h (kv_heads x vdim), no biases;
query head i uses key/value head floor(i / (heads / kv_heads)).  Every head of q and k is divided by its own root mean
square over dim (eps inside the root) and multiplied by a weight of size dim that the heads share; rotary positions
turn the first `rotary_dims` dimensions of every head of q and k (pairing i with i + rotary_dims / 2).  The score
(q . k) * scale becomes softcap * tanh(score / softcap) (softcap 0: as it is); position i sees j <= i with
floor(i / chunk) = floor(j / chunk), chunks counted from the sequence's first position (chunk 0: every j <= i);
ordinary softmax.  The concatenated heads are multiplied by sigmoid(Wg h) and projected by Wo.

Options that other designs use: `qk_norm` "unit" divides the heads of q and k by their root mean square without a
weight (after the rotation, which does not change a head's sum of squares, so the division is done on the way in);
`q_temp` (coef, every) multiplies the query at position p by 1 + coef ln(floor((p + 1) / every) + 1), a temperature
that grows with the sequence; `sink` adds one to the softmax's denominator, p_j = exp(s_j) / (1 + sum exp(s_j)): a key
of score 0 that has no value, so a query may attend to nothing.

q, k, v and the gate are one stacked product whose float32 accumulators one kernel turns into the queries and the
cache rows (`ops.head_norm_rope_cache`); the attention itself is the library's grouped-query attention (tcgen05 for
prompts, split keys for single tokens) with the cap and the chunk as arguments.  Keys and values share one stored head size, the larger of dim and vdim (the extra
columns are zero: scores and sums do not change).
"""
from __future__ import annotations

from typing import Optional

import torch

from ..kernels import ops
from .attention import _check_kernel_limits, stored_head_size
from .base import KVSpec, Mixer, PartSpec, register_part, shared_part
from .linear import Linear


class CappedAttention(Mixer):
    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, dim: int, vdim: int, scale: float,
                 eps: float, softcap: float = 0.0, chunk: int = 0, qk_norm=True, gate: bool = True,
                 position: Optional[PartSpec] = None, rotary_dims: int = 0, sink: bool = False,
                 q_temp: Optional[tuple] = None,
                 dtype: torch.dtype = torch.bfloat16, device: torch.device = torch.device("cuda")):
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} heads are not a multiple of {num_kv_heads} key/value heads")
        if position is not None and (rotary_dims % 2 or not 0 < rotary_dims <= dim):
            raise ValueError(f"{rotary_dims} rotated dimensions do not fit vectors of size {dim}")
        if softcap < 0.0 or chunk < 0:
            raise ValueError(f"a cap ({softcap}) and a chunk ({chunk}) cannot be negative")
        self.hidden_size, self.nh, self.nkv = int(hidden_size), int(num_heads), int(num_kv_heads)
        self.dim, self.vdim = int(dim), int(vdim)
        self.scale, self.eps, self.softcap, self.chunk = float(scale), float(eps), float(softcap), int(chunk)
        if qk_norm not in (True, False, "unit"):
            raise ValueError(f"qk_norm is True (with weights), False or 'unit' (without), got {qk_norm!r}")
        self.unit_norm = qk_norm == "unit"
        self.qk_norm, self.gate, self.sink = qk_norm is True, bool(gate), bool(sink)
        self.temp_coef, self.temp_every = (0.0, 0) if q_temp is None else (float(q_temp[0]), int(q_temp[1]))
        if self.temp_every < 0:
            raise ValueError(f"a query temperature steps every {self.temp_every} positions")
        self.dtype, self.device = dtype, device
        self.stored = stored_head_size(max(self.dim, self.vdim), dtype)
        _check_kernel_limits(self.nh, self.nkv, self.stored, dtype)
        self.position = shared_part("position", position, dtype, device) if position is not None else None
        self.rotary_dims = int(rotary_dims) if position is not None else 0
        self.q_width, self.k_width, self.v_width = self.nh * self.dim, self.nkv * self.dim, self.nkv * self.vdim
        self.o_width = self.nh * self.vdim
        self.gate_col = self.q_width + self.k_width + self.v_width
        self.proj = Linear(hidden_size, self.gate_col + (self.o_width if self.gate else 0), dtype, device, name="qkvg",
                           pad_width=True)
        self.o = Linear(self.nh * self.stored, hidden_size, dtype, device, name="o", pad_width=True)
        self.wq = self.wk = None

    def cache_spec(self) -> KVSpec:
        return KVSpec(self.nkv, self.stored)

    def limit_positions(self, n: int) -> None:
        limit = getattr(self.position, "limit_positions", None)
        if limit is not None:
            limit(n)

    def weight_shapes(self):
        shapes = {"q": ((self.q_width, self.hidden_size), "normal"), "k": ((self.k_width, self.hidden_size), "normal"),
                  "v": ((self.v_width, self.hidden_size), "normal"), "o": ((self.hidden_size, self.o_width), "normal")}
        if self.qk_norm:
            shapes.update(q_norm=((self.dim,), "ones"), k_norm=((self.dim,), "ones"))
        if self.gate:
            shapes["g"] = ((self.o_width, self.hidden_size), "normal")
        return shapes

    def load(self, q, k, v, o, q_norm=None, k_norm=None, g=None) -> None:
        self.proj.load([q, k, v] + ([g] if self.gate else []))
        if tuple(o.shape) != (self.hidden_size, self.o_width):
            raise ValueError(f"weight 'o' of shape {tuple(o.shape)} does not fit ({self.hidden_size}, {self.o_width})")
        if self.stored != self.vdim:             # zero columns where the stored heads have their extra columns
            wide = torch.zeros((self.hidden_size, self.nh, self.stored), dtype=o.dtype, device=o.device)
            wide[:, :, : self.vdim] = o.view(self.hidden_size, self.nh, self.vdim)
            o = wide.view(self.hidden_size, self.nh * self.stored)
        self.o.load([o])
        if self.qk_norm:
            for t in (q_norm, k_norm):
                if tuple(t.shape) != (self.dim,):
                    raise ValueError(f"a head norm weight of shape {tuple(t.shape)} does not fit ({self.dim},)")
            self.wq = q_norm.to(device=self.device, dtype=torch.float32).contiguous()
            self.wk = k_norm.to(device=self.device, dtype=torch.float32).contiguous()

    def scratch_to_clear(self, ctx, tokens: int, writes_cache: bool = True) -> Optional[torch.Tensor]:
        """The projections' float32 buffer, if this step's product adds slices of K into it (decode-sized steps):
        the launch before this mixer clears it in passing."""
        if not self.proj.meets_by_adds(tokens, torch.float32):
            return None
        buf = ctx.workspace.get("capped_proj", (tokens, self.proj.out_features), torch.float32)
        return buf if buf.numel() % 4 == 0 else None

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx, cache_view, writes_cache: bool = True,
                scratch_cleared: bool = False) -> None:
        if not writes_cache:
            raise ValueError("this attention writes its own keys and values; it cannot read another place's")
        T = x.shape[0]
        ws = ctx.workspace
        group = cache_view.group
        proj = ws.get("capped_proj", (T, self.proj.out_features), torch.float32)
        self.proj.forward(x, proj, y_is_zero=scratch_cleared)
        table = self.position.fused_rotary_table() if self.position is not None else None
        D = self.stored
        q = ws.get("capped_q", (T, self.nh * D), self.dtype)
        ops.head_norm_rope_cache(proj, self.wq, self.wk, self.eps, table, self.rotary_dims, ctx.positions, q,
                                 group.dest_rows, cache_view.k, cache_view.v, self.nh, self.nkv, self.dim, self.vdim, D,
                                 group.page_size, unit_norm=self.unit_norm, temp_coef=self.temp_coef,
                                 temp_every=self.temp_every)
        attn = ws.get("capped_attn", (T, self.nh * D), self.dtype)
        if self.dtype == torch.float32:
            ops.attention_f32(q, cache_view.k, cache_view.v, attn, group.block_table, ctx.token_seq, ctx.positions,
                              self.nh, self.nkv, D, group.page_size, 0, self.scale, self.chunk, self.softcap, sink=self.sink)
        elif ctx.is_decode:
            ops.attention_bf16_decode(q, cache_view.k, cache_view.v, attn, group.block_table, ctx.kv_len, self.nh,
                                      self.nkv, D, group.page_size, 0, self.scale, ctx.workspace,
                                      min(ctx.max_kv_len_bound, self.chunk) if self.chunk else ctx.max_kv_len_bound,
                                      chunk=self.chunk, softcap=self.softcap, sink=self.sink)
        elif ops.attention_tc_supported(self.nh, self.nkv, D):
            ops.attention_tc_prefill(q, cache_view.k, cache_view.v, attn, group.block_table, ctx.q_start, ctx.kv_len,
                                     ctx.n_seqs, ctx.max_q_len, self.nh, self.nkv, D, group.page_size, 0, self.scale,
                                     self.chunk, self.softcap, sink=self.sink)
        else:
            ops.attention_bf16_prefill(q, cache_view.k, cache_view.v, attn, group.block_table, ctx.q_start, ctx.kv_len,
                                       ctx.n_seqs, ctx.max_q_len, self.nh, self.nkv, D, group.page_size, 0, self.scale,
                                       self.chunk, self.softcap, sink=self.sink)
        if self.gate:
            ops.sigmoid_gate(attn, proj[:, self.gate_col:], self.nh, self.vdim, D)
        self.o.forward_add(attn, residual)


register_part("mixer", "capped_attention", CappedAttention)
