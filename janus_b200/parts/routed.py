"""A feed-forward made of experts of which every token uses a few.

`experts` gated feed-forwards without biases, expert(x) = Wd (silu(Wg x) * (Wu x)).  The router's logits z = Wr h are
float32 (the product's own accumulators), the scores s = sigmoid(z); a token's `top` experts are those with the
largest scores (the lower index wins a tie) and their weights are those scores as they are, not renormalized.  The
weight multiplies the expert's INPUT: out = sum over the chosen e of expert_e(s_e h).

Steps of few (token, expert) pairs, every single-token step among them, stream each chosen expert's rows once for
up to four of the tokens that chose it (`ops.experts_few_tokens`: two launches with a block per (rows, expert),
float32 sums, nothing read back by the host, so the step can be recorded into a CUDA graph).  Prompt steps of the
bfloat16 engine with more pairs sort the (token, choice) pairs by expert, gather the weighted rows in that order and
run the experts' two products on the tensor cores over their rows; the results are added back token by token in the
order of the token's choices.  Where the sizes allow it (width and inner width multiples of 128) the sort is a kernel
(`ops.expert_plan`), and each of the two products is ONE launch over the stack of all experts' matrices whose tiles
that kernel listed (`ops.gemm_bf16_grouped`): the host never reads the choice.  Other sizes read the choice back
and launch each expert's products by themselves.  The float32 engine always streams.

Options that other designs use.  `score` "softmax": the scores are the softmax of the logits over all experts (still
taken as they are).  `groups` (count, keep): the experts form `count` equal groups of neighbours, a group's score is
its largest score, and only experts of the `keep` best groups can be chosen.  `weight_on` "output": the weight
multiplies the expert's output, out = sum over the chosen e of s_e expert_e(h).  `shared_size`: one more gated
feed-forward of that inner width runs for every token and is added; with `shared_gate` it is multiplied by
sigmoid(wsg . h), one number per token (the gate's row rides along in the router's product, and because the last
product is linear the gate multiplies the rows that product reads).
"""
from __future__ import annotations

from typing import List, Optional

import numpy as np
import torch

from ..kernels import ops
from .base import FeedForward, register_part
from .linear import GatedLinear, Linear

FEW_PAIRS = 64           # up to this many (token, expert) pairs a bfloat16 prompt step streams the experts' rows
MAX_STREAM_PAIRS = 65535  # pairs of one launch of the streaming kernels


class RoutedExperts(FeedForward):
    def __init__(self, hidden_size: int, intermediate_size: int, experts: int, top: int, score: str = "sigmoid",
                 groups: Optional[tuple] = None, weight_on: str = "input", shared_size: Optional[int] = None,
                 shared_gate: bool = False,
                 dtype: torch.dtype = torch.bfloat16, device: torch.device = torch.device("cuda")):
        if not 1 <= top <= experts:
            raise ValueError(f"a token uses {top} of {experts} experts")
        if score not in ("sigmoid", "softmax") or weight_on not in ("input", "output"):
            raise ValueError(f"scores are 'sigmoid' or 'softmax' and weigh the 'input' or the 'output', got "
                             f"{score!r}, {weight_on!r}")
        self.softmax, self.weight_on_output = score == "softmax", weight_on == "output"
        self.groups, self.keep = (0, 0) if groups is None else (int(groups[0]), int(groups[1]))
        if groups is not None and (self.groups < 1 or self.groups > 64 or experts % self.groups
                                   or not 1 <= self.keep <= self.groups or self.keep * (experts // self.groups) < top):
            raise ValueError(f"{self.groups} groups of which {self.keep} are kept do not fit {experts} experts "
                             f"and {top} a token")
        self.shared_size = None if shared_size is None else int(shared_size)
        self.shared_gate = bool(shared_gate) and self.shared_size is not None
        if top > 16:
            raise ValueError(f"at most 16 experts a token are supported, got {top}")
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        self.experts, self.top = int(experts), int(top)
        self.dtype, self.device = dtype, device
        # the router's product also makes the shared expert's gate: one more row
        self.router = Linear(hidden_size, experts + (1 if self.shared_gate else 0), dtype, device, name="router",
                             pad_width=True)
        self.shared_gate_up = self.shared_down = None
        if self.shared_size is not None:
            self.shared_gate_up = GatedLinear(hidden_size, self.shared_size, dtype, device, name="shared_gate_up",
                                              pad_width=True)
            self.shared_down = Linear(self.shared_size, hidden_size, dtype, device, name="shared_down", pad_width=True)
        self.w_gate = self.w_up = self.w_down = None           # [E, F, W], [E, F, W], [E, W, F] row-major
        self.gate_up: List[GatedLinear] = []                   # bfloat16 engine: the experts' tensor-core products
        self.down: List[Linear] = []
        # ... or, where tiles never straddle two experts, the packed stacks of all experts' matrices
        self.grouped = (dtype == torch.bfloat16 and hidden_size % 128 == 0 and intermediate_size % 128 == 0
                        and experts <= ops.EXPERT_PLAN_MAX_EXPERTS)
        self.gate_up_stack = self.down_stack = None

    def weight_shapes(self):
        W, F = self.hidden_size, self.intermediate_size
        shapes = {"router": ((self.experts, W), "normal")}
        for e in range(self.experts):
            shapes.update({f"e{e}_gate": ((F, W), "normal"), f"e{e}_up": ((F, W), "normal"),
                           f"e{e}_down": ((W, F), "normal")})
        if self.shared_size is not None:
            shapes.update({"shared_gate": ((self.shared_size, W), "normal"), "shared_up": ((self.shared_size, W), "normal"),
                           "shared_down": ((W, self.shared_size), "normal")})
            if self.shared_gate:
                shapes["shared_sg"] = ((1, W), "normal")
        return shapes

    def load(self, router: torch.Tensor, shared_gate: Optional[torch.Tensor] = None,
             shared_up: Optional[torch.Tensor] = None, shared_down: Optional[torch.Tensor] = None,
             shared_sg: Optional[torch.Tensor] = None, **experts: torch.Tensor) -> None:
        self.router.load([router] + ([shared_sg] if self.shared_gate else []))
        if self.shared_size is not None:
            self.shared_gate_up.load(shared_gate, shared_up)
            self.shared_down.load([shared_down])
        W, F, E = self.hidden_size, self.intermediate_size, self.experts

        def stack(kind: str, shape) -> torch.Tensor:
            ts = [experts[f"e{e}_{kind}"] for e in range(E)]
            for t in ts:
                if tuple(t.shape) != shape:
                    raise ValueError(f"an expert's '{kind}' of shape {tuple(t.shape)} does not fit {shape}")
            return torch.stack([t.to(device=self.device, dtype=self.dtype) for t in ts]).contiguous()

        self.w_gate, self.w_up, self.w_down = stack("gate", (F, W)), stack("up", (F, W)), stack("down", (W, F))
        self.gate_up, self.down = [], []
        if self.grouped:
            self.gate_up_stack = ops.pack_gated(self.w_gate.reshape(E * F, W), self.w_up.reshape(E * F, W))
            self.down_stack = ops.pack_weight(self.w_down.reshape(E * W, F))
        elif self.dtype == torch.bfloat16:
            for e in range(E):
                gu = GatedLinear(W, F, self.dtype, self.device, name="expert_gate_up", pad_width=True)
                gu.load(self.w_gate[e], self.w_up[e])
                dn = Linear(F, W, self.dtype, self.device, name="expert_down", pad_width=True)
                dn.load([self.w_down[e]])
                self.gate_up.append(gu)
                self.down.append(dn)

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx) -> None:
        T = x.shape[0]
        ws = ctx.workspace
        logits = ws.get("router_logits", (T, self.router.out_features), torch.float32)
        self.router.forward(x, logits)
        if self.shared_size is not None:
            shared = ws.get("shared_act", (T, self.shared_size), self.dtype)
            self.shared_gate_up.forward(x, shared, ctx)
            if self.shared_gate:
                ops.scale_rows_sigmoid(shared, logits[:, self.experts])
            self.shared_down.forward_add(shared, residual)
        sel_e = ws.get("router_experts", (T, self.top), torch.int32)
        sel_w = ws.get("router_weights", (T, self.top), torch.float32)
        ops.route_topk(logits, self.top, sel_e, sel_w, softmax=self.softmax, groups=self.groups, keep=self.keep,
                       experts=self.experts)
        pairs = T * self.top
        if self.dtype == torch.bfloat16 and not ctx.is_decode and pairs > FEW_PAIRS:
            if self.grouped:
                self._grouped(x, sel_e, sel_w, residual, ctx)
            else:
                self._by_expert(x, sel_e, sel_w, residual, ctx)
            return
        act = ws.get("experts_act", (pairs, self.intermediate_size), torch.float32)
        rows = max(1, MAX_STREAM_PAIRS // self.top)
        for t0 in range(0, T, rows):
            t1 = min(T, t0 + rows)
            ops.experts_few_tokens(x[t0:t1], sel_e[t0:t1], sel_w[t0:t1], self.w_gate, self.w_up, self.w_down,
                                   act[t0 * self.top: t1 * self.top], residual[t0:t1],
                                   weight_on_output=self.weight_on_output)

    def _grouped(self, x: torch.Tensor, sel_e: torch.Tensor, sel_w: torch.Tensor, residual: torch.Tensor, ctx) -> None:
        """The tensor-core path of a prompt step without the host: sort, gather, two grouped products, add back."""
        T, W, F, E, top = x.shape[0], self.hidden_size, self.intermediate_size, self.experts, self.top
        pairs = T * top
        ws = ctx.workspace
        max_gu = ops.grouped_max_items(pairs, E, F, "swiglu")
        max_dn = ops.grouped_max_items(pairs, E, W, "store")
        index = ws.get("experts_index", (2, pairs), torch.int32)
        table_gu = ws.get("experts_gate_up_tiles", (4 + 4 * max_gu,), torch.int32)
        table_dn = ws.get("experts_down_tiles", (4 + 4 * max_dn,), torch.int32)
        ops.expert_plan(sel_e, E, F, W, index[0], index[1], table_gu, table_dn)
        rows = ws.get("experts_rows", (pairs, W), self.dtype)
        ops.expert_gather(x, index[0], None if self.weight_on_output else sel_w, top, rows)
        act = ws.get("experts_act_rows", (pairs, F), self.dtype)
        ops.gemm_bf16_grouped(rows, self.gate_up_stack, act, table_gu, max_gu, mode="swiglu", label="expert_gate_up")
        results = ws.get("experts_results", (pairs, W), torch.float32)
        ops.gemm_bf16_grouped(act, self.down_stack, results, table_dn, max_dn, mode="store", label="expert_down")
        ops.expert_scatter(results, index[1], top, residual, weights=sel_w if self.weight_on_output else None)

    def _by_expert(self, x: torch.Tensor, sel_e: torch.Tensor, sel_w: torch.Tensor, residual: torch.Tensor, ctx) -> None:
        """The tensor-core path of a prompt step: the host reads the choice, sorts the (token, choice) pairs by expert
        and launches each expert's products over its rows."""
        T, W, F, top = x.shape[0], self.hidden_size, self.intermediate_size, self.top
        pairs = T * top
        chosen = sel_e.reshape(-1).cpu().numpy()                  # waits for the router
        order = np.argsort(chosen, kind="stable").astype(np.int32)
        where = np.empty(pairs, dtype=np.int32)
        where[order] = np.arange(pairs, dtype=np.int32)
        counts = np.bincount(chosen, minlength=self.experts)
        index = torch.from_numpy(np.concatenate([order, where])).to(self.device)
        ws = ctx.workspace
        rows = ws.get("experts_rows", (pairs, W), self.dtype)
        ops.expert_gather(x, index[:pairs], None if self.weight_on_output else sel_w, top, rows)
        act = ws.get("experts_act_rows", (pairs, F), self.dtype)
        results = ws.get("experts_results", (pairs, W), torch.float32)
        start = 0
        for e in range(self.experts):
            n = int(counts[e])
            if n:
                self.gate_up[e].forward(rows[start:start + n], act[start:start + n], ctx)
                self.down[e].forward(act[start:start + n], results[start:start + n])
                start += n
        ops.expert_scatter(results, index[pairs:], top, residual, weights=sel_w if self.weight_on_output else None)


register_part("feed_forward", "routed_experts", RoutedExperts)
