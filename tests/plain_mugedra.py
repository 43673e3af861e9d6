"""A plain, slow implementation of the Mugedra decoder on the CPU: one function per mechanism,
written from the design's equations, sharing no code with the library.  Everything runs in one
dtype (float64) on whole sequences; the mixers take and return an explicit state, so that the
tests can run a sequence in one piece, in portions or token by token and compare.

Notation: T tokens, W width, H query heads, G key/value heads, d query/key size, e value size,
E experts.  Linear weights are [out, in] and applied as W x.
"""
from __future__ import annotations

import json
import math
import os
import struct
from typing import Dict, List, Optional

import torch

DT = torch.float64


# ---------------------------------------------------------------------------------------------
# reading a model folder (an independent reader of the file format)
# ---------------------------------------------------------------------------------------------
def read_folder(model_dir: str):
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    with open(os.path.join(model_dir, "model.safetensors"), "rb") as f:
        raw = f.read()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + n])
    data = raw[8 + n:]
    kinds = {"BF16": torch.bfloat16, "F32": torch.float32, "F16": torch.float16, "I32": torch.int32}
    out: Dict[str, torch.Tensor] = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        a, b = meta["data_offsets"]
        t = torch.frombuffer(bytearray(data[a:b]), dtype=kinds[meta["dtype"]]).reshape(meta["shape"]).clone()
        out[name] = t.to(DT) if t.is_floating_point() else t
    return cfg, out


# ---------------------------------------------------------------------------------------------
# small pieces
# ---------------------------------------------------------------------------------------------
def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x divided by its root mean square over the last axis, eps inside the root."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def layer_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """(x - mean) / sqrt(mean of squared deviations + eps) * w, no bias."""
    mu = x.mean(dim=-1, keepdim=True)
    dev = x - mu
    return dev / torch.sqrt((dev * dev).mean(dim=-1, keepdim=True) + eps) * w


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.logaddexp(z, torch.zeros_like(z))


# ---------------------------------------------------------------------------------------------
# rotary positions with a frequency ramp
# ---------------------------------------------------------------------------------------------
def rotary_frequencies(dims: int, base: float, scaling: Optional[dict]):
    """(one frequency per pair, the amplitude of cos and sin).  f_i = base^(-2i/dims); with
    scaling (factor, original, fast, slow): pair(t) = dims ln(original / (2 pi t)) / (2 ln base),
    lo = max(floor(pair(fast)), 0), hi = min(ceil(pair(slow)), dims - 1),
    ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1); f_i <- f_i / factor * ramp_i + f_i (1 - ramp_i);
    amplitude 0.1 ln(factor) + 1."""
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=DT)
    if scaling is None:
        return f, 1.0

    def pair(turns: float) -> float:
        return dims * math.log(scaling["original"] / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(pair(scaling["fast"])), 0)
    hi = min(math.ceil(pair(scaling["slow"])), dims - 1)
    ramp = torch.tensor([min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0) for i in range(half)], dtype=DT)
    return f / scaling["factor"] * ramp + f * (1.0 - ramp), 0.1 * math.log(scaling["factor"]) + 1.0


def rotate(x: torch.Tensor, positions: torch.Tensor, dims: int, base: float, scaling: Optional[dict]) -> torch.Tensor:
    """x [T, heads, d]: dimension i < dims/2 is paired with i + dims/2; (u, v) -> (u c - v s, v c + u s);
    dimensions from `dims` on pass unchanged."""
    f, amp = rotary_frequencies(dims, base, scaling)
    angle = positions.to(DT)[:, None] * f[None, :]
    c, s = (torch.cos(angle) * amp)[:, None, :], (torch.sin(angle) * amp)[:, None, :]
    half = dims // 2
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


# ---------------------------------------------------------------------------------------------
# left mixer: chunked softmax attention with a soft cap and an output gate
# ---------------------------------------------------------------------------------------------
def chunk_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float, start: int = 0,
                    past: Optional[dict] = None):
    """h [T, W], the tokens at positions start .. start + T - 1 of one sequence; `past` holds the keys
    and values of the positions before.  Returns (output [T, W], new past)."""
    T = h.shape[0]
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w["q"].T).view(T, H, d)
    k = (h @ w["k"].T).view(T, G, d)
    v = (h @ w["v"].T).view(T, G, e)
    q = rms_unit(q, eps) * w["q.norm"]
    k = rms_unit(k, eps) * w["k.norm"]
    pos = torch.arange(start, start + T)
    rot = m.get("rot")
    if rot:
        q = rotate(q, pos, rot["dims"], rot["base"], rot.get("scaling"))
        k = rotate(k, pos, rot["dims"], rot["base"], rot.get("scaling"))
    if past is not None:
        k, v = torch.cat([past["k"], k]), torch.cat([past["v"], v])
    size = (m.get("mask") or {}).get("size")
    cap = m.get("softcap")
    out = torch.zeros(T, H, e, dtype=DT)
    for t in range(T):
        i = start + t
        first = (i // size) * size if size else 0
        for head in range(H):
            g = head // (H // G)
            s = (k[first:i + 1, g] @ q[t, head]) * m["scale"]
            if cap:
                s = cap * torch.tanh(s / cap)
            p = torch.softmax(s, dim=0)
            out[t, head] = p @ v[first:i + 1, g]
    gate = torch.sigmoid(h @ w["g"].T)
    return (out.reshape(T, H * e) * gate) @ w["o"].T, {"k": k, "v": v}


# ---------------------------------------------------------------------------------------------
# right mixer: the gated delta rule
# ---------------------------------------------------------------------------------------------
def short_conv(u: torch.Tensor, weight: torch.Tensor, tail: Optional[torch.Tensor]):
    """u [T, C]; weight [C, taps] whose last column meets the current token; `tail` the taps - 1 inputs
    before u (zeros at a sequence's start).  Returns (silu(convolution), new tail)."""
    taps = weight.shape[1]
    if tail is None:
        tail = torch.zeros(taps - 1, u.shape[1], dtype=DT)
    full = torch.cat([tail, u])
    out = torch.zeros_like(u)
    for t in range(u.shape[0]):
        for j in range(taps):
            out[t] += weight[:, j] * full[t + j]
    return silu(out), full[full.shape[0] - (taps - 1):]


def gated_delta(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float, state: Optional[dict] = None):
    """Per head with state S [d, e]: S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q."""
    T = h.shape[0]
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    state = state or {}
    q, tq = short_conv(h @ w["q"].T, w["q.conv"], state.get("q"))
    k, tk = short_conv(h @ w["k"].T, w["k.conv"], state.get("k"))
    v, tv = short_conv(h @ w["v"].T, w["v.conv"], state.get("v"))
    q, k, v = q.view(T, G, d), k.view(T, G, d), v.view(T, H, e)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w["b"].T)                                           # [T, H]
    decay = torch.exp(-torch.exp(w["A_log"]) * softplus(h @ w["a"].T + w["dt_bias"]))   # [T, H]
    S = state.get("S")
    S = torch.zeros(H, d, e, dtype=DT) if S is None else S.clone()
    o = torch.zeros(T, H, e, dtype=DT)
    for t in range(T):
        for head in range(H):
            g = head // (H // G)
            S[head] = decay[t, head] * S[head]
            u = beta[t, head] * (v[t, head] - S[head].T @ k[t, g])
            S[head] = S[head] + torch.outer(k[t, g], u)
            o[t, head] = S[head].T @ q[t, g]
    o = rms_unit(o, eps) * w["norm"]
    gate = silu(h @ w["g"].T).view(T, H, e)
    return (o * gate).reshape(T, H * e) @ w["o"].T, {"q": tq, "k": tk, "v": tv, "S": S}


def parallel_mixer(h, w: Dict[str, torch.Tensor], m: dict, eps: float, start: int = 0, state: Optional[dict] = None):
    """Half the sum of the two branches, each divided by its root mean square over the width and weighted."""
    state = state or {}
    sub = lambda side: {n[len(side) + 1:]: t for n, t in w.items() if n.startswith(side + ".")}   # noqa: E731
    left, past = chunk_attention(h, sub("left"), m["left"], eps, start, state.get("left"))
    right, rec = gated_delta(h, sub("right"), m["right"], eps, state.get("right"))
    out = 0.5 * (rms_unit(left, eps) * w["left.out"] + rms_unit(right, eps) * w["right.out"])
    return out, {"left": past, "right": rec}


# ---------------------------------------------------------------------------------------------
# feed-forward: experts chosen by sigmoid scores, the score on the expert's input
# ---------------------------------------------------------------------------------------------
def routed_feed_forward(h: torch.Tensor, w: Dict[str, torch.Tensor], experts: int, top: int) -> torch.Tensor:
    scores = torch.sigmoid(h @ w["router"].T)                  # [T, E]
    out = torch.zeros(h.shape[0], w["e0.down"].shape[0], dtype=DT)
    for t in range(h.shape[0]):
        for e in torch.topk(scores[t], top).indices.tolist():
            x = scores[t, e] * h[t]
            out[t] += w[f"e{e}.down"] @ (silu(w[f"e{e}.gate"] @ x) * (w[f"e{e}.up"] @ x))
    return out


# ---------------------------------------------------------------------------------------------
# the model
# ---------------------------------------------------------------------------------------------
def layer_runs(cfg: dict) -> List[tuple]:
    """(layer, whether the embedding output joins x before it) in the order the layers run."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, False) for i in range(n)]
    runs = [(i, False) for i in range(loop["start"])]
    for p in range(loop["times"]):
        for i in range(loop["start"], loop["stop"]):
            runs.append((i, p > 0 and i == loop["start"]))
    return runs + [(i, False) for i in range(loop["stop"], n)]


class PlainMugedra:
    def __init__(self, cfg: dict, tensors: Dict[str, torch.Tensor]):
        self.cfg = cfg
        self.t = {k: (v.to(DT) if v.is_floating_point() else v) for k, v in tensors.items()}
        self.eps = cfg["norm"]["eps"]
        self.runs = layer_runs(cfg)

    def _sub(self, prefix: str) -> Dict[str, torch.Tensor]:
        return {n[len(prefix):]: v for n, v in self.t.items() if n.startswith(prefix)}

    def new_state(self) -> dict:
        return {"length": 0, "runs": [None] * len(self.runs)}

    def forward(self, tokens, state: Optional[dict] = None, layers_out: Optional[list] = None):
        """Logits [T, vocab] of the tokens, continuing `state` (changed in place)."""
        state = state if state is not None else self.new_state()
        start = state["length"]
        x = self.t["embed"][torch.as_tensor(tokens, dtype=torch.long)]
        emb = x
        for r, (i, joins) in enumerate(self.runs):
            layer, p = self.cfg["layers"][i], f"l{i}."
            if joins:
                x = x + emb
            h = layer_norm(x, self.t[p + "norm1"], self.eps)
            y, state["runs"][r] = parallel_mixer(h, self._sub(p + "mix."), layer["mixer"], self.eps, start,
                                                 state["runs"][r])
            x = x + y * self.t[p + "ls1"]
            if layer.get("mlp") is not None:
                h = layer_norm(x, self.t[p + "norm2"], self.eps)
                router = layer["mlp"]["router"]
                x = x + routed_feed_forward(h, self._sub(p + "mlp."), router["experts"], router["top"]) * self.t[p + "ls2"]
            if layers_out is not None:
                layers_out.append(x.clone())
        state["length"] = start + len(tokens)
        return layer_norm(x, self.t["final.norm"], self.eps) @ self.t["head"].T
