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
def chunk_softmax(q, k, v, start: int, scale: float, cap: Optional[float], size: Optional[int]) -> torch.Tensor:
    """q [T, H, d] at positions start .. start + T - 1; k [start + T, G, d], v [start + T, G, e] from position 0 on.
    Position i sees j <= i with floor(i / size) = floor(j / size); scores are capped as cap tanh(s / cap)."""
    T, H, G = q.shape[0], q.shape[1], k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=DT)
    for t in range(T):
        i = start + t
        first = (i // size) * size if size else 0
        for head in range(H):
            g = head // (H // G)
            s = (k[first:i + 1, g] @ q[t, head]) * scale
            if cap:
                s = cap * torch.tanh(s / cap)
            out[t, head] = torch.softmax(s, dim=0) @ v[first:i + 1, g]
    return out


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
    out = chunk_softmax(q, k, v, start, m["scale"], m.get("softcap"), (m.get("mask") or {}).get("size"))
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


def delta_recurrence(q, k, v, beta, decay, S=None):
    """q, k [T, G, d] (already unit vectors), v [T, H, e], beta and decay [T, H].  Per head with state S [d, e]:
    S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q.  Returns (o [T, H, e], S [H, d, e])."""
    T, G, d = q.shape
    H, e = v.shape[1], v.shape[2]
    S = torch.zeros(H, d, e, dtype=DT) if S is None else S.clone()
    o = torch.zeros(T, H, e, dtype=DT)
    for t in range(T):
        for head in range(H):
            g = head // (H // G)
            S[head] = decay[t, head] * S[head]
            u = beta[t, head] * (v[t, head] - S[head].T @ k[t, g])
            S[head] = S[head] + torch.outer(k[t, g], u)
            o[t, head] = S[head].T @ q[t, g]
    return o, S


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
    o, S = delta_recurrence(q, k, v, beta, decay, state.get("S"))
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
def routed_feed_forward(h: torch.Tensor, w: Dict[str, torch.Tensor], experts: int, top: int,
                        margins: Optional[list] = None) -> torch.Tensor:
    """out = sum over the `top` experts e with the largest s_e = sigmoid(router h) of expert_e(s_e h).  `margins`
    collects, per call, the smallest gap between a chosen and a not chosen expert's logit."""
    z = h @ w["router"].T
    scores = torch.sigmoid(z)                                  # [T, E]
    if margins is not None and top < experts and h.shape[0]:
        ordered = torch.sort(z, dim=1, descending=True).values
        margins.append(float((ordered[:, top - 1] - ordered[:, top]).min()))
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
        self.margins: List[float] = []     # the routers' smallest gaps between chosen and not chosen, per call

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
                x = x + routed_feed_forward(h, self._sub(p + "mlp."), router["experts"], router["top"],
                                            self.margins) * self.t[p + "ls2"]
            if layers_out is not None:
                layers_out.append(x.clone())
        state["length"] = start + len(tokens)
        return layer_norm(x, self.t["final.norm"], self.eps) @ self.t["head"].T


# ---------------------------------------------------------------------------------------------
# whole sequences, pieces, random models
# ---------------------------------------------------------------------------------------------
def forward(cfg: dict, w: Dict[str, torch.Tensor], ids) -> torch.Tensor:
    """Logits [T, vocab] of one sequence run in one piece."""
    return PlainMugedra(cfg, w).forward(ids)


def forward_in_pieces(cfg: dict, w: Dict[str, torch.Tensor], ids, sizes) -> torch.Tensor:
    """The same sequence cut into pieces of the given sizes, each continuing the state the one before left."""
    model = PlainMugedra(cfg, w)
    state, out, at = model.new_state(), [], 0
    for n in sizes:
        out.append(model.forward(ids[at:at + n], state))
        at += n
    assert at == len(ids)
    return torch.cat(out)


def random_weights(cfg: dict, seed: int) -> Dict[str, torch.Tensor]:
    """Random tensors for a configuration, rounded to bfloat16 values (as a stored model's are)."""
    g = torch.Generator().manual_seed(seed)
    W = int(cfg["width"])

    def rnd(*shape, s=1.0, mean=0.0):
        return (torch.randn(*shape, generator=g) * s + mean).to(torch.bfloat16).to(DT)

    w = {"embed": rnd(cfg["vocab"], W), "final.norm": rnd(W, s=0.1, mean=1.0), "head": rnd(cfg["vocab"], W, s=W ** -0.5)}
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        a, r = layer["mixer"]["left"], layer["mixer"]["right"]
        w[p + "norm1"], w[p + "ls1"] = rnd(W, s=0.1, mean=1.0), rnd(W, s=0.2, mean=0.8)
        H, G, d, e = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
        m = p + "mix.left."
        w[m + "q"], w[m + "k"], w[m + "v"] = rnd(H * d, W, s=W ** -0.5), rnd(G * d, W, s=W ** -0.5), rnd(G * e, W, s=W ** -0.5)
        w[m + "q.norm"], w[m + "k.norm"] = rnd(d, s=0.2, mean=1.0), rnd(d, s=0.2, mean=1.0)
        w[m + "g"], w[m + "o"] = rnd(H * e, W, s=W ** -0.5), rnd(W, H * e, s=(H * e) ** -0.5)
        H, G, d, e, taps = r["heads"], r["kv_heads"], r["dim"], r["vdim"], r["conv"]
        m = p + "mix.right."
        w[m + "q"], w[m + "k"], w[m + "v"] = rnd(G * d, W, s=W ** -0.5), rnd(G * d, W, s=W ** -0.5), rnd(H * e, W, s=W ** -0.5)
        w[m + "q.conv"], w[m + "k.conv"], w[m + "v.conv"] = (rnd(G * d, taps, s=taps ** -0.5), rnd(G * d, taps, s=taps ** -0.5),
                                                             rnd(H * e, taps, s=taps ** -0.5))
        w[m + "b"], w[m + "a"] = rnd(H, W, s=W ** -0.5), rnd(H, W, s=W ** -0.5)
        w[m + "A_log"], w[m + "dt_bias"] = rnd(H, s=0.7, mean=-2.0), rnd(H, s=0.7)
        w[m + "norm"], w[m + "g"], w[m + "o"] = rnd(e, s=0.1, mean=1.0), rnd(H * e, W, s=W ** -0.5), rnd(W, H * e, s=(H * e) ** -0.5)
        w[p + "mix.left.out"], w[p + "mix.right.out"] = rnd(W, s=0.1, mean=1.0), rnd(W, s=0.1, mean=1.0)
        if layer.get("mlp") is not None:
            F, E = layer["mlp"]["expert"]["ff"], layer["mlp"]["router"]["experts"]
            w[p + "norm2"], w[p + "ls2"] = rnd(W, s=0.1, mean=1.0), rnd(W, s=0.2, mean=0.8)
            w[p + "mlp.router"] = rnd(E, W, s=2.0 * W ** -0.5)
            for x in range(E):
                w[p + f"mlp.e{x}.gate"], w[p + f"mlp.e{x}.up"] = rnd(F, W, s=W ** -0.5), rnd(F, W, s=W ** -0.5)
                w[p + f"mlp.e{x}.down"] = rnd(W, F, s=F ** -0.5)
    return w


def save_folder(cfg: dict, w: Dict[str, torch.Tensor], out_dir: str, dtype=torch.bfloat16) -> str:
    """Write config.json and model.safetensors (an independent writer of the file format)."""
    os.makedirs(out_dir, exist_ok=True)
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(cfg, f)
    header, blobs, at = {}, [], 0
    names = {torch.bfloat16: "BF16", torch.float32: "F32"}
    for name, t in w.items():
        t = t.to(dtype).contiguous()
        raw = t.view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": names[dtype], "shape": list(t.shape), "data_offsets": [at, at + len(raw)]}
        blobs.append(raw)
        at += len(raw)
    head = json.dumps(header).encode()
    head += b" " * (-len(head) % 8)
    with open(os.path.join(out_dir, "model.safetensors"), "wb") as f:
        f.write(struct.pack("<Q", len(head)) + head + b"".join(blobs))
    return out_dir
