"""A plain, slow implementation of the Buludra decoder on the CPU: one function per mechanism,
written from the design's equations, sharing no code with the library.  Everything runs in one
dtype (float64); the mixers take and return an explicit state, so that the tests can run a
sequence in one piece, in portions or token by token and compare.

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


def read_folder(model_dir: str):
    """config.json and the tensors of model.safetensors (an independent reader of the file format)."""
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


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def log_sigmoid(z: torch.Tensor) -> torch.Tensor:
    return -torch.logaddexp(-z, torch.zeros_like(z))


def rotate_half(x: torch.Tensor, positions: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """x [T, heads, d]: dimension i < dims/2 is paired with i + dims/2, angle p * base^(-2i/dims);
    (u, v) -> (u c - v s, v c + u s); dimensions from `dims` on pass unchanged."""
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=DT)
    angle = positions.to(DT)[:, None] * f[None, :]
    c, s = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


def query_temperature(positions: torch.Tensor, coef: float, every: int) -> torch.Tensor:
    """1 + coef ln(floor((p + 1) / every) + 1) for every position p."""
    steps = torch.div(positions + 1, every, rounding_mode="floor").to(DT)
    return 1.0 + coef * torch.log(steps + 1.0)


# ---------------------------------------------------------------------------------------------
# softmax attention over all earlier keys, with or without a sink in the denominator
# ---------------------------------------------------------------------------------------------
def causal_attention(q, k, v, start: int, scale: float, sink: bool) -> torch.Tensor:
    """q [T, H, d] at positions start .. start + T - 1; k [start + T, G, d], v [start + T, G, e] from position 0 on.
    Position i sees every j <= i.  With a sink the weights are exp(s_j) / (1 + sum exp(s_j))."""
    T, H, G = q.shape[0], q.shape[1], k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=DT)
    for t in range(T):
        i = start + t
        for head in range(H):
            g = head // (H // G)
            s = (k[:i + 1, g] @ q[t, head]) * scale
            if sink:
                p = torch.softmax(torch.cat([s, torch.zeros(1, dtype=DT)]), dim=0)[:-1]
            else:
                p = torch.softmax(s, dim=0)
            out[t, head] = p @ v[:i + 1, g]
    return out


def temperature_attention(p: dict, w: Dict[str, torch.Tensor], pre: str, h: torch.Tensor, start: int, eps: float,
                          state: Optional[dict]):
    """Mixer 'attention': per-head norm of q and k with a shared weight, no rotation, a query temperature."""
    T, H, G, d, e = h.shape[0], p["heads"], p["kv_heads"], p["dim"], p["vdim"]
    pos = torch.arange(start, start + T)
    q = (h @ w[pre + "q"].T).view(T, H, d)
    k = (h @ w[pre + "k"].T).view(T, G, d)
    v = (h @ w[pre + "v"].T).view(T, G, e)
    q = rms_unit(q, eps) * w[pre + "q.norm"]
    k = rms_unit(k, eps) * w[pre + "k.norm"]
    if p.get("q_temp") is not None:
        q = q * query_temperature(pos, p["q_temp"]["coef"], p["q_temp"]["every"])[:, None, None]
    if state is not None:
        k, v = torch.cat([state["k"], k]), torch.cat([state["v"], v])
    o = causal_attention(q, k, v, start, p["scale"], sink=False)
    return o.reshape(T, H * e) @ w[pre + "o"].T, {"k": k, "v": v}


def sink_attention(p: dict, w: Dict[str, torch.Tensor], pre: str, h: torch.Tensor, start: int, eps: float,
                   state: Optional[dict]):
    """Left branch of 'parallel': rotation of the leading dimensions, then q and k divided by their root mean square,
    a sink in the softmax."""
    T, H, G, d, e = h.shape[0], p["heads"], p["kv_heads"], p["dim"], p["vdim"]
    pos = torch.arange(start, start + T)
    q = (h @ w[pre + "q"].T).view(T, H, d)
    k = (h @ w[pre + "k"].T).view(T, G, d)
    v = (h @ w[pre + "v"].T).view(T, G, e)
    if p.get("rot") is not None:
        q = rotate_half(q, pos, p["rot"]["dims"], p["rot"]["base"])
        k = rotate_half(k, pos, p["rot"]["dims"], p["rot"]["base"])
    q, k = rms_unit(q, eps), rms_unit(k, eps)
    if state is not None:
        k, v = torch.cat([state["k"], k]), torch.cat([state["v"], v])
    o = causal_attention(q, k, v, start, p["scale"], sink=True)
    return o.reshape(T, H * e) @ w[pre + "o"].T, {"k": k, "v": v}


# ---------------------------------------------------------------------------------------------
# gated linear attention: a decay per key channel
# ---------------------------------------------------------------------------------------------
def decay_recurrence(q, k, v, alpha, S: Optional[torch.Tensor] = None):
    """q, k, alpha [T, H, d], v [T, H, e]: S_t = diag(alpha_t) S_(t-1) + k_t v_t^T, o_t = S_t^T q_t; returns (o, S)."""
    T, H, d, e = q.shape[0], q.shape[1], q.shape[2], v.shape[2]
    S = torch.zeros(H, d, e, dtype=DT) if S is None else S.clone()
    o = torch.zeros(T, H, e, dtype=DT)
    for t in range(T):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hde,hd->he", S, q[t])
    return o, S


def channel_decays(low: torch.Tensor, a2: torch.Tensor, bias: torch.Tensor, tau: float) -> torch.Tensor:
    """sigmoid(z)^(1/tau) with z = A2 low + bias."""
    return torch.exp(log_sigmoid(low @ a2.T + bias) / tau)


def gated_linear_attention(p: dict, w: Dict[str, torch.Tensor], pre: str, h: torch.Tensor, eps: float,
                           state: Optional[dict]):
    T, H, d, e = h.shape[0], p["heads"], p["dim"], p["vdim"]
    q = (h @ w[pre + "q"].T).view(T, H, d) * d ** -0.5
    k = (h @ w[pre + "k"].T).view(T, H, d)
    v = (h @ w[pre + "v"].T).view(T, H, e)
    alpha = channel_decays(h @ w[pre + "a1"].T, w[pre + "a2"], w[pre + "a2.b"], p["tau"]).view(T, H, d)
    o, S = decay_recurrence(q, k, v, alpha, None if state is None else state["S"])
    o = rms_unit(o, eps) * w[pre + "norm"]
    y = o.reshape(T, H * e) * silu(h @ w[pre + "g"].T)
    return y @ w[pre + "o"].T, {"S": S}


# ---------------------------------------------------------------------------------------------
# matrix memory with exponential gates and a running maximum
# ---------------------------------------------------------------------------------------------
def log_gates(zi, zf, bias_i, bias_f, cap: float):
    """The logarithms of the input and the forget gate: cap tanh((zi + bi) / cap), logsigmoid(cap tanh((zf + bf) / cap))."""
    return cap * torch.tanh((zi + bias_i) / cap), log_sigmoid(cap * torch.tanh((zf + bias_f) / cap))


def exp_gate_recurrence(q, k, v, gi, gf, state: Optional[dict] = None):
    """q, k [T, H, d], v [T, H, e], log gates gi, gf [T, H].  With the running maximum m (0 at the start):
    m_t = max(gf + m, gi); S_t = exp(gf + m - m_t) S + exp(gi - m_t) k v^T; n likewise with k alone;
    o_t = S_t^T q / (max(|n_t . q|, exp(-m_t)) + 1e-6).  Returns (o, state)."""
    T, H, d, e = q.shape[0], q.shape[1], q.shape[2], v.shape[2]
    if state is None:
        S, n, m = torch.zeros(H, d, e, dtype=DT), torch.zeros(H, d, dtype=DT), torch.zeros(H, dtype=DT)
    else:
        S, n, m = state["S"].clone(), state["n"].clone(), state["m"].clone()
    o = torch.zeros(T, H, e, dtype=DT)
    for t in range(T):
        m_new = torch.maximum(gf[t] + m, gi[t])
        keep, take = torch.exp(gf[t] + m - m_new), torch.exp(gi[t] - m_new)
        S = keep[:, None, None] * S + take[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        n = keep[:, None] * n + take[:, None] * k[t]
        m = m_new
        below = torch.maximum((n * q[t]).sum(-1).abs(), torch.exp(-m)) + 1e-6
        o[t] = torch.einsum("hde,hd->he", S, q[t]) / below[:, None]
    return o, {"S": S, "n": n, "m": m}


def matrix_memory(p: dict, w: Dict[str, torch.Tensor], pre: str, h: torch.Tensor, eps: float, state: Optional[dict]):
    T, H, d, e = h.shape[0], p["heads"], p["dim"], p["vdim"]
    q = (h @ w[pre + "q"].T).view(T, H, d) * d ** -0.5
    k = (h @ w[pre + "k"].T).view(T, H, d)
    v = (h @ w[pre + "v"].T).view(T, H, e)
    gi, gf = log_gates(h @ w[pre + "i"].T, h @ w[pre + "f"].T, w[pre + "i.b"], w[pre + "f.b"], p["gate_cap"])
    o, new_state = exp_gate_recurrence(q, k, v, gi, gf, state)
    y = rms_unit(o, eps).reshape(T, H * e) * w[pre + "norm"] * torch.sigmoid(h @ w[pre + "g"].T)
    return y @ w[pre + "o"].T, new_state


def parallel_mixer(p: dict, w, pre: str, h, start: int, eps: float, state: Optional[dict]):
    left, ls = sink_attention(p["left"], w, pre + "left.", h, start, eps, None if state is None else state["left"])
    right, rs = matrix_memory(p["right"], w, pre + "right.", h, eps, None if state is None else state["right"])
    return p["left_scale"] * left + p["right_scale"] * right, {"left": ls, "right": rs}


# ---------------------------------------------------------------------------------------------
# feed-forwards
# ---------------------------------------------------------------------------------------------
def gated_ff(w, pre: str, h: torch.Tensor) -> torch.Tensor:
    return (silu(h @ w[pre + "gate"].T) * (h @ w[pre + "up"].T)) @ w[pre + "down"].T


MARGINS: List[float] = []       # the smallest gap of logits that a choice of experts or of groups rested on, per call


def choose_experts(z: torch.Tensor, top: int, groups: Optional[dict]):
    """z [T, E] router logits.  Scores are the softmax over all experts; experts outside the `keep` groups with the
    largest best score cannot be chosen; the `top` largest remaining scores are taken as they are."""
    T, E = z.shape
    s = torch.softmax(z, dim=-1)
    allowed = torch.ones(T, E, dtype=torch.bool)
    if groups is not None:
        count, keep = groups["count"], groups["keep"]
        best = s.view(T, count, E // count).max(dim=-1).values
        kept = torch.zeros(T, count, dtype=torch.bool)
        kept.scatter_(1, best.topk(keep, dim=-1).indices, True)
        allowed = kept[:, :, None].expand(T, count, E // count).reshape(T, E)
        if keep < count:
            ranked = z.view(T, count, E // count).max(dim=-1).values.sort(dim=-1, descending=True).values
            MARGINS.append(float((ranked[:, keep - 1] - ranked[:, keep]).min()))
    chosen = torch.where(allowed, s, torch.full_like(s, -1.0)).topk(top, dim=-1).indices
    ranked = torch.where(allowed, z, torch.full_like(z, -1e30)).sort(dim=-1, descending=True).values
    if top < int(allowed[0].sum()):
        MARGINS.append(float((ranked[:, top - 1] - ranked[:, top]).min()))
    return chosen, s.gather(1, chosen)


def expert_ff(m: dict, w, pre: str, h: torch.Tensor) -> torch.Tensor:
    r = m["router"]
    chosen, weight = choose_experts(h @ w[pre + "router"].T, r["top"], r.get("groups"))
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(r["top"]):
            out[t] += weight[t, j] * gated_ff(w, f"{pre}e{int(chosen[t, j])}.", h[t:t + 1])[0]
    if m.get("shared") is not None:
        out = out + gated_ff(w, pre + "shared.", h) * torch.sigmoid(h @ w[pre + "shared.sg"].T)
    return out


# ---------------------------------------------------------------------------------------------
# the whole model
# ---------------------------------------------------------------------------------------------
def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: List[int], state: Optional[dict] = None, start: int = 0,
            layers_out: Optional[list] = None, rounded: bool = False):
    """Logits [T, vocab] of `tokens` at positions start .., from `state` (None: a sequence's beginning), and the
    state after them.  `layers_out` collects the residual stream after every layer.  `rounded`: what every norm hands
    to the products behind it is rounded to bfloat16 values, the one rounding of a bfloat16 engine that reaches the
    recurrent mixers (their projections, gates and states are 32-bit from there on)."""
    eps = cfg["norm"]["eps"]
    handed = (lambda h: h.to(torch.bfloat16).to(DT)) if rounded else (lambda h: h)
    x = w["embed"][torch.tensor(tokens)]
    new_state = {}
    for i, layer in enumerate(cfg["layers"]):
        pre = f"l{layer.get('weights_of', i)}."
        h = handed(rms_unit(x, eps) * w[pre + "norm1"])
        st = None if state is None else state[i]
        kind, p = layer["type"], layer["mixer"]
        if kind == "attention":
            y, new_state[i] = temperature_attention(p, w, pre + "mix.", h, start, eps, st)
        elif kind == "gla":
            y, new_state[i] = gated_linear_attention(p, w, pre + "mix.", h, eps, st)
        elif kind == "parallel":
            y, new_state[i] = parallel_mixer(p, w, pre + "mix.", h, start, eps, st)
        else:
            raise ValueError(kind)
        x = x + y
        m = layer.get("mlp")
        if m is not None:
            h = handed(rms_unit(x, eps) * w[pre + "norm2"])
            x = x + (gated_ff(w, pre + "mlp.", h) if m["kind"] == "dense" else expert_ff(m, w, pre + "mlp.", h))
        if layers_out is not None:
            layers_out.append(x.clone())
    logits = handed(rms_unit(x, eps) * w["final.norm"]) @ w["head"].T
    cap = cfg.get("logit_softcap")
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return logits, new_state


def greedy(cfg: dict, w, prompt: List[int], n: int) -> List[int]:
    logits, state = forward(cfg, w, prompt)
    out, pos = [], len(prompt)
    for _ in range(n):
        out.append(int(torch.argmax(logits[-1])))
        logits, state = forward(cfg, w, out[-1:], state, pos)
        pos += 1
    return out


def forward_in_pieces(cfg: dict, w, tokens: List[int], pieces: List[int]) -> torch.Tensor:
    """The same logits, the tokens fed in portions of the given sizes from the state the portions before left."""
    out, state, at = [], None, 0
    for n in pieces:
        logits, state = forward(cfg, w, tokens[at:at + n], state, at)
        out.append(logits)
        at += n
    assert at == len(tokens)
    return torch.cat(out)


# ---------------------------------------------------------------------------------------------
# random weights and model folders
# ---------------------------------------------------------------------------------------------
def random_weights(cfg: dict, seed: int, rank: int = 6) -> Dict[str, torch.Tensor]:
    """Random tensors for a configuration, rounded to bfloat16 values (as a stored model's are).  `rank`: rows of a
    gated-linear-attention layer's first decay matrix (the configuration does not give it)."""
    g = torch.Generator().manual_seed(seed)
    W = int(cfg["width"])

    def rnd(*shape, s=1.0, mean=0.0):
        return (torch.randn(*shape, generator=g) * s + mean).to(torch.bfloat16).to(DT)

    def attention(m: str, a: dict, normed: bool):
        H, G, d, e = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
        w[m + "q"], w[m + "k"], w[m + "v"] = rnd(H * d, W, s=W ** -0.5), rnd(G * d, W, s=W ** -0.5), rnd(G * e, W, s=W ** -0.5)
        w[m + "o"] = rnd(W, H * e, s=(H * e) ** -0.5)
        if normed:
            w[m + "q.norm"], w[m + "k.norm"] = rnd(d, s=0.2, mean=1.0), rnd(d, s=0.2, mean=1.0)

    def linear_qkvgo(m: str, r: dict):
        H, d, e = r["heads"], r["dim"], r["vdim"]
        w[m + "q"], w[m + "k"], w[m + "v"] = rnd(H * d, W, s=W ** -0.5), rnd(H * d, W, s=W ** -0.5), rnd(H * e, W, s=W ** -0.5)
        w[m + "g"], w[m + "o"] = rnd(H * e, W, s=W ** -0.5), rnd(W, H * e, s=(H * e) ** -0.5)

    def gated(m: str, F: int):
        w[m + "gate"], w[m + "up"], w[m + "down"] = rnd(F, W, s=W ** -0.5), rnd(F, W, s=W ** -0.5), rnd(W, F, s=F ** -0.5)

    w = {"embed": rnd(cfg["vocab"], W), "final.norm": rnd(W, s=0.1, mean=1.0), "head": rnd(cfg["vocab"], W, s=W ** -0.5)}
    for i, layer in enumerate(cfg["layers"]):
        if layer.get("weights_of") is not None:
            continue
        p, mx = f"l{i}.", layer["mixer"]
        w[p + "norm1"] = rnd(W, s=0.1, mean=1.0)
        if layer["type"] == "attention":
            attention(p + "mix.", mx, True)
        elif layer["type"] == "gla":
            m = p + "mix."
            linear_qkvgo(m, mx)
            H, d = mx["heads"], mx["dim"]
            rk = mx.get("rank", rank)
            w[m + "a1"], w[m + "a2"] = rnd(rk, W, s=W ** -0.5), rnd(H * d, rk, s=2.0 * rk ** -0.5)
            w[m + "a2.b"], w[m + "norm"] = rnd(H * d, s=1.0, mean=2.0), rnd(mx["vdim"], s=0.1, mean=1.0)
        else:
            attention(p + "mix.left.", mx["left"], False)
            m, r = p + "mix.right.", mx["right"]
            linear_qkvgo(m, r)
            H = r["heads"]
            w[m + "i"], w[m + "f"] = rnd(H, W, s=2.0 * W ** -0.5), rnd(H, W, s=2.0 * W ** -0.5)
            w[m + "i.b"], w[m + "f.b"] = rnd(H, s=1.0), rnd(H, s=1.0, mean=2.0)
            w[m + "norm"] = rnd(H * r["vdim"], s=0.1, mean=1.0)
        mlp = layer.get("mlp")
        if mlp is None:
            continue
        w[p + "norm2"] = rnd(W, s=0.1, mean=1.0)
        if mlp["kind"] == "dense":
            gated(p + "mlp.", mlp["ff"])
            continue
        w[p + "mlp.router"] = rnd(mlp["router"]["experts"], W, s=2.0 * W ** -0.5)
        for x in range(mlp["router"]["experts"]):
            gated(p + f"mlp.e{x}.", mlp["expert"]["ff"])
        if mlp.get("shared") is not None:
            gated(p + "mlp.shared.", mlp["shared"]["ff"])
            w[p + "mlp.shared.sg"] = rnd(1, W, s=2.0 * W ** -0.5)
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
