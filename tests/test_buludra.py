"""The Buludra design in the library against the plain implementation of `plain_buludra.py`: small configurations made
here (sizes and options that differ from each other in every respect), random weights, every comparison on logits or on
one mechanism's output.  CPU tests cover the plain implementation itself, the configuration reader and the model
description; GPU tests cover the kernels one mechanism at a time and the engine: prompts, portions, single tokens,
unequal batches, slots and pages used again, far keys, the first tokens, long decoding, generation."""
import copy
import json
import math
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_buludra as P
from helpers import BF16_TOL, FP32_TOL, ROOT, random_tokens, rel_err


def tol_for(dtype):
    """The float32 engine is held to the library's float32 bound.  In bfloat16 the models here are 36 to 128 wide and
    deep in roundings (norms of heads, products, gates, two mixers a layer): twice the library's bound; a key seen or
    missed by mistake, a lost state or a sink left out moves these logits by far more (the tests below show it)."""
    return FP32_TOL if dtype == "float32" else 2 * BF16_TOL


class Judge:
    """How the engine's rows are held against the plain logits.  The float32 engine: every block of rows within the
    library's float32 bound.  The bfloat16 engine: the rows of a whole test together, against the plain implementation
    with its norms' outputs rounded to bfloat16.  This design has places where rounding alone moves a row far: at a
    sequence's first positions a matrix memory's output is S^T q over a divisor that follows |n . q|, and the head's
    norm then stretches whatever is left to unit length, so a query nearly at right angles to the few keys so far
    turns the rounding of the layer's input into the sign of that head's output, and the states of the layers behind
    carry it on (a drawn configuration with key size 4 moves its first row by 0.68 of the largest logit that way, in
    the engine and in the plain implementation with that one rounding alike).  With the same rounding on both sides
    what is left are the engine's other roundings (queries, cached keys and values, softmax weights, activations
    between products): most rows must be within the bound (all but one in twenty), and no row as far off as a missed
    key, a lost state or a sink left out puts it (the cases below show how far that is)."""

    def __init__(self, dtype):
        self.dtype, self.rows = dtype, []

    def add(self, out, ref, what=None):
        if self.dtype == "float32":
            assert rel_err(out, ref) < FP32_TOL, what
            return
        got, want = np.asarray(out, dtype=np.float64), np.asarray(ref, dtype=np.float64)
        assert got.shape == want.shape and np.isfinite(got).all(), what
        scale = np.abs(want).max() + 1e-12
        self.rows += [(float(np.abs(g - r).max() / scale), what) for g, r in zip(got, want)]

    def done(self):
        if self.dtype == "float32" or not self.rows:
            return
        errs = sorted(self.rows, key=lambda x: -x[0])
        over = [e for e in errs if e[0] >= tol_for(self.dtype)]
        assert len(over) <= max(1, len(errs) // 20), (len(over), len(errs), errs[:5])
        assert errs[0][0] < 0.35, errs[:5]


def attention(heads, kv_heads, dim, vdim, scale, q_temp=None):
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale)
    if q_temp:
        m["q_temp"] = dict(coef=q_temp[0], every=q_temp[1])
    return m


def gla(heads, dim, vdim, tau, rank):
    return dict(heads=heads, dim=dim, vdim=vdim, tau=tau, rank=rank)


def side_by_side(left, rot, right, left_scale, right_scale):
    left = dict(left)
    if rot:
        left["rot"] = dict(dims=rot[0], base=rot[1])
    return dict(left=left, right=dict(zip(("heads", "dim", "vdim", "gate_cap"), right)), left_scale=left_scale,
                right_scale=right_scale)


def dense(ff):
    return dict(kind="dense", ff=ff)


def moe(ff, experts, top, groups=None, shared=None):
    router = dict(experts=experts, top=top)
    if groups:
        router["groups"] = dict(count=groups[0], keep=groups[1])
    m = dict(kind="moe", expert=dict(ff=ff), router=router)
    if shared:
        m["shared"] = dict(ff=shared)
    return m


def layer(kind, mixer, mlp=None, weights_of=None):
    d = dict(type=kind, mixer=mixer, mlp=mlp)
    if weights_of is not None:
        d["weights_of"] = weights_of
    return d


# every mixer; a layer run twice with the same tensors; part of every head rotated; experts in groups with a shared one,
# and all experts of a layer chosen; a layer without a feed-forward; a temperature that steps every 7 positions
_A1 = layer("attention", attention(4, 1, 16, 8, 0.25, (0.4, 7)), moe(48, 6, 2, (3, 2), 40))
CFG_A = dict(architecture="Buludra", vocab=160, width=64, norm=dict(eps=1e-5), logit_softcap=8.0,
             layers=[layer("parallel", side_by_side(attention(4, 2, 16, 24, 0.3), (8, 1000.0), (2, 8, 16, 8.0), 0.7, 1.2), dense(96)),
                     _A1,
                     layer("gla", gla(3, 8, 16, 4.0, 5)),
                     dict(_A1, weights_of=1),
                     layer("parallel", side_by_side(attention(2, 2, 32, 16, 0.15), None, (3, 16, 8, 15.0), 1.0, 0.5), moe(32, 4, 4))])
# values that happen to be 1 or equal: one head, one group that is kept, one expert a token, a temperature every
# position, rotation of the whole head, as many key/value heads as heads, no cap on the logits
_B2 = layer("parallel", side_by_side(attention(3, 3, 8, 8, 0.5), (8, 50.0), (1, 24, 40, 3.0), 1.0, 1.0), dense(40))
CFG_B = dict(architecture="Buludra", vocab=200, width=96, norm=dict(eps=1e-6),
             layers=[layer("gla", gla(1, 24, 40, 1.0, 1), dense(64)),
                     layer("attention", attention(3, 3, 8, 32, 0.5, (0.2, 1)), moe(40, 4, 1, (1, 1))),
                     _B2,
                     dict(_B2, weights_of=2),
                     layer("attention", attention(6, 2, 24, 16, 0.2), moe(64, 3, 1, None, 24))])
# widths that are multiples of nothing: the bfloat16 products run on zero-padded operands, loads are scalar
CFG_C = dict(architecture="Buludra", vocab=75, width=36, norm=dict(eps=1e-5), logit_softcap=30.0,
             layers=[layer("parallel", side_by_side(attention(2, 1, 10, 7, 0.3), (6, 100.0), (3, 5, 9, 6.0), 0.9, 0.8), moe(13, 4, 2, (2, 1), 11)),
                     layer("gla", gla(2, 7, 5, 16.0, 3), dense(22)),
                     layer("attention", attention(3, 3, 6, 11, 0.4, (0.3, 64)))])
# sizes that the tensor-core kernels take (the first layer's experts as grouped products); key sizes above 64 and 128
CFG_D = dict(architecture="Buludra", vocab=128, width=128, norm=dict(eps=1e-5), logit_softcap=15.0,
             layers=[layer("parallel", side_by_side(attention(8, 2, 32, 64, 0.18), (32, 250000.0), (4, 32, 32, 12.0), 0.8, 0.9), moe(128, 8, 2, (4, 2), 128)),
                     layer("gla", gla(2, 72, 64, 8.0, 16), dense(256)),
                     layer("attention", attention(4, 4, 64, 64, 0.125, (0.3, 16)), moe(32, 4, 3, None, 64)),
                     layer("parallel", side_by_side(attention(4, 1, 64, 32, 0.125), (16, 10000.0), (1, 136, 16, 20.0), 0.5, 1.5), None)])
CONFIGS = {"A": CFG_A, "B": CFG_B, "C": CFG_C, "D": CFG_D}
TAGS = 4          # features that carry a token's class for the routers (see `decisive`)


def sharpened(w, factor=2.0):
    """Attention with normed heads made peaked, so that a key that is wrongly seen or missed moves the logits: the
    queries' norm weight is what scales the scores.  (The unit-norm attention is peaked by its configured scale.)"""
    out = dict(w)
    for name in w:
        if name.endswith(".mix.q.norm"):
            out[name] = (w[name] * factor).to(torch.bfloat16).to(P.DT)
    return out


def decisive(cfg, w):
    """Routers whose choice no rounding turns: the last TAGS features of the residual stream carry the token's class
    (id mod TAGS) from the embedding, no sublayer writes them (the rows of every last product that would are zero),
    and a router reads next to nothing else: every class has its own order of the experts with gaps between their
    logits."""
    out = dict(w)
    W = cfg["width"]
    emb = w["embed"].clone()
    emb[:, W - TAGS:] = 0.0
    for tok in range(cfg["vocab"]):
        emb[tok, W - TAGS + tok % TAGS] = 4.0
    out["embed"] = emb
    for name in w:
        if name.endswith(".o") or name.endswith(".down"):
            t = w[name].clone()
            t[W - TAGS:] = 0.0
            out[name] = t
    for i, lay in enumerate(cfg["layers"]):
        if lay.get("mlp") is None or lay["mlp"]["kind"] != "moe" or lay.get("weights_of") is not None:
            continue
        E = lay["mlp"]["router"]["experts"]
        r = (w[f"l{i}.mlp.router"] * 0.03).to(torch.bfloat16).to(P.DT)
        g = torch.Generator().manual_seed(1000 + i)
        for c in range(TAGS):
            order = torch.randperm(E, generator=g)
            r[order, W - TAGS + c] = (torch.linspace(-1.0, 1.0, E, dtype=P.DT) * 0.5 * E / 3.0).to(torch.bfloat16).to(P.DT)
        out[f"l{i}.mlp.router"] = r
    return out


def weights_for(cfg, seed, sharpen=2.0):
    return decisive(cfg, sharpened(P.random_weights(cfg, seed), sharpen))


def folder(tmp_path, cfg, seed, sharpen=2.0):
    w = weights_for(cfg, seed, sharpen)
    d = P.save_folder(cfg, w, str(tmp_path / f"model{seed}"))
    return d, w


def plain_logits(cfg, w, ids, dtype="float32"):
    """The plain implementation's logits, with the check that no router's choice was a close call.  For the bfloat16
    engine the plain implementation rounds what its norms hand on to bfloat16 too (see `Judge`)."""
    P.MARGINS.clear()
    out, _ = P.forward(cfg, w, list(ids), rounded=dtype == "bfloat16")
    assert not P.MARGINS or min(P.MARGINS) > 0.02, min(P.MARGINS)
    return out


# ------------------------------------------------------------------------------------------------
# without a device
# ------------------------------------------------------------------------------------------------
def test_the_plain_implementation_gives_the_same_logits_in_pieces():
    for name, cfg in CONFIGS.items():
        w = weights_for(cfg, 3)
        ids = random_tokens(90, cfg["vocab"], 7)
        whole = plain_logits(cfg, w, ids)
        pieces = P.forward_in_pieces(cfg, w, ids, [1, 1, 2, 3, 60, 1, 22])
        assert float((whole - pieces).abs().max()) < 1e-9, name


def test_the_plain_mechanisms_follow_their_definitions_on_cases_done_by_hand():
    one = lambda *x: torch.tensor(x, dtype=P.DT)  # noqa: E731
    # a sink: one key of score ln 3 weighs 3 / (1 + 3); without it the key takes everything
    q, k, v = one([[1.0]]).view(1, 1, 1), one([[math.log(3.0)]]).view(1, 1, 1), one([[8.0]]).view(1, 1, 1)
    assert abs(float(P.causal_attention(q, k, v, 0, 1.0, True)) - 6.0) < 1e-12
    assert abs(float(P.causal_attention(q, k, v, 0, 1.0, False)) - 8.0) < 1e-12
    # the temperature counts the positions from 1: with every = 3, positions 0, 1 give 1 and position 2 gives 1 + c ln 2
    t = P.query_temperature(torch.arange(7), 0.5, 3)
    assert torch.allclose(t, one(1.0, 1.0, 1 + 0.5 * math.log(2), 1 + 0.5 * math.log(2), 1 + 0.5 * math.log(2),
                                 1 + 0.5 * math.log(3), 1 + 0.5 * math.log(3)))
    # rotation pairs dimension i with i + dims / 2 and leaves the rest: a quarter turn at position 1 with frequency pi / 2
    x = one(1.0, 2.0, 3.0, 4.0, 5.0).view(1, 1, 5)
    y = P.rotate_half(x, torch.tensor([1]), 4, 1.0)          # base 1: every frequency is 1, the angle is 1
    c, s = math.cos(1.0), math.sin(1.0)
    assert torch.allclose(y.flatten(), one(1 * c - 3 * s, 2 * c - 4 * s, 3 * c + 1 * s, 4 * c + 2 * s, 5.0))
    # the decay acts on the rows of the state that belong to key channels; the output is read after the write
    qq, kk = one([1.0, 1.0]).view(1, 1, 2), one([2.0, 3.0]).view(1, 1, 2)
    vv, al = one([1.0, 10.0, 100.0]).view(1, 1, 3), one([0.5, 0.25]).view(1, 1, 2)
    o1, S1 = P.decay_recurrence(qq, kk, vv, al)
    assert torch.allclose(S1[0], torch.outer(kk[0, 0], vv[0, 0])) and torch.allclose(o1[0, 0], 5.0 * vv[0, 0])
    o2, S2 = P.decay_recurrence(qq, kk, vv, al, S1)
    assert torch.allclose(S2[0], torch.outer(one(3.0, 3.75), vv[0, 0])) and torch.allclose(o2[0, 0], 6.75 * vv[0, 0])
    # sigmoid(z)^(1/tau): z = 0, tau = 2 gives sqrt(1/2)
    assert abs(float(P.channel_decays(one(0.0), one(1.0).view(1, 1), one(0.0), 2.0)) - 0.5 ** 0.5) < 1e-12
    # exponential gates: the maximum starts at 0 (not at minus infinity), so after a forget gate of -0.5 and an input
    # gate of -2 it is -0.5, the input is taken as exp(-1.5) and the divisor is max(|n . q|, exp(0.5)) + 1e-6; a second
    # token with input gate 3 raises the maximum to 3
    gi, gf = one([-2.0]).view(1, 1), one([-0.5]).view(1, 1)
    o, st = P.exp_gate_recurrence(qq, kk, vv, gi, gf)
    take = math.exp(-1.5)
    assert abs(float(st["m"]) + 0.5) < 1e-12 and torch.allclose(st["n"][0], take * kk[0, 0])
    assert torch.allclose(o[0, 0], take * 5.0 * vv[0, 0] / (max(take * 5.0, math.exp(0.5)) + 1e-6))
    o, st2 = P.exp_gate_recurrence(qq, kk, vv, one([3.0]).view(1, 1), gf, st)
    keep = math.exp(-0.5 - 0.5 - 3.0)
    assert abs(float(st2["m"]) - 3.0) < 1e-12 and torch.allclose(st2["n"][0], (keep * take + 1.0) * kk[0, 0])
    nq = (keep * take + 1.0) * 5.0
    assert torch.allclose(o[0, 0], nq * vv[0, 0] / (max(nq, math.exp(-3.0)) + 1e-6))
    # the gates are capped before they are used
    a, b = P.log_gates(one(100.0), one(100.0), one(0.0), one(0.0), 2.0)
    assert abs(float(a) - 2.0) < 1e-9 and abs(float(b) - float(P.log_sigmoid(one(2.0)))) < 1e-9
    # the choice: softmax scores, the best `keep` groups by their best expert, then the best experts among them
    z = one([0.0, 5.0, 4.0, 4.5, 1.0, 1.5])
    chosen, weight = P.choose_experts(z, 2, dict(count=3, keep=1))
    assert sorted(chosen[0].tolist()) == [0, 1] and torch.allclose(weight.sum(), torch.softmax(z, -1)[0, :2].sum())
    chosen, _ = P.choose_experts(z, 2, dict(count=3, keep=2))
    assert sorted(chosen[0].tolist()) == [1, 3]
    chosen, _ = P.choose_experts(z, 2, None)
    assert sorted(chosen[0].tolist()) == [1, 3]
    chosen, _ = P.choose_experts(z, 3, dict(count=2, keep=1))
    assert sorted(chosen[0].tolist()) == [0, 1, 2]
    # the weight multiplies the expert's OUTPUT and the shared expert is gated by one number per token
    W = 2
    wts = {"m.router": one([0.0, 0.0], [1.0, 0.0]), "m.shared.sg": one([0.0, 1.0]).view(1, 2)}
    for name in ("e0", "e1", "shared"):
        wts[f"m.{name}.gate"], wts[f"m.{name}.up"] = torch.eye(W, dtype=P.DT), torch.ones(W, W, dtype=P.DT)
        wts[f"m.{name}.down"] = torch.eye(W, dtype=P.DT) * (3.0 if name == "e1" else 1.0)
    h = one([1.0, -2.0]).view(1, 2)
    base = P.silu(h[0]) * h[0].sum()
    s = torch.softmax(one(0.0, 1.0), -1)
    got = P.expert_ff(dict(router=dict(experts=2, top=2)), wts, "m.", h)
    assert torch.allclose(got[0], s[0] * base + s[1] * 3.0 * base)
    got = P.expert_ff(dict(router=dict(experts=2, top=1), shared=dict(ff=2)), wts, "m.", h)
    assert torch.allclose(got[0], s[1] * 3.0 * base + base / (1.0 + math.exp(2.0)))


def test_configuration_is_read_by_key_and_written_back():
    from janus_b200.config import ConfigError, resolve_architecture
    for cfg in CONFIGS.values():
        arch = resolve_architecture(cfg)
        c = arch.config_class.from_dict(cfg)
        assert json.loads(json.dumps(c.to_dict())) == json.loads(json.dumps(cfg))
    arch = resolve_architecture(CFG_A)
    c = arch.config_class.from_dict(CFG_A)
    assert c.layers[2].mlp is None and c.layers[1].mlp.top == 2 and c.layers[1].mlp.groups == 3 and c.layers[1].mlp.keep == 2
    assert c.layers[4].mixer.left.rot_dims == 0 and c.layers[0].mixer.left.rot_dims == 8 and c.layers[3].weights_of == 1
    assert c.owner(3) == 1 and c.owner(4) == 4 and c.layers[4].mlp.shared_ff == 0 and c.logit_softcap == 8.0
    assert arch.config_class.from_dict(CFG_B).logit_softcap == 0.0
    # a layer may name a layer that itself uses another's tensors: the chain ends at the one that has them
    chain = copy.deepcopy(CFG_A)
    chain["layers"].append(dict(copy.deepcopy(_A1), weights_of=3))
    assert [arch.config_class.from_dict(chain).owner(i) for i in range(6)] == [0, 1, 2, 1, 4, 1]
    # the rank of a decay's projection is what the tensor's shape says, where there is a tensor
    c2 = c.with_tensor_shapes(lambda name: (9, 64) if name == "l2.mix.a1" else None)
    assert c2.layers[2].mixer.rank == 9 and c.layers[2].mixer.rank == 5
    for path, value, word in ((("layers", 0, "type"), "serial", "type"), (("layers", 0, "mlp", "kind"), "sparse", "kind"),
                              (("layers", 0, "mixer", "left", "kv_heads"), 3, "heads"), (("norm",), None, "norm"),
                              (("layers", 0, "mixer", "left", "rot", "dims"), 7, "dims"),
                              (("layers", 1, "mlp", "router", "top"), 7, "top"),
                              (("layers", 1, "mlp", "router", "groups", "count"), 4, "groups"),
                              (("layers", 1, "mlp", "router", "groups", "keep"), 4, "groups"),
                              (("layers", 3, "weights_of"), 3, "weights_of"), (("layers", 3, "weights_of"), 2, "layers"),
                              (("layers", 3, "weights_of"), 9, "weights_of"),
                              (("layers", 0, "mixer", "right"), None, "right"), (("layers", 2, "mixer", "tau"), -1.0, "tau")):
        bad = copy.deepcopy(CFG_A)
        at = bad
        for k in path[:-1]:
            at = at[k]
        at[path[-1]] = value
        with pytest.raises(ConfigError, match=word):
            arch.config_class.from_dict(bad)


def test_the_model_description_names_every_tensor_once_and_gives_every_run_its_own_place():
    from janus_b200.config import resolve_architecture
    from janus_b200.models.buludra import buludra_spec
    for cfg in CONFIGS.values():
        arch = resolve_architecture(cfg)
        c = arch.config_class.from_dict(cfg)
        names = {s.name: tuple(s.shape) for s in arch.weight_specs(c)}
        want = {k: tuple(v.shape) for k, v in P.random_weights(cfg, 0).items()}
        assert names == want
    c = resolve_architecture(CFG_A).config_class.from_dict(CFG_A)
    spec = buludra_spec(c)
    assert len(spec.layers) == 4 and [e.layer for e in spec.schedule] == [0, 1, 2, 1, 3]
    assert spec.layers[2].feed_forward is None and spec.layers[2].feed_forward_norm is None
    names = {s.name for s in resolve_architecture(CFG_A).weight_specs(c)}
    assert "l2.norm2" not in names and "l3.norm1" not in names and "l1.mlp.shared.sg" in names


def sink_case(seed=5):
    """A model of one layer of two mixers side by side whose attention branch alone speaks (the other's factor is 0),
    and a prompt: whatever the sink takes from the softmax's weights shows in the logits."""
    cfg = dict(architecture="Buludra", vocab=64, width=32, norm=dict(eps=1e-5),
               layers=[layer("parallel", side_by_side(attention(2, 1, 8, 8, 0.2), (4, 100.0), (1, 4, 4, 5.0), 1.5, 0.0))])
    return cfg, P.random_weights(cfg, seed), random_tokens(70, 64, seed)


def far_token_case(kind, seed=6):
    """A model of one recurrent layer and two prompts that differ in their first token only.  The first token's key
    is made loud in one key channel (its embedding has a feature that no other token has, and the key projection
    reads it), and the last token's query asks for that channel: what the last position says, 300 tokens on, is what
    the state kept of the first token's value."""
    mixer = (gla(2, 8, 8, 64.0, 4) if kind == "gla"
             else side_by_side(attention(2, 1, 8, 8, 0.2), None, (2, 8, 8, 10.0), 0.0, 1.0))
    cfg = dict(architecture="Buludra", vocab=64, width=32, norm=dict(eps=1e-5), layers=[layer(kind, mixer)])
    w = P.random_weights(cfg, seed)
    m = "l0.mix." if kind == "gla" else "l0.mix.right."
    if kind == "gla":
        w[m + "a2.b"] = w[m + "a2.b"] + 4.0          # slow decays: about sigmoid(6)^(1/64) a token
    else:
        w[m + "f.b"] = w[m + "f.b"] + 6.0
    first_a, first_b, last = 0, 1, 2
    emb = w["embed"].clone()
    emb[:, 30:] = 0.0
    emb[first_b, :30] = -emb[first_a, :30]             # opposite values
    emb[first_a, 30] = emb[first_b, 30] = emb[last, 31] = 6.0
    w["embed"] = emb
    for name, col in ((m + "k", 30), (m + "q", 31)):
        t = w[name].clone()
        t[:, 30:] = 0.0
        t[0, col] = 8.0 if col == 31 else 48.0
        w[name] = t
    w[m + "o"] = (w[m + "o"] * 4.0).to(torch.bfloat16).to(P.DT)          # the mixer speaks up beside the embedding
    middle = [3 + t % 61 for t in random_tokens(298, 64, seed)]
    return cfg, w, [first_a] + middle + [last], [first_b] + middle + [last]


def test_the_cases_made_for_the_sink_and_for_far_tokens_show_in_the_plain_logits():
    cfg, w, ids = sink_case()
    with_sink = plain_logits(cfg, w, ids)
    original = P.causal_attention
    try:
        P.causal_attention = lambda q, k, v, start, scale, sink: original(q, k, v, start, scale, False)
        without = plain_logits(cfg, w, ids)
    finally:
        P.causal_attention = original
    assert rel_err(without, with_sink) > 5 * BF16_TOL
    assert rel_err(without[40:50], with_sink[40:50]) > FP32_TOL * 10   # behind 40 keys it still shows to the float32 engine
    for kind in ("gla", "parallel"):
        cfg, w, a, b = far_token_case(kind)
        assert rel_err(plain_logits(cfg, w, a)[-1:], plain_logits(cfg, w, b)[-1:]) > 4 * BF16_TOL, kind


# ------------------------------------------------------------------------------------------------
# on the device: one mechanism at a time
# ------------------------------------------------------------------------------------------------
gpu = pytest.mark.gpu


def load(d, dtype, max_tokens=2048, **kw):
    import janus_b200
    return janus_b200.load(d, dtype=dtype, max_tokens=max_tokens, **kw)


@gpu
def test_the_weighted_join_of_two_branches_and_the_row_gate_against_their_formulas():
    from janus_b200.kernels import ops
    g = torch.Generator().manual_seed(0)
    for T, W in ((7, 64), (5, 36), (3, 200), (1, 8)):
        r, ya, yb = (torch.randn(T, W, generator=g) for _ in range(3))
        rd, yad, ybd = r.cuda(), ya.cuda(), yb.cuda()
        ops.join_norm(rd, ya=yad, yb=ybd, mult=0.7, mult_b=-1.3)
        assert rel_err(rd.cpu(), r.to(P.DT) + 0.7 * ya.to(P.DT) - 1.3 * yb.to(P.DT)) < 1e-6
        assert float(yad.abs().sum()) == 0.0 and float(ybd.abs().sum()) == 0.0
        for dtype, tol in ((torch.float32, 1e-6), (torch.bfloat16, 1e-2)):
            x = torch.randn(T, W, generator=g).to(dtype)
            wide = torch.randn(T, 5, generator=g)
            xd = x.cuda()
            ops.scale_rows_sigmoid(xd, wide.cuda()[:, 3])
            assert rel_err(xd.float().cpu(), x.to(P.DT) * torch.sigmoid(wide[:, 3:4].to(P.DT))) < tol


@gpu
def test_head_preparation_with_a_weightless_norm_and_with_a_temperature_against_the_plain_steps():
    """Queries and cache rows as the two attention mixers make them: rotation of part of the head, then the division
    by the root mean square; and normed heads with weights, no rotation, times the temperature of the position."""
    from janus_b200.kernels import ops
    from janus_b200.parts.base import PartSpec, make_part
    g = torch.Generator().manual_seed(1)
    for H, G, d, e, rot in ((4, 2, 16, 24, 8), (2, 1, 10, 7, 6), (3, 3, 8, 8, 8), (2, 2, 64, 32, 0)):
        T, D = 9, max(d, e)
        positions = torch.tensor([0, 1, 5, 6, 7, 62, 63, 64, 700], dtype=torch.int32)
        proj = torch.randn(T, H * d + G * (d + e) + 3, generator=g)
        q64 = proj[:, :H * d].to(P.DT).view(T, H, d)
        k64 = proj[:, H * d:(H + G) * d].to(P.DT).view(T, G, d)
        v64 = proj[:, (H + G) * d:(H + G) * d + G * e].to(P.DT).view(T, G, e)
        dest = torch.tensor([3, 64, 65, 2, 1, 0, 130, 131, 70], dtype=torch.int32)
        for mode in ("unit", "temperature"):
            kc, vc = torch.zeros(3, G, 64, D, device="cuda"), torch.zeros(3, G, 64, D, device="cuda")
            q_out = torch.full((T, H * D), 7.0, device="cuda")
            if mode == "unit":
                table = None
                if rot:
                    part = make_part("position", PartSpec("ramped_rotary", dict(dims=rot, theta=100.0, max_positions=1024,
                                                                                scaling=None)), torch.float32, torch.device("cuda"))
                    table = part.fused_rotary_table()
                ops.head_norm_rope_cache(proj.cuda(), None, None, 1e-5, table, rot, positions.cuda(), q_out, dest.cuda(), kc, vc,
                                         H, G, d, e, D, 64, unit_norm=True)
                qw = P.rms_unit(P.rotate_half(q64, positions, rot, 100.0) if rot else q64, 1e-5)
                kw = P.rms_unit(P.rotate_half(k64, positions, rot, 100.0) if rot else k64, 1e-5)
            else:
                wq, wk = torch.randn(d, generator=g), torch.randn(d, generator=g)
                ops.head_norm_rope_cache(proj.cuda(), wq.cuda(), wk.cuda(), 1e-5, None, 0, positions.cuda(), q_out, dest.cuda(),
                                         kc, vc, H, G, d, e, D, 64, temp_coef=0.3, temp_every=7)
                qw = P.rms_unit(q64, 1e-5) * wq.to(P.DT) * P.query_temperature(positions, 0.3, 7)[:, None, None]
                kw = P.rms_unit(k64, 1e-5) * wk.to(P.DT)
            got_q = q_out.cpu().view(T, H, D)
            assert rel_err(got_q[:, :, :d], qw) < 1e-5 and float(got_q[:, :, d:].abs().sum()) == 0.0, (mode, H, d)
            rows_k = kc.cpu().permute(0, 2, 1, 3).reshape(3 * 64, G, D)[dest.long()]
            rows_v = vc.cpu().permute(0, 2, 1, 3).reshape(3 * 64, G, D)[dest.long()]
            assert rel_err(rows_k[:, :, :d], kw) < 1e-5 and rel_err(rows_v[:, :, :e], v64) < 1e-6, (mode, H, d)


def _pages(lens, nkv, hd, g, dtype=torch.bfloat16):
    """Keys and values of sequences of the given lengths laid out in pages out of order, with a block table."""
    n_pages = sum((n + 63) // 64 for n in lens) + 3
    order = torch.randperm(n_pages, generator=g).tolist()
    kc = torch.zeros(n_pages, nkv, 64, hd, dtype=dtype)
    vc = torch.zeros_like(kc)
    table = torch.zeros(len(lens), max((n + 63) // 64 for n in lens) + 1, dtype=torch.int32)
    ks, vs = [], []
    for i, n in enumerate(lens):
        k = torch.randn(n, nkv, hd, generator=g).to(dtype)
        v = torch.randn(n, nkv, hd, generator=g).to(dtype)
        ks.append(k)
        vs.append(v)
    return kc, vc, table, ks, vs, order


def _fill(kc, vc, table, ks, vs, order):
    for i, (k, v) in enumerate(zip(ks, vs)):
        n = k.shape[0]
        for pg in range((n + 63) // 64):
            page = order.pop()
            table[i, pg] = page
            rows = slice(pg * 64, min(n, pg * 64 + 64))
            kc[page, :, : rows.stop - rows.start] = k[rows].transpose(0, 1)
            vc[page, :, : rows.stop - rows.start] = v[rows].transpose(0, 1)


@gpu
@pytest.mark.parametrize("nh,nkv,hd", [(8, 2, 64), (4, 4, 128), (6, 2, 32), (4, 1, 24)])
def test_prompt_attention_kernels_with_a_sink_against_the_plain_softmax(nh, nkv, hd):
    """The tensor-core prompt kernel, the mma.sync one and the float32 one on the same pages: a prompt from position 0
    (whose first tokens see one, two, three keys beside the sink) and a portion that starts at position 300 of a
    longer sequence.  One key far back, the last of a page, is made loud for the last queries: its value must come
    through, weighed against the sink."""
    from janus_b200.kernels import ops
    g = torch.Generator().manual_seed(hd)
    scale = 1.5 * hd ** -0.5
    lens, starts = (333, 500), (0, 300)
    kc, vc, table, ks, vs, order = _pages(lens, nkv, hd, g)
    qs, want = [], []
    for i, (n, start) in enumerate(zip(lens, starts)):
        q = torch.randn(n - start, nh, hd, generator=g).to(torch.bfloat16)
        if i == 1:
            ks[i][63] = ks[i][63] * 0.0 + 3.0                   # key 63, the last row of the sequence's first page
            q[-5:] = q[-5:].abs()                               # the last queries point its way
            vs[i][63] = 5.0
        qs.append(q)
        want.append(P.causal_attention(q.to(P.DT), ks[i].to(P.DT), vs[i].to(P.DT), start, scale, True))
    _fill(kc, vc, table, ks, vs, order)
    assert float(want[1][-1].mean()) > 2.0                      # the loud key's value dominates there
    q = torch.cat(qs).reshape(-1, nh * hd).cuda()
    want = torch.cat(want).reshape(-1, nh * hd)
    q_start = torch.tensor([0, lens[0] - starts[0], lens[0] - starts[0] + lens[1] - starts[1]], dtype=torch.int32).cuda()
    kv_len = torch.tensor(lens, dtype=torch.int32).cuda()
    out = torch.zeros_like(q)
    args = (q, kc.cuda(), vc.cuda(), out, table.cuda(), q_start, kv_len, 2, lens[0], nh, nkv, hd, 64, 0, scale)
    if ops.attention_tc_supported(nh, nkv, hd):
        ops.attention_tc_prefill(*args, sink=True)
        assert rel_err(out.float().cpu(), want) < 1e-2
        out.zero_()
    ops.attention_bf16_prefill(*args, sink=True)
    assert rel_err(out.float().cpu(), want) < 1e-2
    token_seq = torch.tensor([0] * (lens[0] - starts[0]) + [1] * (lens[1] - starts[1]), dtype=torch.int32).cuda()
    positions = torch.cat([torch.arange(starts[i], lens[i], dtype=torch.int32) for i in range(2)]).cuda()
    out32 = torch.zeros(q.shape, device="cuda")
    ops.attention_f32(q.float(), kc.float().cuda(), vc.float().cuda(), out32, table.cuda(), token_seq, positions, nh, nkv,
                      hd, 64, 0, scale, sink=True)
    assert rel_err(out32.cpu(), want) < 1e-5
    # without the flag the kernels still give the ordinary softmax
    ops.attention_f32(q.float(), kc.float().cuda(), vc.float().cuda(), out32, table.cuda(), token_seq, positions, nh, nkv,
                      hd, 64, 0, scale)
    plain = torch.cat([P.causal_attention(qs[i].to(P.DT), ks[i].to(P.DT), vs[i].to(P.DT), starts[i], scale, False)
                       for i in range(2)]).reshape(-1, nh * hd)
    assert rel_err(out32.cpu(), plain) < 1e-5 and rel_err(plain, want) > 0.05
    ops.check_kernel_status(q.device)


@gpu
@pytest.mark.parametrize("nh,nkv,hd", [(8, 2, 64), (4, 4, 128), (6, 1, 32)])
def test_single_token_attention_with_a_sink_whole_and_in_splits(nh, nkv, hd):
    """One query a sequence over 1, 2, 64, 65 and 900 keys: the kernel alone and with the keys cut into splits that a
    second kernel joins (the sink is counted once, where they are joined).  A loud key at a page's first row."""
    from janus_b200.engine.workspace import Workspace
    from janus_b200.kernels import ops
    g = torch.Generator().manual_seed(hd + 1)
    scale = 1.5 * hd ** -0.5
    lens = (1, 2, 64, 65, 900)
    kc, vc, table, ks, vs, order = _pages(lens, nkv, hd, g)
    ks[4][128] = 3.0
    vs[4][128] = -4.0
    q = torch.randn(len(lens), nh, hd, generator=g).to(torch.bfloat16)
    q[4] = q[4].abs()
    _fill(kc, vc, table, ks, vs, order)
    want = torch.cat([P.causal_attention(q[i:i + 1].to(P.DT), ks[i].to(P.DT), vs[i].to(P.DT), n - 1, scale, True)
                      for i, n in enumerate(lens)]).reshape(len(lens), nh * hd)
    assert float(want[4].mean()) < -2.0
    ws = Workspace(torch.device("cuda"))
    kv_len = torch.tensor(lens, dtype=torch.int32).cuda()
    for splits in (1, 2, 5):
        out = torch.zeros(len(lens), nh * hd, dtype=torch.bfloat16, device="cuda")
        ops.attention_bf16_decode(q.reshape(len(lens), nh * hd).cuda(), kc.cuda(), vc.cuda(), out, table.cuda(), kv_len, nh,
                                  nkv, hd, 64, 0, scale, ws, max(lens), n_splits=splits, sink=True)
        assert rel_err(out.float().cpu(), want) < 1e-2, splits


def _step_tensors(lengths, slots):
    q_start = torch.tensor([0] + list(np.cumsum(lengths)), dtype=torch.int32, device="cuda")
    return q_start, torch.tensor(slots, dtype=torch.int32, device="cuda")


@gpu
@pytest.mark.parametrize("H,d,e", [(4, 8, 16), (3, 5, 9), (2, 64, 64), (1, 200, 24), (2, 32, 40), (2, 96, 130), (1, 256, 16),
                                   (2, 33, 65)])
@pytest.mark.parametrize("kind", ["decays", "gates"])
@pytest.mark.parametrize("lead", [1, 0])
def test_the_recurrence_kernels_against_the_plain_recurrences(lead, kind, H, d, e):
    """Three sequences of unequal lengths in slots out of order: a prompt step (one sequence long enough to run in
    segments), a second portion from the state the first left, then single tokens; outputs, the divisors' effect and
    the final state against the plain recurrence run in one piece.  With decays per key channel, and with exponential
    gates, a normalizer and a running maximum."""
    from janus_b200.engine.workspace import Workspace
    from janus_b200.kernels import ops
    g = torch.Generator().manual_seed(d * 100 + e + lead)
    gates = kind == "gates"
    total, slots = (700, 3, 71), [2, 0, 3]
    rank, tau, cap = 3, 8.0, 6.0
    ld = 2 * H * d + H * e + (2 * H if gates else rank) + lead
    ld += 0 if lead else -ld % 4
    q_col, k_col, v_col, x_col = lead, lead + H * d, lead + 2 * H * d, lead + 2 * H * d + H * e
    seqs = [torch.randn(n, ld, generator=g) for n in total]
    for s in seqs:
        s[:, x_col:] *= 3.0
    a2 = torch.randn(H * d, rank, generator=g)
    a2_bias = torch.randn(H * d, generator=g) + 2.0
    bias_i, bias_f = torch.randn(H, generator=g), torch.randn(H, generator=g) + 2.0
    per_head = d * (e + 1) if gates else d * e
    state = torch.zeros(5, H * per_head + (H if gates else 0) + 2, device="cuda")
    ws = Workspace(torch.device("cuda"))
    got = [[] for _ in total]
    at = [0, 0, 0]
    for portion in ((600, 2, 40), (97, 0, 29), (1, 1, 1), (1, 0, 1), (1, 0, 0)):
        live = [i for i, n in enumerate(portion) if n]
        proj = torch.cat([seqs[i][at[i]:at[i] + portion[i]] for i in live]).cuda()
        lengths = [portion[i] for i in live]
        q_start, seq_slot = _step_tensors(lengths, [slots[i] for i in live])
        T = proj.shape[0]
        out = torch.empty(T, H * e, device="cuda")
        if gates:
            gate_buf = torch.empty(T, H, 4, device="cuda")
            ops.exp_gates(proj, x_col, x_col + H, bias_i.cuda(), bias_f.cuda(), cap, gate_buf, state, H * per_head, q_start,
                          seq_slot, len(live), H)
            den = torch.empty(T, H, device="cuda")
            ops.gated_linear_scan(proj, q_col, k_col, v_col, d ** -0.5, gate_buf, out, state, q_start, seq_slot, len(live), H,
                                  d, e, max(lengths), ws, divisors=den)
            out = out.view(T, H, e) / den.view(T, H, 1)
        else:
            dec = torch.empty(T, H * d, device="cuda")
            ops.gla_decay(proj, x_col, rank, a2.t().contiguous().cuda(), a2_bias.cuda(), tau, dec)
            ops.gated_linear_scan(proj, q_col, k_col, v_col, d ** -0.5, dec, out, state, q_start, seq_slot, len(live), H, d, e,
                                  max(lengths), ws)
        out = out.reshape(T, H * e).cpu()
        row = 0
        for i in live:
            got[i].append(out[row:row + portion[i]])
            row += portion[i]
            at[i] += portion[i]
    assert at == list(total)
    for i, s in enumerate(seqs):
        s64, n = s.to(P.DT), s.shape[0]
        q = s64[:, q_col:k_col].view(n, H, d) * d ** -0.5
        k, v = s64[:, k_col:v_col].view(n, H, d), s64[:, v_col:x_col].view(n, H, e)
        kept = state[slots[i]].cpu()
        if gates:
            gi, gf = P.log_gates(s64[:, x_col:x_col + H], s64[:, x_col + H:x_col + 2 * H], bias_i.to(P.DT), bias_f.to(P.DT), cap)
            o, st = P.exp_gate_recurrence(q, k, v, gi, gf)
            heads = kept[:H * per_head].view(H, per_head)
            assert rel_err(heads[:, :d * e].reshape(H, d, e), st["S"]) < 5e-5, i
            assert rel_err(heads[:, d * e:], st["n"]) < 5e-5 and rel_err(kept[H * per_head:H * per_head + H], st["m"]) < 1e-5, i
        else:
            alpha = P.channel_decays(s64[:, x_col:x_col + rank], a2.to(P.DT), a2_bias.to(P.DT), tau).view(n, H, d)
            o, S = P.decay_recurrence(q, k, v, alpha)
            assert rel_err(kept[:H * d * e].view(H, d, e), S) < 5e-5, i
        assert rel_err(torch.cat(got[i]), o.reshape(n, H * e)) < 5e-5, i
    assert float(state[1].abs().sum()) == 0.0 and float(state[4].abs().sum()) == 0.0      # slots nobody had
    assert float(state[:, -2:].abs().sum()) == 0.0                                         # nothing behind the state


@gpu
def test_head_norm_with_divisors_and_a_weight_per_head_against_its_formula():
    from janus_b200.kernels import ops
    g = torch.Generator().manual_seed(2)
    for T, H, e in ((6, 3, 9), (4, 2, 64), (2, 5, 8), (3, 1, 40)):
        o = torch.randn(T, H * e, generator=g) * 4
        wide = torch.randn(T, H * e + 5, generator=g)
        weight = torch.randn(H * e, generator=g)
        den = torch.rand(T, H, generator=g) * 3 + 0.1
        want = (P.rms_unit(o.to(P.DT).view(T, H, e) / den.to(P.DT)[:, :, None], 1e-5).reshape(T, H * e) * weight.to(P.DT)
                * torch.sigmoid(wide[:, 3:3 + H * e].to(P.DT)))
        out = torch.empty(T, H * e, device="cuda")
        ops.head_norm_gate(o.cuda(), wide.cuda()[:, 3:3 + H * e], weight.cuda(), 1e-5, out, H, e, sigmoid=True, denom=den.cuda())
        assert rel_err(out.cpu(), want) < 1e-5


@gpu
def test_router_with_softmax_scores_and_groups_and_experts_weighted_on_their_outputs():
    from janus_b200.kernels import ops
    g = torch.Generator().manual_seed(3)
    for T, E, top, groups in ((50, 12, 3, (3, 2)), (9, 6, 2, (3, 1)), (7, 8, 8, None), (40, 40, 4, (8, 3)), (5, 4, 1, (1, 1)),
                              (11, 6, 3, (2, 1))):
        z = torch.randn(T, E + 1, generator=g) * 2            # one more column rides along and is not an expert
        want_e, want_w = P.choose_experts(z[:, :E].to(P.DT), top, dict(count=groups[0], keep=groups[1]) if groups else None)
        sel_e = torch.empty(T, top, dtype=torch.int32, device="cuda")
        sel_w = torch.empty(T, top, device="cuda")
        ops.route_topk(z.cuda(), top, sel_e, sel_w, softmax=True, groups=groups[0] if groups else 0,
                       keep=groups[1] if groups else 0, experts=E)
        assert sel_e.cpu().tolist() == want_e.tolist()          # both take the largest first
        assert rel_err(sel_w.cpu(), want_w) < 1e-5
    for T, W, F, E, top, dtype in ((9, 64, 48, 5, 2, torch.float32), (1, 36, 13, 4, 4, torch.float32),
                                   (20, 64, 32, 6, 3, torch.bfloat16)):
        wts = {"m.router": torch.randn(E, W, generator=g).to(torch.bfloat16).to(P.DT)}
        for x in range(E):
            wts[f"m.e{x}.gate"] = (torch.randn(F, W, generator=g) * W ** -0.5).to(torch.bfloat16).to(P.DT)
            wts[f"m.e{x}.up"] = (torch.randn(F, W, generator=g) * W ** -0.5).to(torch.bfloat16).to(P.DT)
            wts[f"m.e{x}.down"] = (torch.randn(W, F, generator=g) * F ** -0.5).to(torch.bfloat16).to(P.DT)
        h = torch.randn(T, W, generator=g).to(torch.bfloat16)
        want = P.expert_ff(dict(router=dict(experts=E, top=top)), wts, "m.", h.to(P.DT))
        zz = (h.to(P.DT) @ wts["m.router"].T).float().cuda()
        sel_e = torch.empty(T, top, dtype=torch.int32, device="cuda")
        sel_w = torch.empty(T, top, device="cuda")
        ops.route_topk(zz, top, sel_e, sel_w, softmax=True)
        stack = lambda kind: torch.stack([wts[f"m.e{x}.{kind}"] for x in range(E)]).to(dtype).cuda().contiguous()  # noqa: E731
        out = torch.zeros(T, W, device="cuda")
        act = torch.empty(T * top, F, device="cuda")
        ops.experts_few_tokens(h.to(dtype).cuda(), sel_e, sel_w, stack("gate"), stack("up"), stack("down"), act, out,
                               weight_on_output=True)
        assert rel_err(out.cpu(), want) < (1e-5 if dtype == torch.float32 else 1e-2), (T, W, F, E, top)
        # the pairs in the experts' order and back: rows gathered as they are, a weighted sum per token
        chosen = sel_e.reshape(-1).cpu().numpy()
        order = np.argsort(chosen, kind="stable").astype(np.int32)
        where = np.empty(T * top, dtype=np.int32)
        where[order] = np.arange(T * top, dtype=np.int32)
        rows = torch.empty(T * top, W, dtype=dtype, device="cuda")
        ops.expert_gather(h.to(dtype).cuda(), torch.from_numpy(order).cuda(), None, top, rows)
        assert torch.equal(rows.cpu(), h.to(dtype)[torch.from_numpy(order).long() // top])
        results = torch.randn(T * top, W, generator=g)
        acc = torch.zeros(T, W, device="cuda")
        ops.expert_scatter(results.cuda(), torch.from_numpy(where).cuda(), top, acc, weights=sel_w)
        want_acc = (results[torch.from_numpy(where).long()].view(T, top, W).to(P.DT) * sel_w.cpu().to(P.DT)[:, :, None]).sum(1)
        assert rel_err(acc.cpu(), want_acc) < 1e-5


# ------------------------------------------------------------------------------------------------
# on the device: the engine
# ------------------------------------------------------------------------------------------------
def _one_mixer(cfg, which):
    """A model of one layer with that layer's mixer alone (no feed-forward)."""
    lay = dict(copy.deepcopy(cfg["layers"][which]), mlp=None)
    lay.pop("weights_of", None)
    return dict(cfg, layers=[lay])


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", [0, 1, 2, 4])
def test_each_mixer_alone_in_a_layer_without_feed_forward(tmp_path, which, dtype):
    from janus_b200.engine import StepEntry
    cfg = _one_mixer(CFG_A, which)
    d, w = folder(tmp_path, cfg, 20 + which)
    model = load(d, dtype, max_tokens=512, max_slots=2)
    ids = random_tokens(150, cfg["vocab"], which)
    ref = plain_logits(cfg, w, ids, dtype)
    slot = model.alloc_slot()
    out = [model.step([StepEntry(slot, ids[:100], range(100))]).cpu(), model.step([StepEntry(slot, ids[100:140], range(40))]).cpu()]
    out += [model.step([StepEntry(slot, [t], [0])]).cpu() for t in ids[140:]]
    judge = Judge(dtype)
    judge.add(torch.cat(out), ref)
    judge.done()
    model.check()


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_whole_prompts_of_unequal_lengths_in_one_step(tmp_path, name, dtype):
    from janus_b200.engine import StepEntry
    cfg = CONFIGS[name]
    d, w = folder(tmp_path, cfg, 11)
    model = load(d, dtype, max_tokens=64 * 16, max_slots=4)
    seqs = [random_tokens(n, cfg["vocab"], n) for n in (1, 64, 330, 129)]
    slots = [model.alloc_slot() for _ in seqs]
    out = model.step([StepEntry(s, ids, range(len(ids))) for s, ids in zip(slots, seqs)]).cpu()
    row, judge = 0, Judge(dtype)
    for ids in seqs:
        judge.add(out[row:row + len(ids)], plain_logits(cfg, w, ids, dtype), len(ids))
        row += len(ids)
    model.check()
    judge.done()


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_portions_then_single_tokens_in_a_batch_and_slots_used_again(tmp_path, name, dtype):
    """Prompts cut into portions of 2 to 64 tokens, unequal requests in one batch, then one token each until the
    shorter ones have ended; afterwards other requests take the freed slots and pages (and find the recurrences'
    states, normalizers and running maxima zeroed).  Every row is compared with the whole sequence's plain logits."""
    from janus_b200.engine import StepEntry
    cfg = CONFIGS[name]
    d, w = folder(tmp_path, cfg, 12)
    judge = Judge(dtype)
    model = load(d, dtype, max_tokens=64 * 9, max_slots=3)
    for round_no, lengths in enumerate(((140, 75, 20), (90, 130, 129))):
        seqs = [random_tokens(n, cfg["vocab"], 7 * round_no + n) for n in lengths]
        ref = [plain_logits(cfg, w, ids, dtype) for ids in seqs]
        slots = [model.alloc_slot() for _ in seqs]
        at = [0, 0, 0]
        for portion in ((2, 3, 2), (62, 5, 3), (1, 40, 2), (17, 2, 2)):
            entries, spans = [], []
            for i, n in enumerate(portion):
                entries.append(StepEntry(slots[i], seqs[i][at[i]:at[i] + n], range(n)))
                spans.append((i, at[i], n))
                at[i] += n
            out = model.step(entries).cpu()
            row = 0
            for i, lo, n in spans:
                judge.add(out[row:row + n], ref[i][lo:lo + n], (round_no, i, lo, n))
                row += n
        live = [0, 1, 2]
        while live:
            out = model.step([StepEntry(slots[i], [seqs[i][at[i]]], [0]) for i in live]).cpu()
            for row, i in enumerate(live):
                judge.add(out[row:row + 1], ref[i][at[i]:at[i] + 1], (round_no, i, at[i]))
                at[i] += 1
            for i in [i for i in live if at[i] == len(seqs[i])]:
                model.free_slot(slots[i])
                live.remove(i)
        model.engine.cache.check()
    model.check()
    judge.done()


def drawn_config(seed):
    """A configuration drawn from a seed: two to five layers of any mixer, feed-forward or none, sizes that are
    multiples of nothing as often as not, a layer that uses another's tensors now and then."""
    r = np.random.RandomState(seed)
    pick = lambda *xs: xs[r.randint(len(xs))]  # noqa: E731
    W = int(pick(32, 40, 64, 72, 36, 128))
    layers = []
    for i in range(r.randint(2, 6)):
        if layers and r.rand() < 0.2:
            j = r.randint(len(layers))
            if "weights_of" not in layers[j]:
                layers.append(dict(layers[j], weights_of=j))
                continue
        kind = pick("attention", "gla", "parallel")
        G = int(pick(1, 2, 3))
        H = G * int(pick(1, 2, 3))
        d, e = int(pick(4, 8, 10, 16, 24, 32, 40)), int(pick(4, 8, 9, 16, 24, 32))
        if kind == "attention":
            mixer = attention(H, G, d, e, float(pick(0.2, 0.3, d ** -0.5)), pick(None, (0.3, int(pick(1, 5, 64))), (0.1, 3)))
        elif kind == "gla":
            mixer = gla(int(pick(1, 2, 3)), d, e, float(pick(1.0, 4.0, 16.0)), int(pick(1, 2, 5, 8)))
        else:
            rot = pick(None, (2 * (1 + r.randint(d // 2)), float(pick(50.0, 10000.0))))
            mixer = side_by_side(attention(H, G, d, e, float(pick(0.1, 0.2, 0.3))), rot,
                                 (int(pick(1, 2, 4)), int(pick(4, 8, 12, 40)), int(pick(4, 8, 20, 72)), float(pick(3.0, 8.0, 15.0))),
                                 float(pick(0.5, 0.8, 1.0)), float(pick(0.9, 1.0, 1.3)))
        which = r.randint(4)
        if which == 0:
            mlp = None
        elif which == 1:
            mlp = dense(int(pick(24, 40, 64, 100)))
        else:
            count = int(pick(1, 2, 3, 4))
            per = int(pick(1, 2, 3))
            keep = 1 + r.randint(count)
            top = 1 + r.randint(min(keep * per, 4))
            mlp = moe(int(pick(16, 24, 33, 64)), count * per, top, pick(None, (count, keep)), pick(None, int(pick(8, 20, 32))))
        layers.append(layer(kind, mixer, mlp))
    return dict(architecture="Buludra", vocab=int(pick(50, 97, 128)), width=W, norm=dict(eps=float(pick(1e-5, 1e-6))),
                logit_softcap=pick(None, 10.0, 30.0), layers=layers)


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", list(range(1, 17)))
def test_configurations_drawn_from_a_seed(tmp_path, seed, dtype):
    """Whatever the sizes, the order of the layers and the options: a prompt, a portion, single tokens and a second
    request beside them give the plain logits."""
    from janus_b200.engine import StepEntry
    cfg = drawn_config(seed)
    cfg = {k: v for k, v in cfg.items() if v is not None}
    d, w = folder(tmp_path, cfg, 100 + seed)
    model = load(d, dtype, max_tokens=64 * 8, max_slots=2)
    a, b = random_tokens(150, cfg["vocab"], seed), random_tokens(40, cfg["vocab"], seed + 50)
    ra, rb = plain_logits(cfg, w, a, dtype), plain_logits(cfg, w, b, dtype)
    sa, sb = model.alloc_slot(), model.alloc_slot()
    judge, text = Judge(dtype), json.dumps(cfg)
    out = model.step([StepEntry(sa, a[:70], range(70)), StepEntry(sb, b[:33], [0, 32])]).cpu()
    judge.add(out[:70], ra[:70], text)
    judge.add(out[70:], rb[[0, 32]], text)
    out = model.step([StepEntry(sa, a[70:143], range(73))]).cpu()
    judge.add(out, ra[70:143], text)
    for j in range(7):
        out = model.step([StepEntry(sa, [a[143 + j]], [0]), StepEntry(sb, [b[33 + j]], [0])]).cpu()
        judge.add(out[:1], ra[143 + j:144 + j], text)
        judge.add(out[1:], rb[33 + j:34 + j], text)
    model.check()
    judge.done()


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_batch_gives_every_request_what_it_gets_alone(tmp_path, dtype):
    """The engine against itself: four unequal requests in one batch (prompt, then single tokens) and each alone, on
    slots and pages that other requests held before; rows differ by rounding at most."""
    from janus_b200.engine import StepEntry
    cfg = CFG_A
    d, _ = folder(tmp_path, cfg, 13)
    model = load(d, dtype, max_tokens=64 * 12, max_slots=4)
    seqs = [random_tokens(n, cfg["vocab"], 50 + n) for n in (100, 3, 65, 31)]
    alone = []
    for ids in seqs:
        slot = model.alloc_slot()
        rows = [model.step([StepEntry(slot, ids[:-2], [len(ids) - 3])]).cpu()] if len(ids) > 2 else []
        rows += [model.step([StepEntry(slot, [t], [0])]).cpu() for t in ids[max(len(ids) - 2, 0):]] if len(ids) > 2 else \
            [model.step([StepEntry(slot, ids[:1], [0])]).cpu()] + [model.step([StepEntry(slot, [t], [0])]).cpu() for t in ids[1:]]
        alone.append(torch.cat(rows))
        model.free_slot(slot)
    slots = [model.alloc_slot() for _ in seqs]
    first = model.step([StepEntry(s, ids[:-2], [len(ids) - 3]) for s, ids in zip(slots, seqs)]).cpu()
    tails = [model.step([StepEntry(s, [ids[len(ids) - 2 + j]], [0]) for s, ids in zip(slots, seqs)]).cpu() for j in range(2)]
    slack = 1e-5 if dtype == "float32" else BF16_TOL
    for i, ids in enumerate(seqs):
        together = torch.stack([first[i], tails[0][i], tails[1][i]])
        assert rel_err(together, alone[i][-3:]) < slack, i
    model.check()


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_sink_shows_and_a_far_token_reaches_through_the_states(tmp_path, dtype):
    from janus_b200.engine import StepEntry
    cfg, w, ids = sink_case()
    d = P.save_folder(cfg, w, str(tmp_path / "sink"))
    model = load(d, dtype, max_tokens=256, max_slots=2)
    ref = plain_logits(cfg, w, ids, dtype)
    slot = model.alloc_slot()
    out = torch.cat([model.step([StepEntry(slot, ids[:40], range(40))]).cpu()]
                    + [model.step([StepEntry(slot, [t], [0])]).cpu() for t in ids[40:]])
    judge = Judge(dtype)
    judge.add(out, ref, "sink")
    judge.done()
    # the far token's case is loud by large numbers (a key of some 200 among keys of 1), and float32 rounding grows
    # with them: twenty times the float32 bound, against an effect of 0.28 and more
    tol = 20 * FP32_TOL if dtype == "float32" else tol_for(dtype)
    for kind in ("gla", "parallel"):
        cfg, w, a, b = far_token_case(kind)
        d = P.save_folder(cfg, w, str(tmp_path / f"far_{kind}"))
        model = load(d, dtype, max_tokens=1024, max_slots=2)
        for ids in (a, b):
            ref = plain_logits(cfg, w, ids, dtype)
            slot = model.alloc_slot()
            got = [model.step([StepEntry(slot, ids[:280], [279])]).cpu()]
            got += [model.step([StepEntry(slot, [t], [0])]).cpu() for t in ids[280:]]
            assert rel_err(torch.cat(got), ref[279:]) < tol, kind
            model.free_slot(slot)


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "C"])
def test_long_decoding_from_the_first_token(tmp_path, name, dtype):
    """200 single tokens from position 0 on (the first tokens see little beside the sink; the temperature steps many
    times; pages fill and new ones are taken), two sequences a step, one of them a few tokens behind."""
    from janus_b200.engine import StepEntry
    cfg = CONFIGS[name]
    d, w = folder(tmp_path, cfg, 17)
    model = load(d, dtype, max_tokens=64 * 8, max_slots=2)
    a, b = random_tokens(200, cfg["vocab"], 1), random_tokens(195, cfg["vocab"], 2)
    ra, rb = plain_logits(cfg, w, a, dtype), plain_logits(cfg, w, b, dtype)
    sa, sb = model.alloc_slot(), model.alloc_slot()
    judge = Judge(dtype)
    for t in range(200):
        entries = [StepEntry(sa, [a[t]], [0])] + ([StepEntry(sb, [b[t - 5]], [0])] if t >= 5 else [])
        out = model.step(entries).cpu()
        judge.add(out[:1], ra[t:t + 1], ("a", t))
        if t >= 5:
            judge.add(out[1:], rb[t - 5:t - 4], ("b", t - 5))
    model.check()
    judge.done()


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_long_prompt_in_one_step_and_in_portions(tmp_path, dtype):
    """700 tokens: the recurrences run in segments, attention reads eleven pages; then the same prompt in portions of
    300, 257 and 143 tokens on a slot that was used before."""
    from janus_b200.engine import StepEntry
    cfg = CFG_D
    d, w = folder(tmp_path, cfg, 19)
    model = load(d, dtype, max_tokens=64 * 24, max_slots=2)
    ids = random_tokens(700, cfg["vocab"], 9)
    ref = plain_logits(cfg, w, ids, dtype)
    want = list(range(0, 700, 7)) + [699]
    slot = model.alloc_slot()
    out = model.step([StepEntry(slot, ids, want)]).cpu()
    judge = Judge(dtype)
    judge.add(out, ref[want], "one step")
    model.free_slot(slot)
    slot = model.alloc_slot()
    at, rows = 0, []
    for n in (300, 257, 143):
        rows.append(model.step([StepEntry(slot, ids[at:at + n], [w_ - at for w_ in want if at <= w_ < at + n])]).cpu())
        at += n
    judge.add(torch.cat(rows), ref[want], "portions")
    judge.done()
    model.check()


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_entry_point_and_the_scheduler(tmp_path, dtype):
    """`load` -> `generate`: five prompts in batches of two; every generated token is the plain implementation's
    pick given the tokens before it.  A folder made by `write_random_model` loads and generates too."""
    import janus_b200
    from janus_b200.weights import write_random_model
    d, w = folder(tmp_path, CFG_A, 31)
    model = janus_b200.load(d, dtype=dtype, max_tokens=1024, max_slots=4)
    prompts = [random_tokens(n, CFG_A["vocab"], 3 + n) for n in (5, 70, 1, 33, 12)]
    out, stats = model.generate(prompts, max_tokens=10, batch_size=2)
    assert stats.batches == 3
    for p, o in zip(prompts, out):
        assert len(o) == 10
        logits = plain_logits(CFG_A, w, list(p) + list(o), dtype)
        for j, tok in enumerate(o):
            row = logits[len(p) - 1 + j]
            slack = 1e-4 if dtype == "float32" else BF16_TOL
            assert float(row.max() - row[tok]) <= slack * float(row.abs().max()), (p, j)
    d2 = write_random_model(CFG_B, str(tmp_path / "gen"), seed=32, dtype="bfloat16", std=0.1, norm_std=0.05)
    cfg2, w2 = P.read_folder(d2)
    assert cfg2["layers"][1]["mlp"]["router"]["experts"] == 4 and set(w2) == set(P.random_weights(CFG_B, 0))
    model = janus_b200.load(d2, dtype=dtype, max_tokens=512, max_slots=2)
    out, _ = model.generate([[1, 2, 3], [4]], max_tokens=6, batch_size=2)
    assert [len(o) for o in out] == [6, 6] and all(0 <= t < CFG_B["vocab"] for o in out for t in o)


@gpu
def test_the_replay_program_serves_the_design(tmp_path):
    """Also from a folder whose configuration does not say the rank of the decay's projection: the tensor's shape does."""
    cfg = copy.deepcopy(CFG_C)
    del cfg["layers"][1]["mixer"]["rank"]
    w = weights_for(CFG_C, 14)
    d = P.save_folder(cfg, w, str(tmp_path / "model"))
    ids = random_tokens(40, cfg["vocab"], 2)
    other = random_tokens(33, cfg["vocab"], 3)
    steps = [dict(step=0, entries=[dict(id="x", tokens=ids[:30], want=[0, 29]), dict(id="y", tokens=other[:31], want=[30])],
                  end=[])]
    for j in range(10):
        entries = [dict(id="x", tokens=[ids[30 + j]], want=[0])]
        if j < 2:
            entries.append(dict(id="y", tokens=[other[31 + j]], want=[0]))
        steps.append(dict(step=j + 1, entries=entries, end=(["y"] if j == 1 else []) + (["x"] if j == 9 else [])))
    out = tmp_path / "out"
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", d, "--dtype", "float32",
                          "--out", str(out), "--max-tokens", "128"],
                         input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=900)
    assert res.returncode == 0, res.stderr[-2000:]
    got = np.concatenate([np.fromfile(out / f"{s['step']}.f32", dtype="<f4").reshape(-1, cfg["vocab"]) for s in steps])
    rx, ry = plain_logits(cfg, w, ids), plain_logits(cfg, w, other)
    want = [rx[0], rx[29], ry[30], rx[30], ry[31], rx[31], ry[32]] + [rx[t] for t in range(32, 40)]
    assert rel_err(got, torch.stack(want)) < FP32_TOL


@gpu
def test_the_command_line_samples_from_the_design(tmp_path):
    """`python -m janus_b200 DIR ...`: greedy tokens are the plain implementation's picks, and sampling with a
    temperature, top-k and a seed runs through the device sampler; a folder with config.json alone runs with
    `--random-weights`."""
    d, w = folder(tmp_path, CFG_D, 15)
    base = [sys.executable, "-m", "janus_b200", d, "3,1,4,1,5", "9,2,6", "--max-tokens", "7", "--dtype", "float32", "--json"]
    env = dict(os.environ, PYTHONPATH=os.pathsep.join([ROOT, os.environ.get("PYTHONPATH", "")]))
    res = subprocess.run(base, capture_output=True, text=True, timeout=900, env=env)
    assert res.returncode == 0, res.stderr[-2000:]
    greedy = json.loads(res.stdout.strip().splitlines()[-1])["tokens"]
    for p, o in zip(([3, 1, 4, 1, 5], [9, 2, 6]), greedy):
        assert len(o) == 7
        logits = plain_logits(CFG_D, w, p + o)
        assert all(int(logits[len(p) - 1 + j].argmax()) == tok for j, tok in enumerate(o))
    res = subprocess.run(base + ["--temperature", "0.9", "--top-k", "12", "--top-p", "0.9", "--seed", "4"],
                         capture_output=True, text=True, timeout=900, env=env)
    assert res.returncode == 0, res.stderr[-2000:]
    sampled = json.loads(res.stdout.strip().splitlines()[-1])["tokens"]
    assert [len(o) for o in sampled] == [7, 7] and all(0 <= t < CFG_D["vocab"] for o in sampled for t in o)
    only_config = tmp_path / "only_config"
    only_config.mkdir()
    (only_config / "config.json").write_text(json.dumps(CFG_A))
    res = subprocess.run([sys.executable, "-m", "janus_b200", str(only_config), "1,2,3", "--max-tokens", "4", "--random-weights",
                          "--json"], capture_output=True, text=True, timeout=900, env=env)
    assert res.returncode == 0, res.stderr[-2000:]
    assert len(json.loads(res.stdout.strip().splitlines()[-1])["tokens"][0]) == 4
