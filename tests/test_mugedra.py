"""The Mugedra design in the library against the plain implementation of `plain_mugedra.py`: small configurations
made here (sizes and options that differ from each other in every respect), random weights, every comparison on
logits or on one mechanism's output.  CPU tests cover the plain implementation itself, the configuration reader and
the model description; GPU tests cover the kernels one mechanism at a time and the engine: prompts, portions, single
tokens, unequal batches, slots and pages used again, the edges of the chunks, far tokens, generation."""
import copy
import json
import math
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_mugedra as P
from helpers import BF16_TOL, FP32_TOL, ROOT, random_tokens, rel_err


def tol_for(dtype):
    """The float32 engine is held to the library's float32 bound.  In bfloat16 the models here are 36 to 128 wide
    and deep in roundings (norms of heads and of branches, products, gates, several layers run up to three times):
    twice the library's bound; a key seen or missed by mistake moves these logits by far more (the tests on the
    chunks' edges show it)."""
    return FP32_TOL if dtype == "float32" else 2 * BF16_TOL


def left(heads, kv_heads, dim, vdim, scale, softcap=None, mask=None, rot=None):
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale)
    if softcap:
        m["softcap"] = softcap
    if mask:
        m["mask"] = dict(size=mask)
    if rot:
        m["rot"] = dict(dims=rot[0], base=rot[1])
        if len(rot) > 2:
            m["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), rot[2]))
    return m


def right(heads, kv_heads, dim, vdim, conv):
    return dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, conv=conv)


def layer(a, r, moe=None):
    mlp = None if moe is None else dict(kind="moe", expert=dict(ff=moe[0]), router=dict(experts=moe[1], top=moe[2]))
    return dict(type="parallel", mixer=dict(left=a, right=r), mlp=mlp)


# a loop of two layers run three times between a first and a last layer; two of five experts; part of every head
# rotated with a frequency ramp; chunks that are no multiple of anything, of exactly a page, and smaller than a tile
CFG_A = dict(architecture="Mugedra", vocab=160, width=64, norm=dict(eps=1e-5), loop=dict(start=1, stop=3, times=3),
             layers=[layer(left(4, 2, 16, 24, 0.3, softcap=4.0, mask=37, rot=(8, 1000.0, (2.0, 64, 8.0, 1.0))),
                           right(4, 2, 8, 16, 3), (48, 5, 2)),
                     layer(left(2, 1, 32, 16, 0.2, softcap=10.0, mask=64, rot=(32, 10000.0)), right(2, 2, 16, 8, 4)),
                     layer(left(4, 4, 8, 8, 0.5, mask=5), right(3, 1, 8, 24, 2), (32, 3, 3)),
                     layer(left(4, 1, 16, 16, 0.25, softcap=2.0, mask=70, rot=(16, 50.0, (8.0, 16, 4.0, 1.0))),
                           right(2, 1, 24, 8, 4), (40, 6, 4))])
# no loop; attention without cap, chunks or rotation; one tap; a single expert; a chunk of just over two pages
CFG_B = dict(architecture="Mugedra", vocab=200, width=96, norm=dict(eps=1e-6),
             layers=[layer(left(3, 3, 8, 32, 0.5), right(1, 1, 24, 8, 1), (40, 1, 1)),
                     layer(left(6, 2, 24, 16, 0.2, mask=130, rot=(24, 50.0)), right(6, 3, 8, 8, 5), (64, 4, 1)),
                     layer(left(2, 1, 16, 8, 0.3, softcap=30.0), right(2, 2, 32, 40, 2))])
# widths that are multiples of nothing: the bfloat16 products run on zero-padded operands, loads are scalar
CFG_C = dict(architecture="Mugedra", vocab=75, width=36, norm=dict(eps=1e-5), loop=dict(start=0, stop=1, times=2),
             layers=[layer(left(2, 1, 10, 7, 0.3, softcap=3.0, mask=33, rot=(6, 100.0)), right(3, 1, 5, 9, 3), (13, 4, 2)),
                     layer(left(3, 3, 6, 11, 0.4, mask=9), right(2, 2, 7, 5, 2), (22, 3, 1))])
# sizes that the tensor-core kernels take (the first layer's experts as grouped products, the second's one by one);
# the whole model is the loop
CFG_D = dict(architecture="Mugedra", vocab=128, width=128, norm=dict(eps=1e-5), loop=dict(start=0, stop=2, times=2),
             layers=[layer(left(8, 2, 32, 32, 0.18, softcap=20.0, mask=100, rot=(32, 250000.0, (8.0, 128, 32.0, 1.0))),
                           right(4, 2, 32, 32, 4), (128, 8, 2)),
                     layer(left(4, 4, 64, 64, 0.125, mask=192, rot=(16, 10000.0)), right(2, 1, 64, 64, 4), (32, 4, 3))])
CONFIGS = {"A": CFG_A, "B": CFG_B, "C": CFG_C, "D": CFG_D}
TAGS = 4          # features that carry a token's class for the routers (see `decisive`)


def sharpened(w, factor=2.0):
    """Attention made peaked, so that a key that is wrongly seen or missed moves the logits: heads are normed, so
    the queries' norm weight is what scales the scores."""
    out = dict(w)
    for name in w:
        if name.endswith(".left.q.norm"):
            out[name] = (w[name] * factor).to(torch.bfloat16).to(P.DT)
    return out


def decisive(cfg, w):
    """Routers whose choice no rounding turns: the last TAGS features of the residual stream carry the token's
    class (id mod TAGS) from the embedding, no sublayer writes them (their layer scales are zero), and a router
    reads next to nothing else: every class has its own order of the experts with gaps between their logits."""
    out = dict(w)
    W = cfg["width"]
    emb = w["embed"].clone()
    emb[:, W - TAGS:] = 0.0
    for tok in range(cfg["vocab"]):
        emb[tok, W - TAGS + tok % TAGS] = 4.0
    out["embed"] = emb
    for i, lay in enumerate(cfg["layers"]):
        for name in (f"l{i}.ls1", f"l{i}.ls2"):
            if name in w:
                t = w[name].clone()
                t[W - TAGS:] = 0.0
                out[name] = t
        if lay["mlp"] is None:
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


def plain_logits(cfg, w, ids):
    """The plain implementation's logits, with the check that no router's choice was a close call."""
    model = P.PlainMugedra(cfg, w)
    out = model.forward(ids)
    assert not model.margins or min(model.margins) > 0.02, min(model.margins)
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
    # one head, state from zero, two tokens: S1 = b1 k1 v1^T; o1 = (k1.q1) b1 v1; then the decay and the correction
    k1, k2 = torch.tensor([[[1.0, 0.0]]], dtype=P.DT), torch.tensor([[[0.6, 0.8]]], dtype=P.DT)
    q = torch.tensor([[[0.5, 0.5]]], dtype=P.DT)
    v1, v2 = torch.tensor([[[2.0, -1.0, 4.0]]], dtype=P.DT), torch.tensor([[[1.0, 1.0, 1.0]]], dtype=P.DT)
    beta, g = torch.tensor([[0.5]], dtype=P.DT), torch.tensor([[0.25]], dtype=P.DT)
    o1, S1 = P.delta_recurrence(q, k1, v1, beta, g)
    assert torch.allclose(S1[0], 0.5 * torch.outer(k1[0, 0], v1[0, 0])) and torch.allclose(o1[0, 0], 0.25 * v1[0, 0])
    o2, S2 = P.delta_recurrence(q, k2, v2, beta, g, S1)
    Sd = 0.25 * S1[0]
    want = Sd + torch.outer(k2[0, 0], 0.5 * (v2[0, 0] - Sd.T @ k2[0, 0]))
    assert torch.allclose(S2[0], want) and torch.allclose(o2[0, 0], want.T @ q[0, 0])
    # the convolution's last column meets the current token; zeros before the start; the tail carries over
    u = torch.tensor([[1.0], [2.0], [3.0]], dtype=P.DT)
    wgt = torch.tensor([[100.0, 10.0, 1.0]], dtype=P.DT)
    y, tail = P.short_conv(u, wgt, None)
    assert torch.allclose(y[:, 0], P.silu(torch.tensor([1.0, 12.0, 123.0], dtype=P.DT))) and tail[:, 0].tolist() == [2.0, 3.0]
    y2, _ = P.short_conv(torch.tensor([[4.0]], dtype=P.DT), wgt, tail)
    assert torch.allclose(y2[:, 0], P.silu(torch.tensor([234.0], dtype=P.DT)))
    # chunks are counted from position 0: with a chunk of 3, position 3 sees itself only, position 5 sees 3, 4, 5
    kk = torch.zeros(6, 1, 2, dtype=P.DT)
    vv = torch.arange(6, dtype=P.DT).view(6, 1, 1)
    out = P.chunk_softmax(torch.zeros(6, 1, 2, dtype=P.DT), kk, vv, 0, 1.0, None, 3)
    assert torch.allclose(out.flatten(), torch.tensor([0.0, 0.5, 1.0, 3.0, 3.5, 4.0], dtype=P.DT))
    # a cap bounds a score: two keys with scores 100 and 0 under a cap of 1 weigh e^tanh(100) : 1
    qq = torch.tensor([[[10.0]]], dtype=P.DT)
    kk = torch.tensor([[[0.0]], [[10.0]]], dtype=P.DT)
    out = P.chunk_softmax(qq, kk, torch.tensor([[[0.0]], [[1.0]]], dtype=P.DT), 1, 1.0, 1.0, None)
    assert abs(float(out) - math.e / (1 + math.e)) < 1e-9
    # the router's weight multiplies the expert's input: with top = all, out = sum_e expert_e(s_e h)
    h = torch.tensor([[1.0, -2.0]], dtype=P.DT)
    wts = {"router": torch.tensor([[0.0, 0.0], [1.0, 0.0]], dtype=P.DT)}
    for e in range(2):
        wts[f"e{e}.gate"], wts[f"e{e}.up"] = torch.eye(2, dtype=P.DT) * (e + 1), torch.ones(2, 2, dtype=P.DT)
        wts[f"e{e}.down"] = torch.eye(2, dtype=P.DT)
    got = P.routed_feed_forward(h, wts, 2, 2)
    want = torch.zeros(2, dtype=P.DT)
    for e, s in enumerate((0.5, 1.0 / (1.0 + math.exp(-1.0)))):
        x = s * h[0]
        want += P.silu((e + 1) * x) * x.sum()
    assert torch.allclose(got[0], want)
    top1 = P.routed_feed_forward(h, wts, 2, 1)
    x = h[0] / (1.0 + math.exp(-1.0))
    assert torch.allclose(top1[0], P.silu(2 * x) * x.sum())
    # the loop: layers 1 and 2 three times, the embedding joins before the second and third pass
    assert P.layer_runs(CFG_A) == [(0, False), (1, False), (2, False), (1, True), (2, False), (1, True), (2, False), (3, False)]
    assert P.layer_runs(CFG_B) == [(0, False), (1, False), (2, False)]
    assert P.layer_runs(CFG_C) == [(0, False), (0, True), (1, False)]


def test_configuration_is_read_by_key_and_written_back():
    from janus_b200.config import ConfigError, resolve_architecture
    for cfg in CONFIGS.values():
        arch = resolve_architecture(cfg)
        c = arch.config_class.from_dict(cfg)
        assert json.loads(json.dumps(c.to_dict())) == json.loads(json.dumps(cfg))
        assert [tuple(r) for r in c.runs()] == P.layer_runs(cfg)
    arch = resolve_architecture(CFG_A)
    c = arch.config_class.from_dict(CFG_A)
    assert c.layers[1].mlp is None and c.layers[0].mlp.top == 2 and c.layers[2].mixer.left.softcap == 0.0
    assert c.layers[2].mixer.left.rot is None and c.layers[0].mixer.left.chunk == 37 and c.loop.times == 3
    for path, value, word in ((("layers", 0, "type"), "serial", "type"), (("layers", 0, "mlp", "kind"), "dense", "kind"),
                              (("layers", 0, "mixer", "left", "kv_heads"), 3, "heads"),
                              (("layers", 0, "mixer", "right", "kv_heads"), 3, "heads"), (("norm",), None, "norm"),
                              (("layers", 0, "mixer", "left", "rot", "dims"), 7, "dims"),
                              (("layers", 0, "mlp", "router", "top"), 6, "top"), (("loop", "stop"), 5, "loop"),
                              (("layers", 0, "mixer", "right"), None, "right")):
        bad = copy.deepcopy(CFG_A)
        at = bad
        for k in path[:-1]:
            at = at[k]
        at[path[-1]] = value
        with pytest.raises(ConfigError, match=word):
            arch.config_class.from_dict(bad)


def test_the_model_description_names_every_tensor_once_and_gives_every_pass_its_own_place():
    from janus_b200.config import resolve_architecture
    from janus_b200.models.mugedra import mugedra_spec
    from janus_b200.parts import KVSpec, StateSpec
    for cfg in CONFIGS.values():
        arch = resolve_architecture(cfg)
        c = arch.config_class.from_dict(cfg)
        names = {s.name: tuple(s.shape) for s in arch.weight_specs(c)}
        want = {k: tuple(v.shape) for k, v in P.random_weights(cfg, 0).items()}
        assert names == want
    c = resolve_architecture(CFG_A).config_class.from_dict(CFG_A)
    spec = mugedra_spec(c)
    assert len(spec.layers) == 4 and [e.layer for e in spec.schedule] == [0, 1, 2, 1, 2, 1, 2, 3]
    assert [e.adds_embedding for e in spec.schedule] == [False, False, False, True, False, True, False, False]
    assert spec.layers[1].feed_forward is None and spec.layers[1].feed_forward_norm is None
    names = {s.name for s in resolve_architecture(CFG_A).weight_specs(c)}
    assert "l1.norm2" not in names and "l1.ls2" not in names and "l1.ls1" in names


# ------------------------------------------------------------------------------------------------
# on the device: one mechanism at a time
# ------------------------------------------------------------------------------------------------
gpu = pytest.mark.gpu


def load(d, dtype, max_tokens=2048, **kw):
    import janus_b200
    return janus_b200.load(d, dtype=dtype, max_tokens=max_tokens, **kw)


@gpu
def test_layer_norm_layer_scale_and_the_join_of_two_branches_against_their_formulas():
    from janus_b200.kernels import ops
    g = torch.Generator().manual_seed(0)
    for T, W in ((7, 64), (5, 36), (3, 200), (1, 8)):
        r = torch.randn(T, W, generator=g) * 3 + 1.5            # a mean far from zero: the norm centers
        ya, yb = torch.randn(T, W, generator=g), torch.randn(T, W, generator=g) * 5
        wa, wb, scale, gamma = (torch.randn(W, generator=g) for _ in range(4))
        r64, ya64, yb64 = r.to(P.DT), ya.to(P.DT), yb.to(P.DT)
        # the norm alone, for chosen rows, with scratch cleared on the way
        out = torch.empty(T, W, device="cuda")
        clear = torch.ones(T * W // 4 * 4, device="cuda")
        ops.join_norm(r.cuda(), gamma=gamma.cuda(), eps=1e-5, center=True, x_out=out, clear=clear)
        assert rel_err(out.cpu(), P.layer_norm(r64, gamma.to(P.DT), 1e-5)) < 1e-5 and float(clear.abs().sum()) == 0.0
        rows = torch.tensor([T - 1, 0], dtype=torch.int32, device="cuda")
        out2 = torch.empty(2, W, device="cuda", dtype=torch.bfloat16)
        ops.join_norm(r.cuda(), gamma=gamma.cuda(), eps=1e-5, center=True, x_out=out2, row_index=rows)
        assert rel_err(out2.float().cpu(), P.layer_norm(r64, gamma.to(P.DT), 1e-5)[[T - 1, 0]]) < 1e-2
        # two branches: r += 1/2 (ya / rms(ya) wa + yb / rms(yb) wb); the branches end zeroed
        rd, yad, ybd = r.cuda(), ya.cuda(), yb.cuda()
        ops.join_norm(rd, ya=yad, yb=ybd, wa=wa.cuda(), wb=wb.cuda(), mult=0.5, eps=1e-5)
        y = 0.5 * (P.rms_unit(ya64, 1e-5) * wa.to(P.DT) + P.rms_unit(yb64, 1e-5) * wb.to(P.DT))
        assert rel_err(rd.cpu(), r64 + y) < 1e-5 and float(yad.abs().sum()) == 0.0 and float(ybd.abs().sum()) == 0.0
        # the layer scale's write and the next norm's read in one launch
        rd, yd = r.cuda(), y.float().cuda()
        ops.join_norm(rd, ya=yd, scale=scale.cuda(), gamma=gamma.cuda(), eps=1e-6, center=True, x_out=out)
        joined = r64 + scale.to(P.DT) * y.float().to(P.DT)
        assert rel_err(rd.cpu(), joined) < 1e-5 and rel_err(out.cpu(), P.layer_norm(joined, gamma.to(P.DT), 1e-6)) < 1e-5
        assert float(yd.abs().sum()) == 0.0
        # the embedding's output joins the stream
        rd = r.cuda()
        ops.join_norm(rd, extra=ya.cuda())
        assert rel_err(rd.cpu(), r64 + ya64) < 1e-6
    # a branch that gave nothing stays nothing (0 / sqrt(0 + eps))
    rd = torch.zeros(2, 16, device="cuda")
    ops.join_norm(rd, ya=torch.zeros(2, 16, device="cuda"), yb=torch.ones(2, 16, device="cuda"),
                  wa=torch.ones(16, device="cuda"), wb=torch.ones(16, device="cuda"), mult=0.5, eps=1e-6)
    assert abs(float(rd[0, 0]) - 0.5) < 1e-5


@gpu
def test_head_norms_and_gates_against_their_formulas():
    from janus_b200.kernels import ops
    g = torch.Generator().manual_seed(1)
    for T, H, e, stored in ((6, 3, 9, 16), (4, 2, 64, 64), (2, 5, 8, 8), (3, 1, 40, 40)):
        o = torch.randn(T, H * e, generator=g) * 4
        wide = torch.randn(T, H * e + 5, generator=g)          # the gate is a view of wider rows
        weight = torch.randn(e, generator=g)
        gate = wide[:, 3:3 + H * e]
        want = (P.rms_unit(o.to(P.DT).view(T, H, e), 1e-5) * weight.to(P.DT)).reshape(T, H * e) * P.silu(gate.to(P.DT))
        out = torch.empty(T, H * e, device="cuda")
        ops.head_norm_gate(o.cuda(), wide.cuda()[:, 3:3 + H * e], weight.cuda(), 1e-5, out, H, e)
        assert rel_err(out.cpu(), want) < 1e-5
        x = torch.zeros(T, H, stored)
        x[:, :, :e] = o.view(T, H, e)
        xd = x.view(T, H * stored).cuda()
        ops.sigmoid_gate(xd, wide.cuda()[:, 3:3 + H * e], H, e, stored)
        want = o.to(P.DT).view(T, H, e) * torch.sigmoid(gate.to(P.DT)).view(T, H, e)
        assert rel_err(xd.cpu().view(T, H, stored)[:, :, :e], want) < 1e-5
        assert float(xd.cpu().view(T, H, stored)[:, :, e:].abs().sum()) == 0.0


def _run_delta_kernels(u, raw, conv_w, a_log, dt_bias, state, lengths, slots, H, G, d, e, taps, single=False):
    """The convolution and the recurrence as the mixer launches them, on hand-made step tensors."""
    from janus_b200.kernels import ops
    C = 2 * G * d + H * e
    T = u.shape[0]
    q_start = torch.tensor([0] + list(np.cumsum(lengths)), dtype=torch.int32, device="cuda")
    token_seq = torch.tensor([i for i, n in enumerate(lengths) for _ in range(n)], dtype=torch.int32, device="cuda")
    seq_slot = torch.tensor(slots, dtype=torch.int32, device="cuda")
    conv = torch.empty(T, C, device="cuda")
    ops.causal_conv_silu(u, 0, C, conv_w, None, taps, state, H * d * e, token_seq, q_start, seq_slot, conv, len(lengths),
                         single_tokens=single)
    out = torch.empty(T, H * e, device="cuda")
    ops.delta_rule(conv, 0, G * d, 2 * G * d, raw, 1, 1 + H, a_log, dt_bias, 1e-6, out, state, 0, q_start, seq_slot,
                   len(lengths), H, G, d, e)
    return out


@gpu
@pytest.mark.parametrize("H,G,d,e,taps", [(4, 2, 8, 16, 3), (3, 1, 5, 9, 2), (2, 2, 64, 64, 4), (1, 1, 200, 24, 1),
                                          (6, 3, 32, 40, 5), (2, 1, 96, 40, 3), (2, 2, 128, 128, 4), (1, 1, 65, 17, 2),
                                          (1, 1, 256, 16, 2)])
def test_convolution_and_delta_rule_kernels_against_the_plain_recurrence(H, G, d, e, taps):
    """Three sequences of unequal lengths in slots out of order: a prompt step, a second portion from the state the
    first left, then single tokens; outputs and the final state against the plain recurrence run in one piece."""
    g = torch.Generator().manual_seed(d * 100 + e)
    C = 2 * G * d + H * e
    total = (150, 3, 71)
    slots = [2, 0, 3]
    conv_w = torch.randn(C, taps, generator=g) * taps ** -0.5
    a_log, dt_bias = torch.randn(H, generator=g) - 2.0, torch.randn(H, generator=g)
    seqs = [dict(u=torch.randn(n, C, generator=g), raw=torch.randn(n, 2 * H + 3, generator=g) * 2) for n in total]
    state = torch.zeros(5, H * d * e + (taps - 1) * C + 3, device="cuda")
    got = [[] for _ in total]
    at = [0, 0, 0]
    steps = [(100, 2, 40), (47, 0, 29), (1, 1, 1), (1, 0, 1), (1, 0, 0)]
    for portion in steps:
        live = [i for i, n in enumerate(portion) if n]
        u = torch.cat([seqs[i]["u"][at[i]:at[i] + portion[i]] for i in live]).cuda()
        raw = torch.cat([seqs[i]["raw"][at[i]:at[i] + portion[i]] for i in live]).cuda()
        lengths = [portion[i] for i in live]
        out = _run_delta_kernels(u, raw, conv_w.cuda(), a_log.cuda(), dt_bias.cuda(), state, lengths,
                                 [slots[i] for i in live], H, G, d, e, taps, single=all(n == 1 for n in lengths)).cpu()
        row = 0
        for i in live:
            got[i].append(out[row:row + portion[i]])
            row += portion[i]
            at[i] += portion[i]
    assert at == list(total)
    for i, s in enumerate(seqs):
        u64, raw64 = s["u"].to(P.DT), s["raw"].to(P.DT)
        y, tail = P.short_conv(u64, conv_w.to(P.DT), None)
        n = y.shape[0]
        q, k, v = y[:, :G * d].view(n, G, d), y[:, G * d:2 * G * d].view(n, G, d), y[:, 2 * G * d:].view(n, H, e)
        q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
        k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
        beta = torch.sigmoid(raw64[:, 1:1 + H])
        decay = torch.exp(-torch.exp(a_log.to(P.DT)) * P.softplus(raw64[:, 1 + H:1 + 2 * H] + dt_bias.to(P.DT)))
        o, S = P.delta_recurrence(q, k, v, beta, decay)
        assert rel_err(torch.cat(got[i]), o.reshape(n, H * e)) < 2e-5, i
        kept = state[slots[i]].cpu()
        assert rel_err(kept[:H * d * e].view(H, d, e), S) < 2e-5, i
        if taps > 1:
            assert rel_err(kept[H * d * e:H * d * e + (taps - 1) * C].view(taps - 1, C), tail) < 1e-6, i
    assert float(state[1].abs().sum()) == 0.0 and float(state[4].abs().sum()) == 0.0      # slots nobody had


@gpu
def test_router_and_expert_kernels_against_the_plain_feed_forward():
    from janus_b200.kernels import ops
    g = torch.Generator().manual_seed(2)
    # ties go to the lower index; the weights are the sigmoids as they are
    logits = torch.tensor([[0.5, 2.0, 2.0, -1.0, 2.0], [3.0, -3.0, 0.0, 0.0, 1.0]], device="cuda")
    sel_e = torch.empty(2, 3, dtype=torch.int32, device="cuda")
    sel_w = torch.empty(2, 3, device="cuda")
    ops.route_topk(logits, 3, sel_e, sel_w)
    assert sel_e.cpu().tolist() == [[1, 2, 4], [0, 4, 2]]
    assert rel_err(sel_w.cpu(), torch.sigmoid(torch.tensor([[2.0, 2.0, 2.0], [3.0, 1.0, 0.0]]))) < 1e-6
    for T, W, F, E, top, dtype in ((9, 64, 48, 5, 2, torch.float32), (1, 36, 13, 4, 4, torch.float32),
                                   (33, 96, 40, 7, 1, torch.float32), (20, 64, 32, 6, 3, torch.bfloat16),
                                   # inner widths that the down product takes in parts
                                   (5, 32, 2100, 3, 1, torch.float32), (6, 40, 4500, 2, 2, torch.bfloat16),
                                   (3, 64, 4096, 2, 1, torch.bfloat16)):
        wts = {"router": torch.randn(E, W, generator=g).to(torch.bfloat16).to(P.DT)}
        for x in range(E):
            wts[f"e{x}.gate"] = (torch.randn(F, W, generator=g) * W ** -0.5).to(torch.bfloat16).to(P.DT)
            wts[f"e{x}.up"] = (torch.randn(F, W, generator=g) * W ** -0.5).to(torch.bfloat16).to(P.DT)
            wts[f"e{x}.down"] = (torch.randn(W, F, generator=g) * F ** -0.5).to(torch.bfloat16).to(P.DT)
        h = (torch.randn(T, W, generator=g)).to(torch.bfloat16)
        want = P.routed_feed_forward(h.to(P.DT), wts, E, top)
        z = (h.to(P.DT) @ wts["router"].T).float().cuda()
        sel_e = torch.empty(T, top, dtype=torch.int32, device="cuda")
        sel_w = torch.empty(T, top, device="cuda")
        ops.route_topk(z, top, sel_e, sel_w)
        stack = lambda kind: torch.stack([wts[f"e{x}.{kind}"] for x in range(E)]).to(dtype).cuda().contiguous()  # noqa: E731
        out = torch.zeros(T, W, device="cuda")
        act = torch.empty(T * top, F, device="cuda")
        ops.experts_few_tokens(h.to(dtype).cuda(), sel_e, sel_w, stack("gate"), stack("up"), stack("down"), act, out)
        assert rel_err(out.cpu(), want) < (1e-5 if dtype == torch.float32 else 1e-2), (T, W, F, E, top)
        # the pairs in the experts' order and back: a gather of weighted rows, a sum per token
        chosen = sel_e.reshape(-1).cpu().numpy()
        order = np.argsort(chosen, kind="stable").astype(np.int32)
        where = np.empty(T * top, dtype=np.int32)
        where[order] = np.arange(T * top, dtype=np.int32)
        rows = torch.empty(T * top, W, dtype=dtype, device="cuda")
        ops.expert_gather(h.to(dtype).cuda(), torch.from_numpy(order).cuda(), sel_w, top, rows)
        flat_w = sel_w.reshape(-1).cpu().to(P.DT)
        want_rows = torch.stack([flat_w[p] * h[p // top].to(P.DT) for p in order.tolist()])
        assert rel_err(rows.float().cpu(), want_rows) < (1e-6 if dtype == torch.float32 else 1e-2)
        results = torch.randn(T * top, W, generator=g)
        acc = torch.zeros(T, W, device="cuda")
        ops.expert_scatter(results.cuda(), torch.from_numpy(where).cuda(), top, acc)
        want_acc = torch.stack([sum(results[where[t * top + j]].to(P.DT) for j in range(top)) for t in range(T)])
        assert rel_err(acc.cpu(), want_acc) < 1e-6


@gpu
@pytest.mark.parametrize("T,W,F,E,top,skip", [(700, 128, 256, 5, 2, 3), (260, 256, 128, 3, 1, None), (90, 128, 128, 40, 3, 0)])
def test_experts_of_a_prompt_sorted_on_the_device_and_served_by_two_grouped_products(T, W, F, E, top, skip):
    """Pairs sorted by expert without the host, the experts' products as one launch each over stacked matrices:
    experts with more rows than a tile, with a few rows, with none."""
    from janus_b200.kernels import ops
    g = torch.Generator().manual_seed(11)
    wts = {"router": torch.randn(E, W, generator=g).to(torch.bfloat16).to(P.DT)}
    if skip is not None:
        wts["router"][skip] = 0.0
        wts["router"][skip, 0] = -50.0                      # with h[:, 0] = 1 nobody chooses this expert
    for x in range(E):
        wts[f"e{x}.gate"] = (torch.randn(F, W, generator=g) * W ** -0.5).to(torch.bfloat16).to(P.DT)
        wts[f"e{x}.up"] = (torch.randn(F, W, generator=g) * W ** -0.5).to(torch.bfloat16).to(P.DT)
        wts[f"e{x}.down"] = (torch.randn(W, F, generator=g) * F ** -0.5).to(torch.bfloat16).to(P.DT)
    h = torch.randn(T, W, generator=g)
    h[:, 0] = 1.0
    h = h.to(torch.bfloat16)
    want = P.routed_feed_forward(h.to(P.DT), wts, E, top)
    z = (h.to(P.DT) @ wts["router"].T).float().cuda()
    sel_e = torch.empty(T, top, dtype=torch.int32, device="cuda")
    sel_w = torch.empty(T, top, device="cuda")
    ops.route_topk(z, top, sel_e, sel_w)
    pairs = T * top
    max_gu, max_dn = ops.grouped_max_items(pairs, E, F, "swiglu"), ops.grouped_max_items(pairs, E, W, "store")
    index = torch.full((2, pairs), -1, dtype=torch.int32, device="cuda")
    t_gu = torch.zeros(4 + 4 * max_gu, dtype=torch.int32, device="cuda")
    t_dn = torch.zeros(4 + 4 * max_dn, dtype=torch.int32, device="cuda")
    ops.expert_plan(sel_e, E, F, W, index[0], index[1], t_gu, t_dn)
    order, where, chosen = index[0].cpu(), index[1].cpu(), sel_e.reshape(-1).cpu()
    assert sorted(order.tolist()) == list(range(pairs))
    assert where[order.long()].tolist() == list(range(pairs))
    in_order = chosen[order.long()]
    assert bool((in_order[1:] >= in_order[:-1]).all())           # an expert's pairs lie next to each other
    if skip is not None:
        assert skip not in set(chosen.tolist())
    counts = torch.bincount(chosen.long(), minlength=E)
    tiles = int(((counts + 255) // 256).sum())
    assert int(t_gu[0]) == tiles * (F // 128) <= max_gu and int(t_dn[0]) == tiles * ((W + 255) // 256) <= max_dn
    stack = lambda kind: torch.cat([wts[f"e{x}.{kind}"] for x in range(E)]).to(torch.bfloat16).cuda().contiguous()  # noqa: E731
    gate_up, down = ops.pack_gated(stack("gate"), stack("up")), ops.pack_weight(stack("down"))
    rows = torch.empty(pairs, W, dtype=torch.bfloat16, device="cuda")
    ops.expert_gather(h.cuda(), index[0], sel_w, top, rows)
    act = torch.full((pairs, F), float("nan"), dtype=torch.bfloat16, device="cuda")
    ops.gemm_bf16_grouped(rows, gate_up, act, t_gu, max_gu, mode="swiglu")
    results = torch.full((pairs, W), float("nan"), device="cuda")
    ops.gemm_bf16_grouped(act, down, results, t_dn, max_dn, mode="store")
    out = torch.zeros(T, W, device="cuda")
    ops.expert_scatter(results, index[1], top, out)
    ops.check_kernel_status(torch.device("cuda"))
    assert rel_err(out.cpu(), want) < 1e-2


@gpu
@pytest.mark.parametrize("tiles", ["1", "2"])
@pytest.mark.parametrize("nh,nkv,hd,chunk,cap", [(8, 2, 64, 130, 5.0), (4, 4, 128, 64, 0.0), (6, 2, 32, 0, 2.0),
                                                 (8, 1, 128, 200, 50.0)])
def test_prompt_attention_kernels_with_chunks_and_a_cap_against_the_plain_softmax(monkeypatch, tiles, nh, nkv, hd, chunk, cap):
    """The tensor-core prompt kernel (one row tile a block, and two), the mma.sync one and the float32 one on the same
    pages: a prompt from position 0 and a portion that starts at position 300 of a longer sequence, pages out of order."""
    from janus_b200.kernels import ops
    if not ops.attention_tc_supported(nh, nkv, hd):
        pytest.skip("the tensor-core kernel does not take this shape")
    monkeypatch.setenv("JANUS_ATTN_TC_TILES", tiles)
    g = torch.Generator().manual_seed(hd + chunk)
    scale = 2.0 * hd ** -0.5
    lens, starts = (333, 500), (0, 300)
    n_pages = sum((n + 63) // 64 for n in lens) + 3
    order = torch.randperm(n_pages, generator=g).tolist()
    kc = torch.zeros(n_pages, nkv, 64, hd, dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    table = torch.zeros(2, 8, dtype=torch.int32)
    qs, want = [], []
    for i, (n, start) in enumerate(zip(lens, starts)):
        k = torch.randn(n, nkv, hd, generator=g).to(torch.bfloat16)
        v = torch.randn(n, nkv, hd, generator=g).to(torch.bfloat16)
        q = torch.randn(n - start, nh, hd, generator=g).to(torch.bfloat16)
        for pg in range((n + 63) // 64):
            page = order.pop()
            table[i, pg] = page
            rows = slice(pg * 64, min(n, pg * 64 + 64))
            kc[page, :, : rows.stop - rows.start] = k[rows].transpose(0, 1)
            vc[page, :, : rows.stop - rows.start] = v[rows].transpose(0, 1)
        qs.append(q)
        want.append(P.chunk_softmax(q.to(P.DT), k.to(P.DT), v.to(P.DT), start, scale, cap or None, chunk or None))
    q = torch.cat(qs).reshape(-1, nh * hd).cuda()
    want = torch.cat(want).reshape(-1, nh * hd)
    q_start = torch.tensor([0, lens[0] - starts[0], lens[0] - starts[0] + lens[1] - starts[1]], dtype=torch.int32).cuda()
    kv_len = torch.tensor(lens, dtype=torch.int32).cuda()
    out = torch.zeros_like(q)
    args = (q, kc.cuda(), vc.cuda(), out, table.cuda(), q_start, kv_len, 2, lens[0], nh, nkv, hd, 64, 0, scale, chunk, cap)
    ops.attention_tc_prefill(*args)
    assert rel_err(out.float().cpu(), want) < 1e-2
    out.zero_()
    ops.attention_bf16_prefill(*args)
    assert rel_err(out.float().cpu(), want) < 1e-2
    if tiles == "1":
        token_seq = torch.tensor([0] * (lens[0] - starts[0]) + [1] * (lens[1] - starts[1]), dtype=torch.int32).cuda()
        positions = torch.cat([torch.arange(starts[i], lens[i], dtype=torch.int32) for i in range(2)]).cuda()
        out32 = torch.zeros(q.shape, device="cuda")
        ops.attention_f32(q.float(), kc.float().cuda(), vc.float().cuda(), out32, table.cuda(), token_seq, positions, nh, nkv,
                          hd, 64, 0, scale, chunk, cap)
        assert rel_err(out32.cpu(), want) < 1e-5
    ops.check_kernel_status(q.device)


def _one_branch(cfg, w, side):
    """The same model with the other branch silenced: its output projection is zero, so its normed output is too."""
    out = dict(w)
    other = "right" if side == "left" else "left"
    for name in w:
        if name.endswith(f".mix.{other}.o"):
            out[name] = torch.zeros_like(w[name])
    return out


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("side", ["left", "right"])
def test_each_branch_alone_in_a_layer_without_feed_forward(tmp_path, side, dtype):
    """One layer, no feed-forward, one branch silent: the logits are final_norm(x + ls1 * 1/2 norm(branch) w) head, with
    the branch from its own plain function.  The attention has a cap that bites, chunks, part of the heads rotated
    with a ramp, unequal key and value sizes; the delta rule more heads than query/key heads and five taps."""
    from janus_b200.engine import StepEntry
    cfg = dict(architecture="Mugedra", vocab=90, width=48, norm=dict(eps=1e-5),
               layers=[layer(left(6, 3, 16, 24, 0.4, softcap=1.5, mask=23, rot=(12, 200.0, (4.0, 32, 8.0, 1.0))),
                             right(4, 2, 16, 24, 5))])
    w = _one_branch(cfg, sharpened(P.random_weights(cfg, 40), 3.0), side)
    ids = random_tokens(100, cfg["vocab"], 41)
    x = w["embed"][torch.tensor(ids)]
    h = P.layer_norm(x, w["l0.norm1"], 1e-5)
    sub = {n[len(f"l0.mix.{side}."):]: t for n, t in w.items() if n.startswith(f"l0.mix.{side}.")}
    if side == "left":
        y, _ = P.chunk_attention(h, sub, cfg["layers"][0]["mixer"]["left"], 1e-5)
    else:
        y, _ = P.gated_delta(h, sub, cfg["layers"][0]["mixer"]["right"], 1e-5)
    x = x + w["l0.ls1"] * 0.5 * P.rms_unit(y, 1e-5) * w[f"l0.mix.{side}.out"]
    ref = P.layer_norm(x, w["final.norm"], 1e-5) @ w["head"].T
    assert rel_err(P.forward(cfg, w, ids), ref) < 1e-9
    d = P.save_folder(cfg, w, str(tmp_path / side))
    model = load(d, dtype)
    s = model.alloc_slot()
    out = model.step([StepEntry(s, ids[:61], range(61))]).cpu()
    assert rel_err(out, ref[:61]) < tol_for(dtype)
    out = model.step([StepEntry(s, ids[61:98], range(37))]).cpu()
    assert rel_err(out, ref[61:98]) < tol_for(dtype)
    for t in (98, 99):
        assert rel_err(model.step([StepEntry(s, [ids[t]], [0])]).cpu(), ref[t:t + 1]) < tol_for(dtype)
    model.check()


# ------------------------------------------------------------------------------------------------
# cases made so that one key or one far token shows (their premises are checked without a device)
# ------------------------------------------------------------------------------------------------
X, Y = 111, 112   # two tokens whose keys every query of the edge case answers to; their values differ


def chunk_edge_case(seed=5):
    """One layer without feed-forward.  Feature W - 1 is the same for every token, so every query has a positive
    first dimension; the tokens X and Y alone have feature 7, which the keys' first dimension reads: their keys
    outweigh all others for every query that sees them.  X sits on the last position of a chunk and Y on the first of
    the next, in the prompt, right before a portion's start and among the single tokens.  A cap of 3 bites on such
    scores."""
    cfg = dict(architecture="Mugedra", vocab=120, width=64, norm=dict(eps=1e-5),
               layers=[layer(left(2, 1, 16, 16, 0.5, softcap=3.0, mask=70, rot=(8, 10000.0)), right(2, 1, 8, 8, 3))])
    w = P.random_weights(cfg, seed)
    W = cfg["width"]
    w["embed"][:, W - 1] = 4.0
    w["embed"][:, 7] = 0.0
    w["embed"][X] = 0.0
    w["embed"][X, 7], w["embed"][X, W - 1] = 8.0, 4.0
    w["embed"][Y, 7] = 8.0
    w["l0.norm1"][7] = w["l0.norm1"][W - 1] = 1.0
    for name, feature in (("q", W - 1), ("k", 7)):
        t = w[f"l0.mix.left.{name}"]
        t[:, feature] = 0.0
        t[8::16] = 0.0                             # dimension 8 of every head (not rotated) reads one feature only
        t[8::16, feature] = 2.0
        w[f"l0.mix.left.{name}.norm"][8] = 3.0
    w["l0.mix.right.out"] = w["l0.mix.right.out"] * 0.25       # the attention leads the sublayer
    w["l0.ls1"] = w["l0.ls1"] * 2.0                             # and the sublayer the logits
    ids = random_tokens(235, 100, 9)
    for edge in (70, 140, 210):
        ids[edge - 1], ids[edge] = X, Y
    ref = P.forward(cfg, w, ids)
    return cfg, w, ids, ref


def far_token_case(seed=6):
    """One layer without feed-forward whose first delta-rule head does not decay.  The filler token's keys are exactly
    zero (the key projection reads two features that only two other tokens have), so after the first positions
    nothing is written and the state carries what position 3 wrote for hundreds of tokens; the attention's chunks
    of 50 positions cannot see that far."""
    cfg = dict(architecture="Mugedra", vocab=90, width=32, norm=dict(eps=1e-5),
               layers=[layer(left(2, 1, 8, 8, 0.3, mask=50), right(2, 1, 8, 8, 2))])
    w = P.random_weights(cfg, seed)
    for tok, feature in ((5, 0), (77, 1), (12, 2)):
        w["embed"][tok] = 0.0
        w["embed"][tok, feature], w["embed"][tok, 3] = 1.0, -1.0      # mean zero: the norm leaves the zeros zero
    w["l0.norm1"][:4] = 1.0
    k, q = w["l0.mix.right.k"], w["l0.mix.right.q"]
    k1, k2 = k[:, 1].clone(), k[:, 2].clone()
    k[:] = 0.0
    k[:, 1], k[:, 2] = k1 * 4.0, k2 * 4.0
    q0 = q[:, 0].clone()
    q[:] = 0.0
    q[:, 0] = q0 * 4.0
    w["l0.mix.right.A_log"][0] = -12.0
    w["l0.mix.left.out"] = w["l0.mix.left.out"] * 0.25          # the recurrence leads the sublayer
    ids = [5] * 400
    ids[3] = 77
    other = list(ids)
    other[3] = 12
    return cfg, w, ids, other, P.forward(cfg, w, ids), P.forward(cfg, w, other)


def test_the_cases_made_for_edges_and_far_tokens_show_in_the_plain_logits():
    cfg, w, ids, ref = chunk_edge_case()
    rows = list(range(60, 235))
    worst = 2 * BF16_TOL
    for change in ("smaller", "larger", "no cap", "no chunks"):
        off = copy.deepcopy(cfg)
        m = off["layers"][0]["mixer"]["left"]
        if change == "smaller":
            m["mask"]["size"] -= 1
        elif change == "larger":
            m["mask"]["size"] += 1
        elif change == "no cap":
            del m["softcap"]
        else:
            del m["mask"]
        assert rel_err(P.forward(off, w, ids)[rows], ref[rows]) > 5 * worst, change
    # the rows right at an edge by themselves: the query on a chunk's first position must not see the one before it,
    # the one after it must see the first
    for size in (69, 71):
        off = copy.deepcopy(cfg)
        off["layers"][0]["mixer"]["left"]["mask"]["size"] = size
        moved = P.forward(off, w, ids)
        for edge in (70, 140, 210):
            rows = [edge, edge + 1]
            assert rel_err(moved[rows], ref[rows]) > 3 * worst, (edge, size)
    cfg, w, ids, other, ref, ref_other = far_token_case()
    assert rel_err(ref_other[-5:], ref[-5:]) > 5 * worst


# ------------------------------------------------------------------------------------------------
# on the device: the engine
# ------------------------------------------------------------------------------------------------
@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_whole_prompts_of_unequal_lengths_in_one_step(tmp_path, name, dtype):
    from janus_b200.engine import StepEntry
    cfg = CONFIGS[name]
    d, w = folder(tmp_path, cfg, 11)
    model = load(d, dtype)
    seqs = [random_tokens(n, cfg["vocab"], 100 + n) for n in (150, 1, 67, 2, 64)]
    slots = [model.alloc_slot() for _ in seqs]
    out = model.step([StepEntry(s, ids, range(len(ids))) for s, ids in zip(slots, seqs)]).cpu()
    ref = torch.cat([plain_logits(cfg, w, ids) for ids in seqs])
    assert rel_err(out, ref) < tol_for(dtype)
    if dtype == "float32":
        at = 0
        for ids in seqs:          # every sequence by itself, the single token too
            assert rel_err(out[at:at + len(ids)], ref[at:at + len(ids)]) < tol_for(dtype), (name, len(ids))
            at += len(ids)
    model.check()


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_portions_then_single_tokens_in_a_batch_and_slots_used_again(tmp_path, name, dtype):
    """Prompts cut into portions of 2 to 64 tokens, unequal requests in one batch, then one token each until the
    shorter ones have ended; afterwards other requests take the freed slots and pages (and find the recurrence's
    state and the convolution's inputs zeroed).  Every row is compared with the whole sequence's plain logits."""
    from janus_b200.engine import StepEntry
    cfg = CONFIGS[name]
    d, w = folder(tmp_path, cfg, 12)
    tol = tol_for(dtype)
    model = load(d, dtype, max_tokens=64 * 9, max_slots=3)
    for round_no, lengths in enumerate(((140, 75, 20), (90, 130, 129))):
        seqs = [random_tokens(n, cfg["vocab"], 7 * round_no + n) for n in lengths]
        ref = [plain_logits(cfg, w, ids) for ids in seqs]
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
                assert rel_err(out[row:row + n], ref[i][lo:lo + n]) < tol, (round_no, i, lo, n)
                row += n
        live = [0, 1, 2]
        while live:
            out = model.step([StepEntry(slots[i], [seqs[i][at[i]]], [0]) for i in live]).cpu()
            for row, i in enumerate(live):
                assert rel_err(out[row:row + 1], ref[i][at[i]:at[i] + 1]) < tol, (round_no, i, at[i])
                at[i] += 1
            for i in [i for i in live if at[i] == len(seqs[i])]:
                model.free_slot(slots[i])
                live.remove(i)
        model.engine.cache.check()
    model.check()


def drawn_config(seed):
    """A configuration drawn from a seed: sizes from small and odd to those of the tensor-core kernels, every
    optional constant present or absent, layers with and without a feed-forward, a loop anywhere or none."""
    import random
    rng = random.Random(seed)
    n_layers = rng.choice([1, 2, 3, 4])
    width = rng.choice([40, 64, 96, 128, 192, 256])
    layers = []
    for _ in range(n_layers):
        kv = rng.choice([1, 2, 3])
        dim = rng.choice([8, 16, 24, 32, 64, 128])
        vdim = rng.choice([dim, dim, 8, 16, 32, 64])
        rot = None
        if rng.random() < 0.75:
            dims = rng.choice([dim, dim // 2, max(2, dim // 4 * 2)])
            rot = (dims, rng.choice([50.0, 10000.0, 250000.0]))
            if rng.random() < 0.6:
                rot += ((rng.choice([2.0, 4.0, 8.0]), rng.choice([16, 64, 128]), rng.choice([4.0, 32.0]), 1.0),)
        a = left(kv * rng.choice([1, 2, 4]), kv, dim, vdim, rng.choice([dim ** -0.5, 0.2, 0.4]),
                 softcap=rng.choice([None, 3.0, 50.0]), mask=rng.choice([None, 3, 16, 41, 64, 100, 128]), rot=rot)
        g = rng.choice([1, 2])
        r = right(g * rng.choice([1, 2, 3]), g, rng.choice([8, 16, 48, 72, 96, 128]), rng.choice([8, 16, 40, 64]),
                  rng.choice([1, 2, 3, 4]))
        moe = None
        if rng.random() < 0.8:
            experts = rng.choice([1, 2, 4, 7, 8])
            moe = (rng.choice([24, 64, 128]), experts, rng.choice([t for t in (1, 2, 3) if t <= experts]))
        layers.append(layer(a, r, moe))
    cfg = dict(architecture="Mugedra", vocab=rng.choice([97, 256, 500]), width=width,
               norm=dict(eps=rng.choice([1e-5, 1e-6])), layers=layers)
    if rng.random() < 0.7:
        start = rng.randrange(n_layers)
        cfg["loop"] = dict(start=start, stop=rng.randrange(start + 1, n_layers + 1), times=rng.choice([1, 2, 3]))
    return cfg


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", list(range(1, 25)))
def test_configurations_drawn_from_a_seed(tmp_path, seed, dtype):
    """Three prompts of unequal length in one step, a second portion each, then token by token while the shorter
    requests end, against the plain implementation's logits of the whole sequences."""
    from janus_b200.engine import StepEntry
    cfg = drawn_config(seed)
    w = weights_for(cfg, 40 + seed)
    for name in [n for n in w if n.endswith(".mlp.router")]:       # wide models: the class decides, not the rest
        w[name][:, :cfg["width"] - TAGS] *= 0.25
    d = P.save_folder(cfg, w, str(tmp_path / f"drawn{seed}"))
    tol = tol_for(dtype)
    model = load(d, dtype, max_tokens=1024, max_slots=3)
    seqs = [random_tokens(n, cfg["vocab"], 300 + 10 * seed + n) for n in (170, 9, 77)]
    ref = [plain_logits(cfg, w, ids) for ids in seqs]
    slots = [model.alloc_slot() for _ in seqs]
    at = [0, 0, 0]
    for portion in ((131, 2, 40), (30, 3, 33)):
        out = model.step([StepEntry(slots[i], seqs[i][at[i]:at[i] + n], range(n)) for i, n in enumerate(portion)]).cpu()
        row = 0
        for i, n in enumerate(portion):
            assert rel_err(out[row:row + n], ref[i][at[i]:at[i] + n]) < tol, (cfg, i, at[i], n)
            row += n
            at[i] += n
    live = [0, 1, 2]
    while live:
        out = model.step([StepEntry(slots[i], [seqs[i][at[i]]], [0]) for i in live]).cpu()
        for row, i in enumerate(live):
            assert rel_err(out[row:row + 1], ref[i][at[i]:at[i] + 1]) < tol, (cfg, i, at[i])
            at[i] += 1
        for i in [i for i in live if at[i] == len(seqs[i])]:
            model.free_slot(slots[i])
            live.remove(i)
    model.check()


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_batch_gives_every_request_what_it_gets_alone(tmp_path, dtype):
    """The same requests alone and together, as prompts and as single tokens: the engine against itself, so the
    bound is the rounding of different tilings only."""
    from janus_b200.engine import StepEntry
    cfg = CONFIGS["D"]
    d, w = folder(tmp_path, cfg, 16)
    model = load(d, dtype, max_tokens=2048, max_slots=5)
    seqs = [random_tokens(n, cfg["vocab"], 50 + n) for n in (130, 9, 70, 201)]
    alone = []
    for ids in seqs:
        s = model.alloc_slot()
        rows = [model.step([StepEntry(s, ids[:-3], range(len(ids) - 3))]).cpu()]
        rows += [model.step([StepEntry(s, [t], [0])]).cpu() for t in ids[-3:]]
        alone.append(torch.cat(rows))
        model.free_slot(s)
    slots = [model.alloc_slot() for _ in seqs]
    out = model.step([StepEntry(s, ids[:-3], range(len(ids) - 3)) for s, ids in zip(slots, seqs)]).cpu()
    together, at = [], 0
    for ids in seqs:
        together.append([out[at:at + len(ids) - 3]])
        at += len(ids) - 3
    for j in range(3):
        out = model.step([StepEntry(s, [ids[len(ids) - 3 + j]], [0]) for s, ids in zip(slots, seqs)]).cpu()
        for i in range(len(seqs)):
            together[i].append(out[i:i + 1])
    bound = 1e-5 if dtype == "float32" else BF16_TOL
    for i in range(len(seqs)):
        assert rel_err(torch.cat(together[i]), alone[i]) < bound, i
    model.check()


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_keys_at_the_edges_of_the_chunks_in_prompts_portions_and_single_tokens(tmp_path, dtype):
    """The case whose plain logits move clearly when the chunk is one position smaller or larger, when the cap is
    left out or when the chunks are: a prompt that holds two edges, single tokens over a third (and over page
    borders), and portions that start right on an edge and right after one."""
    from janus_b200.engine import StepEntry
    cfg, w, ids, ref = chunk_edge_case()
    d = P.save_folder(cfg, w, str(tmp_path / "edge"))
    tol = tol_for(dtype)
    model = load(d, dtype, max_tokens=1024)
    s = model.alloc_slot()
    out = model.step([StepEntry(s, ids[:150], range(150))]).cpu()
    assert rel_err(out, ref[:150]) < tol
    for edge in (70, 140):
        assert rel_err(out[edge - 1:edge + 2], ref[edge - 1:edge + 2]) < tol, edge
    for t in range(150, 235):
        out = model.step([StepEntry(s, [ids[t]], [0])]).cpu()
        assert rel_err(out, ref[t:t + 1]) < tol, t
    model.free_slot(s)
    for cuts in ((70, 70, 1, 69, 2, 23), (71, 2, 68, 69, 1, 1, 23), (3, 66, 2, 139, 25)):
        s = model.alloc_slot()
        at = 0
        for n in cuts:
            out = model.step([StepEntry(s, ids[at:at + n], range(n))]).cpu()
            assert rel_err(out, ref[at:at + n]) < tol, (cuts, at)
            at += n
        assert at == 235
        model.free_slot(s)
    model.check()


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_far_token_reaches_through_the_delta_rule_state(tmp_path, dtype):
    """A head that does not decay carries what position 3 wrote over hundreds of positions: changing that one token
    changes the last plain logits clearly, and the library follows both versions, the prompt in one piece or in
    portions, then single tokens."""
    from janus_b200.engine import StepEntry
    cfg, w, ids, other, ref, ref_other = far_token_case()
    d = P.save_folder(cfg, w, str(tmp_path / "far"))
    model = load(d, dtype, max_tokens=1024)
    for seq, want in ((ids, ref), (other, ref_other)):
        for cuts in ((395,), (2, 2, 130, 261)):
            s = model.alloc_slot()
            at = 0
            for n in cuts:
                out = model.step([StepEntry(s, seq[at:at + n], [n - 1])]).cpu()
                at += n
            assert rel_err(out, want[394:395]) < tol_for(dtype)
            for t in range(395, 400):
                out = model.step([StepEntry(s, [seq[t]], [0])]).cpu()
                assert rel_err(out, want[t:t + 1]) < tol_for(dtype)
            model.free_slot(s)
    model.check()


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_long_decoding_from_the_first_token(tmp_path, name, dtype):
    """A sequence that starts with a single token and grows by one for 200 steps (replayed CUDA graphs): the first
    tokens (fewer than the convolution's taps), page borders at 64 and 128, chunk edges at every size of the
    configuration, every pass of the loop with its own state."""
    from janus_b200.engine import StepEntry
    cfg = CONFIGS[name]
    d, w = folder(tmp_path, cfg, 13)
    ids = random_tokens(200, cfg["vocab"], 21)
    ref = plain_logits(cfg, w, ids)
    model = load(d, dtype, max_tokens=256, max_slots=2)
    s = model.alloc_slot()
    got = [model.step([StepEntry(s, [t], [0])]).cpu() for t in ids]
    assert rel_err(torch.cat(got), ref) < tol_for(dtype)
    for t in (0, 1, 2, 3):
        assert rel_err(got[t], ref[t:t + 1]) < tol_for(dtype), t
    assert model.engine.graph_captures >= 1
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
        logits = plain_logits(CFG_A, w, list(p) + list(o))
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
    d, w = folder(tmp_path, CFG_C, 14)
    ids = random_tokens(40, CFG_C["vocab"], 2)
    other = random_tokens(33, CFG_C["vocab"], 3)
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
    got = np.concatenate([np.fromfile(out / f"{s['step']}.f32", dtype="<f4").reshape(-1, CFG_C["vocab"]) for s in steps])
    rx, ry = plain_logits(CFG_C, w, ids), plain_logits(CFG_C, w, other)
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
