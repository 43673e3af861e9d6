"""The Mugedra decoder as data: a `ModelSpec` made from a `MugedraConfig`.

Every layer is two mixers side by side (`parts.parallel`): grouped-query attention with normed heads, rotary positions
with a frequency ramp, capped scores, a chunked mask and an output gate (`parts.capped_attention`), and the gated delta
rule (`parts.delta_rule`); then a feed-forward of experts chosen by sigmoid scores (`parts.routed`), or none.  The
norms are layer norms with a weight and no bias, pre-norm; what a sublayer produced is multiplied feature by feature by
a weight before it joins the residual stream (`parts.connection` kind `layer_scale`, arrangement `hyper_pre_norm` with
its single stream).  The layers of the configuration's loop are places of the schedule once per pass, each with a cache
and state of its own, and every pass but the first begins with the embedding's output added to the stream
(`ScheduleEntry.adds_embedding`).  Tensor names: `embed`, `l<i>.norm1`, `l<i>.norm2`, `l<i>.ls1`, `l<i>.ls2`,
`l<i>.mix.left.*`, `l<i>.mix.right.*`, `l<i>.mlp.router`, `l<i>.mlp.e<j>.{gate,up,down}`, `final.norm`, `head`.
"""
from __future__ import annotations

from typing import List

from ..config.mugedra import MugedraConfig
from ..config.registry import register_architecture
from ..parts.base import LayerSpec, ModelSpec, PartSpec, ScheduleEntry


def _mixer_spec(config: MugedraConfig, i: int) -> PartSpec:
    m, p = config.layers[i].mixer, f"l{i}.mix."
    a, r = m.left, m.right
    position = None
    if a.rot is not None:
        scaling = None if a.rot.scaling is None else dict(zip(("factor", "original", "fast", "slow"), a.rot.scaling))
        position = PartSpec("ramped_rotary", dict(dims=a.rot.dims, theta=a.rot.base, max_positions=config.max_positions,
                                                  scaling=scaling))
    left = PartSpec("capped_attention",
                    dict(hidden_size=config.width, num_heads=a.heads, num_kv_heads=a.kv_heads, dim=a.dim, vdim=a.vdim,
                         scale=a.scale, eps=config.eps, softcap=a.softcap, chunk=a.chunk, qk_norm=True, gate=True,
                         position=position, rotary_dims=0 if a.rot is None else a.rot.dims))
    right = PartSpec("gated_delta_rule",
                     dict(hidden_size=config.width, num_heads=r.heads, num_kv_heads=r.kv_heads, dim=r.dim, vdim=r.vdim,
                          conv_taps=r.conv, eps=config.eps))
    weights = {"left_out": p + "left.out", "right_out": p + "right.out"}
    weights.update({"left." + n: p + "left." + t for n, t in
                    (("q", "q"), ("k", "k"), ("v", "v"), ("o", "o"), ("g", "g"), ("q_norm", "q.norm"), ("k_norm", "k.norm"))})
    weights.update({"right." + n: p + "right." + t for n, t in
                    (("q", "q"), ("k", "k"), ("v", "v"), ("g", "g"), ("b", "b"), ("a", "a"), ("o", "o"),
                     ("q_conv", "q.conv"), ("k_conv", "k.conv"), ("v_conv", "v.conv"), ("A_log", "A_log"),
                     ("dt_bias", "dt_bias"), ("norm", "norm"))})
    return PartSpec("parallel", dict(hidden_size=config.width, left=left, right=right, eps=config.eps, mult=0.5),
                    weights=weights)


def mugedra_spec(config: MugedraConfig) -> ModelSpec:
    layers: List[LayerSpec] = []
    norm_of = lambda name: PartSpec("layer_norm", dict(width=config.width, eps=config.eps), weights=dict(gamma=name))  # noqa: E731
    scale_of = lambda name: PartSpec("layer_scale", dict(width=config.width), weights=dict(scale=name))   # noqa: E731
    for i, layer in enumerate(config.layers):
        p = f"l{i}."
        feed_forward = None
        extra = (("mixer_connection", "connection", scale_of(p + "ls1")),)
        if layer.mlp is not None:
            weights = {"router": p + "mlp.router"}
            for e in range(layer.mlp.experts):
                weights.update({f"e{e}_{n}": p + f"mlp.e{e}.{n}" for n in ("gate", "up", "down")})
            feed_forward = PartSpec("routed_experts", dict(hidden_size=config.width, intermediate_size=layer.mlp.ff,
                                                           experts=layer.mlp.experts, top=layer.mlp.top), weights=weights)
            extra += (("feed_forward_connection", "connection", scale_of(p + "ls2")),)
        layers.append(LayerSpec(mixer=_mixer_spec(config, i), feed_forward=feed_forward, mixer_norm=norm_of(p + "norm1"),
                                feed_forward_norm=norm_of(p + "norm2") if feed_forward is not None else None,
                                arrangement="hyper_pre_norm", extra=extra))
    # a layer without a feed-forward leaves norm2 and ls2 unread if the file has them
    unused = tuple(f"l{i}.{n}" for i, layer in enumerate(config.layers) if layer.mlp is None for n in ("norm2", "ls2"))
    return ModelSpec(
        hidden_size=config.width, vocab_size=config.vocab, layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i, adds_embedding=joins) for i, joins in config.runs()),
        final_norm=norm_of("final.norm"), embedding_weight="embed", head_weight="head",
        max_positions=config.max_positions, ignorable_weights=unused, pad_head_width=True)


def build_mugedra(config: MugedraConfig, dtype, device):
    from ..engine.model import DecoderModel
    return DecoderModel(mugedra_spec(config), dtype, device)


def mugedra_weight_specs(config: MugedraConfig):
    from ..engine.model import model_weight_specs
    return model_weight_specs(mugedra_spec(config))


register_architecture(MugedraConfig.ARCHITECTURE, MugedraConfig, build_mugedra, mugedra_weight_specs)
