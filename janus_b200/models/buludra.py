"""The Buludra decoder as data: a `ModelSpec` made from a `BuludraConfig`.

Layers differ in their mixer: grouped-query softmax attention with normed heads and a query temperature
(`parts.capped_attention` without cap, chunk, rotation or gate), gated linear attention with a decay per key channel
(`parts.gated_linear`), or two mixers side by side that join as a weighted sum (`parts.parallel` without branch norms):
softmax attention with rotary positions, unit-norm heads and a sink beside the matrix memory with exponential gates
(`parts.gated_linear`).  The feed-forward is a dense gated one (`parts.feedforward`), a mixture of experts chosen by
softmax scores among the best groups, weighted on their outputs, with a gated shared expert (`parts.routed`), or none.
Root-mean-square norms, pre-norm; the logits are soft-capped.  A layer that names `weights_of` is the same `LayerSpec`
run at a second place of the schedule: same tensors, a cache or state of its own.  Tensor names: `embed`,
`l<i>.norm1`, `l<i>.norm2`, `l<i>.mix.*`, `l<i>.mlp.*`, `final.norm`, `head`.
"""
from __future__ import annotations

from typing import Dict, List

from ..config.buludra import BuludraConfig, DenseConfig
from ..config.registry import register_architecture
from ..parts.base import LayerSpec, ModelSpec, PartSpec, ScheduleEntry


def _names(prefix: str, pairs) -> Dict[str, str]:
    return {param: prefix + tensor for param, tensor in pairs}


def _mixer_spec(config: BuludraConfig, i: int) -> PartSpec:
    layer, p = config.layers[i], f"l{i}.mix."
    m = layer.mixer
    if layer.type == "attention":
        return PartSpec("capped_attention",
                        dict(hidden_size=config.width, num_heads=m.heads, num_kv_heads=m.kv_heads, dim=m.dim, vdim=m.vdim,
                             scale=m.scale, eps=config.eps, qk_norm=True, gate=False,
                             q_temp=(m.temp_coef, m.temp_every) if m.temp_every else None),
                        weights=_names(p, (("q", "q"), ("k", "k"), ("v", "v"), ("o", "o"), ("q_norm", "q.norm"),
                                           ("k_norm", "k.norm"))))
    if layer.type == "gla":
        return PartSpec("gated_linear_attention",
                        dict(hidden_size=config.width, num_heads=m.heads, dim=m.dim, vdim=m.vdim, rank=m.rank, tau=m.tau,
                             eps=config.eps),
                        weights=_names(p, (("q", "q"), ("k", "k"), ("v", "v"), ("g", "g"), ("a1", "a1"), ("a2", "a2"),
                                           ("a2_bias", "a2.b"), ("norm", "norm"), ("o", "o"))))
    a, r = m.left, m.right
    position = None
    if a.rot_dims:
        position = PartSpec("ramped_rotary", dict(dims=a.rot_dims, theta=a.rot_base, max_positions=config.max_positions,
                                                  scaling=None))
    left = PartSpec("capped_attention",
                    dict(hidden_size=config.width, num_heads=a.heads, num_kv_heads=a.kv_heads, dim=a.dim, vdim=a.vdim,
                         scale=a.scale, eps=config.eps, qk_norm="unit", gate=False, sink=True, position=position,
                         rotary_dims=a.rot_dims))
    right = PartSpec("matrix_memory",
                     dict(hidden_size=config.width, num_heads=r.heads, dim=r.dim, vdim=r.vdim, gate_cap=r.gate_cap,
                          eps=config.eps))
    weights = {"left." + n: p + "left." + n for n in ("q", "k", "v", "o")}
    weights.update({"right." + n: p + "right." + t for n, t in
                    (("q", "q"), ("k", "k"), ("v", "v"), ("g", "g"), ("i", "i"), ("f", "f"), ("i_bias", "i.b"),
                     ("f_bias", "f.b"), ("norm", "norm"), ("o", "o"))})
    return PartSpec("parallel", dict(hidden_size=config.width, left=left, right=right, eps=config.eps, branch_norm=False,
                                     left_mult=m.left_scale, right_mult=m.right_scale), weights=weights)


def _feed_forward_spec(config: BuludraConfig, i: int) -> PartSpec:
    mlp, p = config.layers[i].mlp, f"l{i}.mlp."
    if isinstance(mlp, DenseConfig):
        return PartSpec("swiglu", dict(hidden_size=config.width, intermediate_size=mlp.ff, pad_width=True),
                        weights=dict(gate=p + "gate", up=p + "up", down=p + "down"))
    weights = {"router": p + "router"}
    for e in range(mlp.experts):
        weights.update({f"e{e}_{n}": p + f"e{e}.{n}" for n in ("gate", "up", "down")})
    if mlp.shared_ff:
        weights.update({"shared_gate": p + "shared.gate", "shared_up": p + "shared.up", "shared_down": p + "shared.down",
                        "shared_sg": p + "shared.sg"})
    return PartSpec("routed_experts",
                    dict(hidden_size=config.width, intermediate_size=mlp.ff, experts=mlp.experts, top=mlp.top,
                         score="softmax", groups=(mlp.groups, mlp.keep) if mlp.groups else None, weight_on="output",
                         shared_size=mlp.shared_ff or None, shared_gate=bool(mlp.shared_ff)), weights=weights)


def buludra_spec(config: BuludraConfig) -> ModelSpec:
    layers: List[LayerSpec] = []
    index_of: Dict[int, int] = {}           # configuration layer with tensors of its own -> index among the LayerSpecs
    norm_of = lambda name: PartSpec("rms_norm", dict(width=config.width, eps=config.eps), weights=dict(gamma=name))  # noqa: E731
    unused = []
    for i, layer in enumerate(config.layers):
        if layer.weights_of is not None:
            continue
        p = f"l{i}."
        feed_forward = _feed_forward_spec(config, i) if layer.mlp is not None else None
        if feed_forward is None:
            unused.append(p + "norm2")      # a layer without a feed-forward leaves norm2 unread if the file has it
        index_of[i] = len(layers)
        layers.append(LayerSpec(mixer=_mixer_spec(config, i), feed_forward=feed_forward, mixer_norm=norm_of(p + "norm1"),
                                feed_forward_norm=norm_of(p + "norm2") if feed_forward is not None else None,
                                arrangement="pre_norm"))
    logit_transforms = ()
    if config.logit_softcap:
        logit_transforms = (PartSpec("scale_soft_cap", dict(scale=1.0, cap=config.logit_softcap)),)
    return ModelSpec(
        hidden_size=config.width, vocab_size=config.vocab, layers=tuple(layers),
        schedule=tuple(ScheduleEntry(index_of[config.owner(i)]) for i in range(len(config.layers))),
        final_norm=norm_of("final.norm"), embedding_weight="embed", head_weight="head",
        max_positions=config.max_positions, ignorable_weights=tuple(unused), logit_transforms=logit_transforms,
        pad_head_width=True)


def build_buludra(config: BuludraConfig, dtype, device):
    from ..engine.model import DecoderModel
    return DecoderModel(buludra_spec(config), dtype, device)


def buludra_weight_specs(config: BuludraConfig):
    from ..engine.model import model_weight_specs
    return model_weight_specs(buludra_spec(config))


register_architecture(BuludraConfig.ARCHITECTURE, BuludraConfig, build_buludra, buludra_weight_specs)
