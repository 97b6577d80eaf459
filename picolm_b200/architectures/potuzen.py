"""Potuzen as a layout of parts: every layer is a `sandwich_norm` arrangement (a norm before and after each
sublayer) around one of three mixers and, if the layer has one, a dense feed-forward with the tanh form of GELU.
This file only fills `PartSpec`s from `PotuzenConfig` and names the tensors (`l<i>.norm1`, `l<i>.mix.*`,
`l<i>.mlp.*`, `embed`, `final.norm`, `head`); the parts know nothing of the design.

A layer that runs with another layer's weights (`weights_of`) is that layer named once more in the schedule: the
model keeps caches and states per run of the schedule, so each run has its own.
"""
from __future__ import annotations

from ..config.potuzen import ARCHITECTURE, PotuzenConfig
from ..config.registry import register_architecture
from ..config.spec import ModelSpec, PartSpec
from ..parts.block import sandwich_norm_layer


def _mixer_spec(cfg: PotuzenConfig, layer) -> PartSpec:
    m, d, eps = layer.mixer, cfg.width, cfg.norm_eps
    if layer.type == "latent_attention":
        return PartSpec("latent_attention", {
            "hidden_size": d, "heads": m["heads"], "dim": m["dim"], "vdim": m["vdim"], "kv_rank": m["kv_rank"],
            "q_rank": m["q_rank"], "scale": m["scale"], "window": m["mask"]["size"], "eps": eps}, prefix="mix")
    if layer.type == "mamba2":
        return PartSpec("mamba2", {
            "hidden_size": d, "heads": m["heads"], "vdim": m["vdim"], "state": m["state"], "groups": m["groups"],
            "conv": m["conv"], "norm_groups": m["norm_groups"], "eps": eps}, prefix="mix")
    if layer.type == "gla":
        # the width of the decay's bottleneck is given by the tensors' shapes (an optional key names it for random weights)
        return PartSpec("gla", {
            "hidden_size": d, "heads": m["heads"], "dim": m["dim"], "vdim": m["vdim"], "tau": m["tau"],
            "decay_rank": m.get("decay_rank"), "eps": eps}, prefix="mix")
    raise ValueError(f"no mixer of type {layer.type!r}")


def potuzen_spec(cfg: PotuzenConfig) -> ModelSpec:
    d = cfg.width

    def norm(name):
        return PartSpec("rmsnorm", {"size": d, "eps": cfg.norm_eps, "name": ""}, prefix=name)

    layers, number, ignored = [], {}, []
    for i, layer in enumerate(cfg.layers):
        if layer.weights_of is not None:
            continue
        ff = None
        if layer.mlp is not None:
            ff = PartSpec("gated_mlp", {"hidden_size": d, "intermediate_size": layer.mlp["ff"], "activation": "gelu_tanh",
                                        "gate_name": "gate", "up_name": "up", "down_name": "down"}, prefix="mlp")
        else:
            ignored.append(rf"^l{i}\.norm2b?$")          # a layer that only mixes has no use for them
        number[i] = len(layers)
        layers.append(sandwich_norm_layer(
            prefix=f"l{i}", mixer=_mixer_spec(cfg, layer), mixer_norm=norm("norm1"), mixer_post_norm=norm("norm1b"),
            feed_forward=ff, feed_forward_norm=norm("norm2") if ff else None,
            feed_forward_post_norm=norm("norm2b") if ff else None))
    schedule = tuple(number[i if layer.weights_of is None else layer.weights_of] for i, layer in enumerate(cfg.layers))
    return ModelSpec(
        architecture=cfg.architecture, hidden_size=d, vocab_size=cfg.vocab,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": d, "name": "embed"}),
        layers=tuple(layers), schedule=schedule,
        final_norm=PartSpec("rmsnorm", {"size": d, "eps": cfg.norm_eps, "name": "norm"}, prefix="final"),
        lm_head=PartSpec("lm_head", {"vocab_size": cfg.vocab, "hidden_size": d, "name": "head"}),
        max_positions=1 << 30,                            # no position encoding: nothing bounds a sequence but the cache
        ignored_tensors=tuple(ignored),
    )


register_architecture(ARCHITECTURE, PotuzenConfig.from_dict, potuzen_spec)
