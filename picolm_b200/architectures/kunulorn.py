"""Kunulorn as a layout of parts: every layer is a `pre_norm` arrangement with layer norms around an `attention`
mixer in its general form (biases, a norm over the whole of q and of k, a partial rotation in neighbouring pairs, a
mask of chunks, value heads of their own width) and a feed-forward that is a `gated_mlp` with clamped branches, a
`routed_mlp`, or absent.  This file only fills `PartSpec`s from `KunulornConfig` and names the tensors (`l<i>.norm1`,
`l<i>.mix.*`, `l<i>.mlp.*`, `embed`, `final.norm`); the parts know nothing of the design.  The logits are taken
against the embedding table itself (the head names the same tensor).

A layer with `kv_from: j` has no key and value tensors and reads the cache of layer j (`LayerSpec.cache_of`).

Constants the design fixes: the slope 1.702 of the dense feed-forward's gate; experts' tensors `e<k>.*`.
"""
from __future__ import annotations

from ..config.kunulorn import ARCHITECTURE, KunulornConfig
from ..config.registry import register_architecture
from ..config.spec import ModelSpec, PartSpec
from ..parts.block import pre_norm_layer

GATE_SLOPE = 1.702


def _mixer_spec(cfg: KunulornConfig, layer) -> PartSpec:
    m = layer.mixer
    position = PartSpec("none")
    if m["rot_dims"] > 0:
        position = PartSpec("rope", {"head_dim": m["dim"], "rotary_dim": m["rot_dims"], "theta": m["rot_base"],
                                     "scaling": None, "pairing": "adjacent", "max_positions": 1 << 30})
    return PartSpec("attention", {
        "hidden_size": cfg.width, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"],
        "value_dim": m["vdim"], "scale": m["scale"], "window": None, "chunk": m["mask_size"], "position": position,
        "bias": True, "bias_suffix": ".b", "qk_norm": {"eps": cfg.norm_eps, "q_name": "q.norm", "k_name": "k.norm"},
        "own_kv": m["kv_from"] is None, "q_name": "q", "k_name": "k", "v_name": "v", "o_name": "o"}, prefix="mix")


def _mlp_spec(cfg: KunulornConfig, mlp) -> PartSpec:
    d = cfg.width
    names = {"gate_name": "gate", "up_name": "up", "down_name": "down"}
    if mlp["kind"] == "dense":
        return PartSpec("gated_mlp", {"hidden_size": d, "intermediate_size": mlp["ff"], "activation": "swish_clamped",
                                      "limit": mlp["limit"], "slope": GATE_SLOPE, **names}, prefix="mlp")
    r = mlp["router"]
    shared = None
    if mlp.get("shared") is not None:
        shared = {"size": mlp["shared"]["ff"], "prefix": "shared", "gate": "sg"}
    return PartSpec("routed_mlp", {
        "hidden_size": d, "experts": r["experts"], "top": r["top"], "expert_size": mlp["expert"]["ff"],
        "route_scale": r["scale"], "groups": r.get("groups"), "correction_name": "correction", "router_name": "router",
        "expert_prefix": "e", "shared": shared, **names}, prefix="mlp")


def kunulorn_spec(cfg: KunulornConfig) -> ModelSpec:
    d = cfg.width

    def norm(name):
        return PartSpec("layernorm", {"size": d, "eps": cfg.norm_eps, "name": ""}, prefix=name)

    layers = []
    for i, layer in enumerate(cfg.layers):
        ff = _mlp_spec(cfg, layer.mlp) if layer.mlp is not None else None
        layers.append(pre_norm_layer(
            prefix=f"l{i}", mixer=_mixer_spec(cfg, layer), feed_forward=ff, mixer_norm=norm("norm1"),
            feed_forward_norm=norm("norm2") if ff is not None else None, cache_of=layer.mixer["kv_from"]))
    return ModelSpec(
        architecture=cfg.architecture, hidden_size=d, vocab_size=cfg.vocab,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": d, "name": "embed",
                                               "scale": cfg.embedding_scale}),
        layers=tuple(layers), schedule=tuple(range(len(layers))),
        final_norm=PartSpec("layernorm", {"size": d, "eps": cfg.norm_eps, "name": "norm"}, prefix="final"),
        lm_head=PartSpec("lm_head", {"vocab_size": cfg.vocab, "hidden_size": d, "name": "embed"}),
        max_positions=1 << 20,                            # the rotation's table is built for the cache's longest sequence
        ignored_tensors=tuple(rf"^l{i}\.norm2$" for i, layer in enumerate(cfg.layers) if layer.mlp is None),
    )


register_architecture(ARCHITECTURE, KunulornConfig.from_dict, kunulorn_spec)
