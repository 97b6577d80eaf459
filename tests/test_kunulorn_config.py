"""The Kunulorn design's configuration, layout and cache plan, on the host."""
import json

import pytest

from test_gpu_kunulorn import MODELS, _attn, _config, _dense, _moe


def test_config_errors_name_the_key():
    from picolm_b200.config import ConfigError, config_from_dict
    layers, kw = MODELS["borrowed"]
    good = _config(layers, **kw)
    assert config_from_dict(good).to_dict() == good
    for path, value, word in ((("layers", 0, "mixer", "mask"), {}, "size"), (("layers", 1, "type"), "conv", "conv"),
                              (("layers", 2, "mixer", "kv_from"), 2, "kv_from"), (("layers", 3, "mixer", "kv_from"), 2, "kv_from"),
                              (("layers", 0, "mlp", "kind"), "sparse", "sparse"), (("layers", 0, "mixer", "rot", "dims"), 7, "rot.dims"),
                              (("layers", 3, "mlp", "router", "top"), 9, "top"), (("layers", 3, "mlp", "router", "groups", "keep"), 7, "groups"),
                              (("layers", 2, "mixer", "vdim"), 16, "vdim"), (("layers", 1, "mixer", "heads"), 3, "heads"),
                              (("embedding",), {}, "scale")):
        bad = json.loads(json.dumps(good))
        node = bad
        for key in path[:-1]:
            node = node[key]
        node[path[-1]] = value
        with pytest.raises(ConfigError, match=word):
            config_from_dict(bad)
    bad = json.loads(json.dumps(good))
    del bad["layers"][0]["mlp"]["limit"]
    with pytest.raises(ConfigError, match="limit"):
        config_from_dict(bad)


def test_layout_and_cache_plan():
    """Layers that borrow keys and values own no cache and no key or value tensors; the head is the embedding table;
    a layer without a feed-forward has two parts; heads are kept at the wider of keys and values, rounded up to 16."""
    from picolm_b200.config import config_from_dict, spec_of
    from picolm_b200.engine.model import Model
    layers, kw = MODELS["borrowed"]
    spec = spec_of(config_from_dict(_config(layers, **kw)))
    assert spec.schedule == (0, 1, 2, 3) and [layer.cache_of for layer in spec.layers] == [None, None, 0, 1]
    assert spec.lm_head.params["name"] == spec.embedding.params["name"] == "embed" and spec.embedding.params["scale"] == 3.5
    model = Model(spec, None)
    names = set(model.expected_tensors())
    assert {"embed", "final.norm", "l0.norm1", "l0.mix.q.b", "l0.mix.k.norm", "l2.mix.q.norm", "l2.mix.o.b", "l1.mlp.router",
            "l1.mlp.correction", "l1.mlp.e3.down", "l3.mlp.shared.sg", "l3.mlp.shared.up", "l0.mlp.gate"} <= names
    assert not {"head", "l2.mix.k", "l2.mix.v.b", "l2.mix.k.norm", "l3.mix.v", "l2.norm2", "l2.mlp.up", "l1.mlp.shared.sg", "l1.mlp.e4.up"} & names
    caches = model.cache_specs()
    assert [(c.kind, c.num_kv_heads, c.head_dim, c.window) for c in caches] == [("kv", 1, 16, None), ("kv", 2, 16, None)]
    wide = Model(spec_of(config_from_dict(_config([_attn(heads=2, kv_heads=2, dim=24, vdim=40)]))), None)
    assert wide.cache_specs()[0].head_dim == 48
    assert wide.expected_tensors()["l0.mix.o"].shape == (40, 80) and wide.expected_tensors()["l0.mix.v.b"].shape == (80,)


def test_routed_feed_forward_refuses_what_cannot_be_chosen():
    from picolm_b200.parts import build_part
    from picolm_b200.config.spec import PartSpec
    params = {"hidden_size": 8, "experts": 6, "top": 3, "expert_size": 4, "route_scale": 1.0, "groups": {"count": 3, "keep": 1},
              "router_name": "router", "expert_prefix": "e", "gate_name": "gate", "up_name": "up", "down_name": "down"}
    with pytest.raises(ValueError, match="cannot give"):
        build_part("feed_forward", PartSpec("routed_mlp", params), None)
    part = build_part("feed_forward", PartSpec("routed_mlp", dict(params, top=2)), None)
    assert set(part.weight_specs()) == {"router"} | {f"e{e}.{n}" for e in range(6) for n in ("gate", "up", "down")}


def test_key_mask_number():
    from picolm_b200.ops.attention import key_mask
    from picolm_b200.ops import KernelError
    assert key_mask(None) == 0 and key_mask(9) == 9 and key_mask(None, 64) == -64
    with pytest.raises(KernelError):
        key_mask(4, 4)
