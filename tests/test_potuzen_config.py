"""The Potuzen design's configuration, layout and cache plan, on the host."""
import json

import pytest

from test_gpu_potuzen import MIXED, _config, _latent, _mamba


def test_config_errors_name_the_key():
    from picolm_b200.config import ConfigError, config_from_dict
    good = _config(MIXED)
    assert config_from_dict(good).to_dict() == good
    for path, value, word in ((("layers", 0, "mixer", "mask"), {}, "size"), (("layers", 1, "type"), "mamba3", "mamba3"),
                              (("layers", 3, "weights_of"), 3, "weights_of"), (("layers", 2, "mixer", "tau"), 0.0, "tau"),
                              (("layers", 1, "mlp", "kind"), "sparse", "sparse")):
        bad = json.loads(json.dumps(good))
        node = bad
        for key in path[:-1]:
            node = node[key]
        node[path[-1]] = value
        with pytest.raises(ConfigError, match=word):
            config_from_dict(bad)
    bad = json.loads(json.dumps(good))
    del bad["layers"][1]["mixer"]["state"]
    with pytest.raises(ConfigError, match="state"):
        config_from_dict(bad)


def test_layout_schedule_and_cache_plan():
    """Shared weights become a second run of the owner in the schedule; every run has a cache or state of its own;
    latent caches keep one row per position and no values; a layer without a feed-forward has three parts."""
    from picolm_b200.config import config_from_dict, spec_of
    from picolm_b200.engine.model import Model
    layers = [_latent(window=9), _mamba(), dict(_latent(window=9), weights_of=0), dict(_mamba(conv=1), mlp=None)]
    spec = spec_of(config_from_dict(_config(layers)))
    assert spec.schedule == (0, 1, 0, 2) and [layer.prefix for layer in spec.layers] == ["l0", "l1", "l3"]
    model = Model(spec, None)
    names = set(model.expected_tensors())
    assert {"embed", "head", "final.norm", "l0.norm1b", "l0.mix.dkv.norm", "l1.mix.conv.b", "l3.mix.A_log"} <= names
    assert not any(n.startswith("l2.") for n in names) and "l3.norm2" not in names and "l3.mlp.up" not in names
    caches = model.cache_specs()
    assert [c.kind for c in caches] == ["kv", "state", "kv", "state"]
    assert caches[0].values is False and caches[0].window == 9 and caches[0].num_kv_heads == 1 and caches[0].head_dim == 20
    m = layers[1]["mixer"]
    ssm = m["heads"] * m["state"] * m["vdim"]
    channels = m["heads"] * m["vdim"] + 2 * m["groups"] * m["state"]
    assert caches[1].shape == (ssm + (m["conv"] - 1) * channels,) and caches[3].shape == (ssm,)
    from picolm_b200.cache import SequenceCache
    cache = SequenceCache(caches, max_tokens=256, max_seqs=3, allocate_storage=False)
    assert len(cache.kv_groups) == 1 and cache.kv_groups[0].layers == [0, 2] and sorted(cache.state_specs) == [1, 3]


def test_random_weights_need_every_size():
    from picolm_b200.config import config_from_dict
    from picolm_b200.weights import random_tensors
    cfg = _config(MIXED)
    del cfg["layers"][2]["mixer"]["decay_rank"]
    with pytest.raises(ValueError, match="a1"):
        random_tensors(config_from_dict(cfg), 0)
