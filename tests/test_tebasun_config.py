"""The Tebasun design's configuration, layout and cache plan, on the host."""
import json

import pytest

from test_gpu_tebasun import _config, _parallel, _rglru, _rot


def _layers():
    return [_rglru(), _parallel(), _rglru(width=32, blocks=2, conv=2, mlp={"kind": "dense", "ff": 24}),
            _parallel(heads=2, kv_heads=1, dim=8, rot=False, ff=None)]


def test_config_errors_name_the_key():
    from picolm_b200.config import ConfigError, config_from_dict
    good = _config(_layers(), loop=(1, 3, 2))
    assert config_from_dict(config_from_dict(good).to_dict()).to_dict() == config_from_dict(good).to_dict()
    for path, value, word in ((("layers", 0, "type"), "lstm", "lstm"), (("layers", 0, "mixer", "blocks"), 5, "blocks"),
                              (("layers", 1, "mixer", "left", "kv_heads"), 3, "kv_heads"),
                              (("layers", 1, "mixer", "left", "vdim"), 8, "vdim"),
                              (("layers", 1, "mixer", "left", "rot", "dims"), 7, "dims"),
                              (("layers", 1, "mixer", "right", "kv_heads"), 3, "kv_heads"),
                              (("layers", 2, "mlp", "kind"), "sparse", "sparse"), (("loop", "stop"), 9, "loop"),
                              (("loop", "times"), 0, "times"), (("token_side", "dim"), 0, "token_side")):
        bad = json.loads(json.dumps(good))
        node = bad
        for key in path[:-1]:
            node = node[key]
        node[path[-1]] = value
        with pytest.raises(ConfigError, match=word):
            config_from_dict(bad)
    for path in (("embedding",), ("norm", "eps"), ("layers", 1, "mixer", "left_scale"), ("layers", 1, "mixer", "right", "conv"),
                 ("layers", 1, "mixer", "left", "rot", "scaling", "fast")):
        bad = json.loads(json.dumps(good))
        node = bad
        for key in path[:-1]:
            node = node[key]
        del node[path[-1]]
        with pytest.raises(ConfigError, match=str(path[-1])):
            config_from_dict(bad)


def test_layout_schedule_and_cache_plan():
    """The looped range is named once per pass; every run owns what it keeps (a state for the diagonal recurrence;
    keys with values, and a state, for the two mixers side by side); the token inputs share one table; a layer
    without a feed-forward has no second norm."""
    from picolm_b200.config import config_from_dict, spec_of
    from picolm_b200.engine.model import Model
    layers = _layers()
    spec = spec_of(config_from_dict(_config(layers, loop=(1, 3, 2))))
    assert spec.schedule == (0, 1, 2, 1, 2, 3) and spec.run_input_at == ((1, 0, False), (3, 1, True))
    model = Model(spec, None)
    names = set(model.expected_tensors())
    assert {"embed", "side.embed", "loop.step", "final.norm", "final.norm.alpha", "final.norm.b", "l0.norm1.alpha",
            "l0.mix.ra.b", "l1.mix.left.sink", "l1.mix.left.q.norm", "l1.mix.right.q.conv", "l1.mix.right.dt_bias",
            "l2.mlp.down", "l3.side.proj", "l3.side.norm"} <= names
    assert "head" not in names and "l0.norm2" not in names and "l3.mlp.up" not in names and "l1.mix.left.v" not in names
    assert "l3.mix.left.rot" not in names and model.expected_tensors()["side.embed"].shape == (97, 4 * 6)
    caches = model.cache_specs()
    assert [c.kind for c in caches] == ["state", "kv", "state", "state", "kv", "state", "state", "kv", "state"]
    r = layers[1]["mixer"]["right"]
    channels = 2 * r["kv_heads"] * r["dim"] + r["heads"] * r["vdim"]
    assert caches[2].shape == (r["heads"] * r["dim"] * r["vdim"] + (r["conv"] - 1) * channels,)
    assert caches[0].shape == (48 + 2 * 48,) and caches[3].shape == (32 + 32,)
    assert caches[1].num_kv_heads == 2 and caches[1].head_dim == 16 and caches[1].values and caches[1].window is None
    from picolm_b200.cache import SequenceCache
    cache = SequenceCache(caches, max_tokens=256, max_seqs=3, allocate_storage=False)
    assert sorted(i for g in cache.kv_groups for i in g.layers) == [1, 4, 7]
    no_loop = spec_of(config_from_dict(_config(layers, side=None)))
    assert no_loop.schedule == (0, 1, 2, 3) and no_loop.run_input is None
    assert "side.embed" not in Model(no_loop, None).expected_tensors()


def test_random_weights_need_every_size():
    from picolm_b200.config import config_from_dict
    from picolm_b200.weights import random_tensors
    cfg = _config(_layers())
    del cfg["layers"][1]["mixer"]["right"]["rank"]
    with pytest.raises(ValueError, match="a1"):
        random_tensors(config_from_dict(cfg), 0)
