"""The Fupapel design's configuration, layout and cache plan, on the host."""
import json

import pytest

from test_gpu_fupapel import _attn, _attn2, _config, _latent, _moe


def _layers():
    return [_attn(), _attn2(kv_heads=1), _latent(mlp=None), _attn2(kv_heads=1, chunk=5, kv_from=1, mlp=_moe(top=1, identity=0, groups=None)),
            _attn(rot=0, chunk=None)]


def _edit(config, path, value=None, delete=False):
    bad = json.loads(json.dumps(config))
    node = bad
    for key in path[:-1]:
        node = node[key]
    if delete:
        del node[path[-1]]
    else:
        node[path[-1]] = value
    return bad


def test_config_errors_name_the_key():
    from picolm_b200.config import ConfigError, config_from_dict
    good = _config(_layers())
    assert config_from_dict(good).to_dict() == good
    for path, value, word in ((("layers", 0, "type"), "lstm", "lstm"), (("layers", 0, "mixer", "kv_heads"), 3, "kv_heads"),
                              (("layers", 0, "mixer", "rot", "dims"), 7, "dims"), (("layers", 0, "mixer", "mask", "size"), 0, "size"),
                              (("layers", 1, "mixer", "conv"), 0, "conv"), (("layers", 1, "mixer", "rot", "scaling", "factor"), "x", "factor"),
                              (("layers", 2, "mixer", "rot", "dims"), 4, "rot_dim"), (("layers", 3, "mixer", "kv_from"), 0, "kv_from"),
                              (("layers", 3, "mixer", "kv_from"), 3, "kv_from"), (("layers", 3, "mixer", "vdim"), 16, "vdim"),
                              (("layers", 0, "mlp", "kind"), "dense", "dense"), (("layers", 0, "mlp", "router", "top"), 9, "top"),
                              (("layers", 0, "mlp", "router", "groups", "count"), 3, "groups"),
                              (("layers", 0, "mlp", "router", "identity"), -1, "identity"), (("width",), 0, "width")):
        with pytest.raises(ConfigError, match=word):
            config_from_dict(_edit(good, path, value))
    assert config_from_dict(_edit(good, ("residual_mult",), delete=True)).residual_mult == 1.0
    for path in (("norm", "eps"), ("vocab",), ("layers", 0, "mixer", "scale"), ("layers", 1, "mixer", "conv"),
                 ("layers", 2, "mixer", "kv_rank"), ("layers", 2, "mixer", "rot"), ("layers", 1, "mixer", "rot", "scaling", "low"),
                 ("layers", 0, "mlp", "expert"), ("layers", 0, "mlp", "router", "experts")):
        with pytest.raises(ConfigError, match=str(path[-1])):
            config_from_dict(_edit(good, path, delete=True))


def test_layout_and_cache_plan():
    """Every layer keeps the row before its shift; attention layers keys and values; convolved ones their tail; the
    latent layer one row a position that serves as key and value; the borrowing layer reads its lender's keys and
    values and keeps its own shift row and tail; a layer without feed-forward has no second norm and no experts."""
    from picolm_b200.cache import SequenceCache
    from picolm_b200.config import config_from_dict, spec_of
    from picolm_b200.engine.model import Model
    spec = spec_of(config_from_dict(_config(_layers(), mult=0.25)))
    assert [layer.arrangement for layer in spec.layers] == ["parallel_norm"] * 5
    assert spec.layers[3].cache_of == 1 and spec.layers[0].params["residual_scale"] == 0.25
    model = Model(spec, None)
    names = model.expected_tensors()
    assert {"embed", "head", "final.norm", "l0.shift", "l0.norm2", "l0.mix.g", "l0.mix.q.norm", "l0.mlp.router", "l0.mlp.e5.down",
            "l1.mix.k.conv", "l1.mix.temp", "l1.mix.sink", "l2.mix.dkv", "l2.mix.sink", "l3.mix.q.conv", "l3.mix.temp"} <= set(names)
    for absent in ("l0.mix.sink", "l0.mix.temp", "l1.mix.g", "l2.norm2", "l2.mlp.router", "l3.mix.k", "l3.mix.v.conv", "l3.mix.k.norm",
                   "l0.mlp.e6.down", "l0.mlp.shared.up"):
        assert absent not in names
    assert names["l0.mlp.router"].shape == (8, 40) and names["l0.mlp.correction"].shape == (8,)
    assert names["l3.mlp.router"].shape == (6, 40) and names["l2.mix.g"].shape == (3, 40) and names["l0.mix.g"].shape == (4 * 24, 40)
    assert names["l2.mix.uq"].shape == (3 * (12 + 8), 28) and names["l2.mix.dkv"].shape == (24 + 8, 40)
    caches = model.cache_specs()
    assert [(c.kind, c.private) for c in caches] == [("state", True), ("kv", False), ("state", True), ("kv", False), ("state", True),
                                                     ("state", True), ("kv", False), ("state", True), ("state", True),
                                                     ("state", True), ("kv", False)]
    assert caches[4].shape == (2 * (4 * 16 + 16 + 8),) and caches[8].shape == (2 * 4 * 16,)
    assert caches[6].values is False and caches[6].num_kv_heads == 1 and caches[6].head_dim == 32
    assert caches[1].head_dim == 32 and caches[3].head_dim == 16            # max(dim, vdim), rounded up to 16
    assert model._run_caches[3] == [(7, True), (3, False), (8, True)]
    cache = SequenceCache(caches, max_tokens=256, max_seqs=3, allocate_storage=False)
    assert sorted(i for g in cache.kv_groups for i in g.layers) == [1, 3, 6, 10]


def test_random_weights_cover_every_tensor():
    from picolm_b200.config import config_from_dict
    from picolm_b200.engine.model import Model
    from picolm_b200.config import spec_of
    from picolm_b200.weights import random_tensors
    cfg = config_from_dict(_config(_layers()))
    tensors = random_tensors(cfg, 0)
    expected = Model(spec_of(cfg), None).expected_tensors()
    assert set(tensors) == set(expected)
    assert all(tuple(tensors[n].shape) == tuple(ws.shape) for n, ws in expected.items())
