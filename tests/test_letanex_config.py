"""Letanex's configuration and its place in the registries (no GPU)."""
import copy

import numpy as np
import pytest

import letanex_helpers as lh
import plain_letanex as plain
from sprout_lm_b200.config import ConfigError, LetanexConfig, parse_config, registered_architectures
from sprout_lm_b200.models.decoder import DecoderModel


def test_registered_and_round_trip():
    assert "Letanex" in registered_architectures()
    for raw, _, _ in lh.CONFIGS.values():
        config = parse_config(raw)
        assert isinstance(config, LetanexConfig)
        assert parse_config(config.to_dict()) == config
        assert config.to_dict()["layers"] == raw["layers"]


def test_model_spec_follows_the_file():
    spec = parse_config(lh.P).model_spec()
    kinds = [layer.mixer.kind for layer in spec.layers]
    assert kinds == ["decay_linear_attention", "multimap_attention", "multimap_attention", "decay_linear_attention",
                     "multimap_attention"]
    assert [layer.feed_forward.kind for layer in spec.layers] == ["routed_experts", "relu2_mlp", "none", "routed_experts",
                                                                  "routed_experts"]
    assert [len(layer.norms) for layer in spec.layers] == [4, 4, 2, 4, 4]
    # the third layer reads the second layer's cache slot and writes nothing
    assert spec.order[2].cache == spec.order[1].cache and not spec.order[2].writes_cache
    assert spec.layers[2].mixer.params["own_kv"] is False and spec.layers[1].mixer.params["own_kv"] is True
    assert spec.layers[1].mixer.params["out_scale"] == pytest.approx(0.7)
    assert spec.layers[4].mixer.params["position"].params["factor"] == 1.0
    assert spec.layers[1].mixer.params["position"].params["factor"] == 4.0
    model = DecoderModel(spec)
    specs = model.cache_specs()
    assert specs[spec.order[1].cache].kv_heads == 2 and specs[spec.order[1].cache].head_dim == 32 \
        and specs[spec.order[1].cache].value_width == 24
    assert specs[spec.order[0].cache] is None                           # a lightning layer keeps nothing per token
    states = model.state_specs()
    assert states[0].shape == (3, 8, 20) and states[3].shape == (1, 24, 8) and states[1] is None
    names = {decl.name: decl.shape for decl in model.tensor_decls()}
    assert names["l0.mlp.router"] == (7, 72) and names["l0.mlp.correction"] == (7,)
    assert names["l0.mlp.e4.gate"] == (24, 72) and "l0.mlp.e5.gate" not in names        # identity experts have no tensors
    assert names["l0.mlp.shared.down"] == (72, 40) and "l3.mlp.shared.gate" not in names
    assert names["l1.mix.q"] == (6 * 2 * 16, 72) and names["l1.mix.k"] == (2 * 2 * 16, 72) and names["l1.mix.v"] == (48, 72)
    assert "l2.mix.k" not in names and "l2.mix.v" not in names and names["l2.mix.lq1"] == (16,)
    assert "l2.norm2" not in names and names["l2.norm1b"] == (72,)
    assert names["l3.mix.g"] == (8, 72) and names["l3.mix.norm"] == (8,)


@pytest.mark.parametrize("edit, text", [
    (lambda c: c["layers"][1]["mixer"].__setitem__("heads", 5), "multiple of kv_heads"),
    (lambda c: c["layers"][1]["mixer"]["rot"].__setitem__("dims", 18), "rot.dims"),
    (lambda c: c["layers"][2]["mixer"].__setitem__("kv_from", 0), "kv_from"),
    (lambda c: c["layers"][2]["mixer"].__setitem__("kv_from", 3), "kv_from"),
    (lambda c: c["layers"][2]["mixer"].__setitem__("vdim", 16), "kv_from"),
    (lambda c: c["layers"][0]["mixer"].__setitem__("decay", [0.5, 0.5]), "decay"),
    (lambda c: c["layers"][0]["mixer"].__setitem__("decay", [0.5, -0.1, 0.5]), "decay"),
    (lambda c: c["layers"][0]["mlp"]["router"].__setitem__("top", 9), "top"),
    (lambda c: c["layers"][0]["mlp"].pop("expert"), "expert"),
    (lambda c: c["layers"][0].__setitem__("type", "window"), "type"),
    (lambda c: c["norm"].pop("eps"), "eps"),
    (lambda c: c.pop("width"), "width"),
])
def test_refusals(edit, text):
    raw = copy.deepcopy(lh.P)
    edit(raw)
    with pytest.raises(ConfigError, match=text):
        parse_config(raw)


def test_plain_mechanisms_agree_with_their_definitions():
    """The oracle's own pieces against direct arithmetic on tiny inputs."""
    rng = np.random.default_rng(0)
    x = rng.normal(size=(3, 6))
    w = rng.normal(size=6)
    got = plain.layer_norm(x, w, 1e-5)
    assert np.allclose(got, (x - x.mean(-1, keepdims=True)) / np.sqrt(x.var(-1, keepdims=True) + 1e-5) * w)
    # rotation by position 0 is the identity; a pair turns by its angle
    v = rng.normal(size=(2, 1, 8))
    rot = {"base": 100.0, "dims": 4, "scaling": {"factor": 2.0}}
    turned = plain.rotate(v, [0, 3], rot)
    assert np.allclose(turned[0], v[0]) and np.allclose(turned[1, 0, 4:], v[1, 0, 4:])
    angle = 3 * 100.0 ** (-2.0 / 4) / 2.0
    assert np.isclose(turned[1, 0, 1], v[1, 0, 1] * np.cos(angle) - v[1, 0, 3] * np.sin(angle))
    # the recurrence in closed form: o_t = sum_{j<=t} decay^(t-j) (q_t . k_j) v_j
    q, k, val = rng.normal(size=(5, 1, 3)), rng.normal(size=(5, 1, 3)), rng.normal(size=(5, 1, 2))
    out, _ = plain.decay_recurrence(q, k, val, [0.8])
    want = sum(0.8 ** (4 - j) * (q[4, 0] @ k[j, 0]) * val[j, 0] for j in range(5))
    assert np.allclose(out[4, 0], want)
    # routing: the correction steers the choice, the weights ignore it
    weights = {"r.router": np.array([[1.0, 0.0], [0.0, 1.0], [0.5, 0.5]]), "r.correction": np.array([0.0, 0.0, 10.0])}
    chosen, weight = plain.route(np.array([[2.0, 0.0]]), weights, "r.", {"experts": 2, "identity": 1, "top": 2, "scale": 3.0})
    s = plain.softmax(np.array([[2.0, 0.0, 1.0]]))
    assert list(chosen[0]) == [2, 0] and np.allclose(weight[0], np.array([s[0, 2], s[0, 0]]) / (s[0, 2] + s[0, 0]) * 3.0)
