"""Tulipel's configuration and host-side pieces (no GPU): config.json in and out, refusals, the run
order's cache slots, tensor declarations, the rotary frequencies against the plain implementation."""
import copy

import numpy as np
import pytest

import plain_tulipel as plain
from tulipel_helpers import P, Q

from sprout_lm_b200.config import ConfigError, TulipelConfig, parse_config
from sprout_lm_b200.models.decoder import DecoderModel
from sprout_lm_b200.parts.rope import InterleavedRotary, ScaledHalfSplitRotary


@pytest.mark.parametrize("raw", [P, Q])
def test_round_trip_and_registry(raw):
    config = parse_config(raw)
    assert isinstance(config, TulipelConfig)
    assert parse_config(config.to_dict()) == config
    assert config.to_dict()["layers"] == raw["layers"]


def test_run_order_shares_cache_slots():
    spec = parse_config(P).model_spec()
    assert [(c.layer, c.cache, c.writes_cache) for c in spec.order] == \
        [(0, 0, True), (1, 1, True), (2, 0, False), (3, 2, True), (4, 1, False)]
    assert spec.cache_slots == 3
    model = DecoderModel(spec)
    assert [(s.kv_heads, s.head_dim, s.value_width) for s in model.cache_specs()] == [(1, 56, 0), (1, 48, 0), (1, 40, 0)]


def test_tensor_declarations():
    names = {d.name: tuple(d.shape) for d in DecoderModel(parse_config(P).model_spec()).tensor_decls()}
    assert names["embed"] == (301, 72) and names["head"] == (301, 72) and names["final.norm"] == (72,)
    assert names["l0.mix.dq"] == (40, 72) and names["l0.mix.uq"] == (3 * 32, 40) and names["l0.mix.dkv"] == (56, 72)
    assert names["l0.mix.uk"] == (3 * 24, 48) and names["l0.mix.uv"] == (3 * 20, 48) and names["l0.mix.sink"] == (3,)
    assert names["l1.mix.q"] == (5 * 32, 72) and "l1.mix.dq" not in names
    assert "l1.norm2" not in names and "l1.mlp.up" not in names          # a layer without a feed-forward
    assert "l2.mix.dkv" not in names and "l2.mix.dkv.norm" not in names  # reads layer 0's rows
    assert names["l2.mix.uk"] == (2 * 12, 48)
    assert [names[f"l{i}.dwa"] for i in range(5)] == [(2,), (3,), (4,), (5,), (6,)]
    assert names["l0.mlp.act"] == (4,)


@pytest.mark.parametrize("change", [
    lambda c: c["layers"][2]["mixer"].__setitem__("kv_from", 2),          # itself
    lambda c: c["layers"][2]["mixer"].__setitem__("kv_from", 1),          # another latent size and rotation
    lambda c: c["layers"][4]["mixer"].__setitem__("kv_from", 2),          # a layer that has no rows of its own
    lambda c: c["layers"][0].__setitem__("type", "window_attention"),
    lambda c: c["layers"][0]["mixer"].pop("q_rank"),
    lambda c: c["layers"][0]["mlp"].__setitem__("kind", "routed"),
    lambda c: c["layers"][3]["mixer"]["rot"].__setitem__("dims", 26),
    lambda c: c.pop("logit_softcap"),
    lambda c: c["norm"].pop("eps"),
    lambda c: c.__setitem__("vocab", 0),
])
def test_refusals(change):
    raw = copy.deepcopy(P)
    change(raw)
    with pytest.raises(ConfigError):
        parse_config(raw)


def test_rotary_frequencies_match_plain():
    for rot, cls in (({"base": 30000.0, "dims": 16, "scaling": {"factor": 4.0, "original": 64, "fast": 16.0, "slow": 2.0}}, ScaledHalfSplitRotary),
                     ({"base": 90000.0, "dims": 6, "scaling": {"factor": 16.0, "original": 32, "fast": 8.0, "slow": 1.0}}, ScaledHalfSplitRotary),
                     ({"base": 20000.0, "dims": 64, "scaling": {"factor": 8.0, "original": 1024, "fast": 32.0, "slow": 1.0}}, ScaledHalfSplitRotary),
                     ({"base": 700.0, "dims": 16}, ScaledHalfSplitRotary), ({"base": 5000.0, "dims": 8}, InterleavedRotary)):
        part = cls("", dims=rot["dims"], theta=rot["base"], max_positions=8, scaling=rot.get("scaling"))
        freq, magnitude = plain.rotation_frequencies(rot)
        assert np.allclose(part.frequencies(), freq, rtol=1e-14, atol=0)
        assert abs(part.magnitude - magnitude) < 1e-15
        if "scaling" in rot:                   # the stretch reaches some pairs and not others
            base = np.array([rot["base"] ** (-2.0 * i / rot["dims"]) for i in range(rot["dims"] // 2)])
            ratio = freq / base
            assert ratio[0] == 1.0 and np.isclose(ratio[-1], 1.0 / rot["scaling"]["factor"])
