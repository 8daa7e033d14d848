"""Lebedra without a GPU: the configuration, the model's spec, and the plain implementation's
own mechanisms on hand-made cases."""
import copy

import pytest
import torch

import plain_lebedra as P
from rosellm_b200.config import ConfigError
from rosellm_b200.config.base import parse_config, resolve_architecture
from rosellm_b200.config.lebedra import LebedraConfig
from rosellm_b200.models.model import named_params_of_spec
from rosellm_b200.parts.base import KVCacheSpec
from rosellm_b200.parts.latent import LatentAttention
from rosellm_b200.parts.standard import rotary_frequencies
from rosellm_b200.cache.sizing import kv_bytes_per_token
from tiny_lebedra import RAW_X, RAW_Y


def test_config_round_trip_and_registry():
    for raw in (RAW_X, RAW_Y):
        cfg = parse_config(raw)
        assert isinstance(cfg, LebedraConfig)
        assert LebedraConfig.from_dict(cfg.to_dict()) == cfg
    cfg = parse_config(RAW_X)
    assert cfg.layers[1].mlp.group_count == 4 and cfg.layers[1].mlp.group_keep == 2
    assert cfg.layers[2].mlp is None and cfg.layers[2].mixer.rot_dims == 2
    assert parse_config(RAW_Y).layers[0].mlp.group_count == 1  # no groups given: one group


@pytest.mark.parametrize("change, word", [
    (lambda r: r.__setitem__("width", 60), "width"),
    (lambda r: r["layers"][0].__setitem__("type", "other"), "type"),
    (lambda r: r["layers"][1]["mlp"]["router"].__setitem__("top", 7), "groups"),
    (lambda r: r["layers"][0]["mixer"]["rot"].__setitem__("dims", 3), "rot.dims"),
    (lambda r: r["layers"][0]["mlp"].__setitem__("kind", "sparse"), "kind"),
    (lambda r: r.pop("norm"), "norm"),
])
def test_config_refusals(change, word):
    raw = copy.deepcopy(RAW_X)
    change(raw)
    with pytest.raises(ConfigError, match=word):
        parse_config(raw)


def test_spec_names_every_tensor_once_and_shares_the_side_table():
    cfg = parse_config(RAW_X)
    spec = resolve_architecture(cfg.to_dict()).build_spec(cfg)
    params = named_params_of_spec(spec)
    names = [n for p in params for n, _ in p.sources()]
    assert names.count("side.embed") == len(cfg.layers)
    rest = [n for n in names if n != "side.embed"]
    assert len(rest) == len(set(rest))
    assert "l1.mlp.e11.down" in names and "l2.norm2" not in names and "l2.mlp.gate" not in names
    assert "l0.mix.dkv.norm" in names and "final.norm" in names and "head" in names
    # layer 2 has no feed-forward: its block arranges a mixer and the token input only
    kinds = [[n for n, _, _ in ls.parts] for ls in spec.layers]
    assert "feed_forward" not in kinds[2] and "token_input" in kinds[2]


def test_latent_cache_is_one_row_a_token():
    m = LatentAttention(hidden_size=64, num_heads=5, plain_dim=8, rot_dim=16, value_dim=12, kv_rank=20, scale=0.4,
                        rot_dims=16, rot_base=1e4, norm_eps=1e-5)
    spec = m.cache_spec()
    assert spec == KVCacheSpec(1, 40, None, planes=1)  # 20 + 16 filled up to a multiple of 8
    assert kv_bytes_per_token({0: spec}, "bfloat16") == 80
    assert kv_bytes_per_token({0: KVCacheSpec(2, 16)}, "float32") == 2 * 2 * 16 * 4
    with pytest.raises(ValueError):
        LatentAttention(hidden_size=64, num_heads=2, plain_dim=8, rot_dim=8, value_dim=8, kv_rank=600, scale=1.0,
                        rot_dims=8, rot_base=1e4, norm_eps=1e-5)


def test_rotary_frequencies():
    f = rotary_frequencies(8, 100.0)
    assert torch.allclose(f, torch.tensor([1.0, 100 ** -0.25, 100 ** -0.5, 100 ** -0.75]), rtol=1e-6)


def test_plain_rotation_keeps_the_rest_and_turns_pairs():
    v = torch.arange(12, dtype=torch.float64).view(1, 1, 12) + 1.0
    out = P.rotate_pairs(v.repeat(2, 1, 1), torch.tensor([0, 3]), dims=4, base=10.0)
    assert torch.equal(out[0], v[0])  # position 0: nothing turns
    assert torch.equal(out[1, 0, 4:], v[0, 0, 4:])  # beyond dims: unchanged
    a = 3.0
    assert out[1, 0, 0] == pytest.approx(1.0 * torch.cos(torch.tensor(a)) - 2.0 * torch.sin(torch.tensor(a)))
    assert out[1, 0, 1] == pytest.approx(2.0 * torch.cos(torch.tensor(a)) + 1.0 * torch.sin(torch.tensor(a)))
    # relative: the dot product of two turned vectors depends on the distance only
    q, k = torch.randn(1, 1, 4, dtype=torch.float64), torch.randn(1, 1, 4, dtype=torch.float64)
    d1 = (P.rotate_pairs(q, torch.tensor([7]), 4, 50.0) * P.rotate_pairs(k, torch.tensor([2]), 4, 50.0)).sum()
    d2 = (P.rotate_pairs(q, torch.tensor([105]), 4, 50.0) * P.rotate_pairs(k, torch.tensor([100]), 4, 50.0)).sum()
    assert d1 == pytest.approx(float(d2), abs=1e-9)


def test_plain_sink_counts_once_and_has_no_value():
    s = torch.zeros(1, 1, 3, dtype=torch.float64)
    p = P.softmax_with_sink(s, torch.tensor([0.0], dtype=torch.float64))
    assert torch.allclose(p, torch.full((1, 1, 3), 0.25, dtype=torch.float64))
    p = P.softmax_with_sink(s, torch.tensor([-1e9], dtype=torch.float64))
    assert torch.allclose(p, torch.full((1, 1, 3), 1 / 3, dtype=torch.float64))


def test_plain_routing_masks_groups_with_minus_infinity():
    """Four experts in two groups, one kept, top 2: with negative choice scores in the better
    group, the other group's experts must still not be chosen (they are -inf, not 0)."""
    w = {"r.router": torch.zeros(4, 2, dtype=torch.float64),
         "r.correction": torch.tensor([-0.9, -0.3, -0.95, -0.99], dtype=torch.float64)}
    idx, weight = P.route(torch.ones(1, 2, dtype=torch.float64), w, "r.", {"experts": 4, "top": 2,
                                                                           "groups": {"count": 2, "keep": 1}})
    assert sorted(idx[0].tolist()) == [0, 1]
    assert torch.allclose(weight, torch.full((1, 2), 0.25, dtype=torch.float64))  # scores without the correction
