"""Porovik without a GPU: configuration, refusals, the spec it builds, cache and state arithmetic, and the
plain implementation's mechanisms on cases small enough to work out by hand."""
import copy
import math

import pytest
import torch

import plain_porovik as P
from tiny_porovik import TINY, load_folder, write_tiny

from rosellm_b200.config.base import ConfigError, parse_config, resolve_architecture
from rosellm_b200.config.porovik import PorovikConfig
from rosellm_b200.models.model import Model, named_params_of_spec
from rosellm_b200.weights.loader import WeightError, match_tensors


def spec_of(raw):
    cfg = parse_config(raw)
    return cfg, resolve_architecture(cfg.to_dict()).build_spec(cfg)


@pytest.mark.parametrize("name", list(TINY))
def test_configuration_round_trip_and_spec(name):
    raw = TINY[name]["raw"]
    cfg, spec = spec_of(raw)
    assert isinstance(cfg, PorovikConfig) and PorovikConfig.from_dict(cfg.to_dict()) == cfg
    assert len(spec.layers) == len(raw["layers"]) and spec.head.kind == "tied_to_embedding"
    kinds = {"attention": "biased_attention", "general_delta": "delta_rule", "hgrn2": "gated_recurrence"}
    mixing = []
    for lr, ls in zip(raw["layers"], spec.layers):
        assert ls.part("mixer").kind == kinds[lr["type"]]
        assert (lr["mlp"] is None) == ("feed_forward" not in [n for n, _, _ in ls.parts])
        if lr["type"] == "attention":
            mixing.append(ls.part("mixer").params["value_mix"])
            assert (mixing[-1] is not None) == bool(lr["mixer"].get("v_mix"))
    taking_part = [m for m in mixing if m is not None]
    assert taking_part[:1] in ([], ["source"]) and all(m == "mix" for m in taking_part[1:])


def test_refusals():
    raw = TINY["A"]["raw"]
    for path, value in ((("layers", 0, "type"), "conv"), (("layers", 0, "mixer", "kv_heads"), 4), (("width",), 60),
                        (("embedding", "bigram", "buckets"), 0), (("layers", 1, "mlp", "router", "top"), 9),
                        (("layers", 3, "mixer", "vdim"), 12), (("layers", 3, "mixer", "kv_heads"), 1), (("norm", "eps"), 0.0), (("layers", 0, "mixer", "q_temp", "every"), 0)):
        bad = copy.deepcopy(raw)
        at = bad
        for k in path[:-1]:
            at = at[k]
        at[path[-1]] = value
        with pytest.raises(ConfigError):
            parse_config(bad)


def test_cache_rows_state_slots_and_a_rank_taken_from_the_file(tmp_path):
    cfg, spec = spec_of(TINY["A"]["raw"])
    m = Model(spec, torch.float32, "cpu")
    kv, st = m.kv_specs(), m.state_specs()
    assert set(kv) == {0, 3} and all(s.planes == 1 for s in kv.values())
    assert kv[0].num_kv_heads == 2 and kv[0].head_dim == 40   # key 20 -> 24, value 10 -> 34, filled up to 40
    assert st["embedding"].shape == (1,) and st["embedding"].dtype == torch.int32
    assert st[1].shape == (3, 24, 24) and st[2].shape == (2, 40, 24) and st[4].shape == (2, 8, 8)
    # without decay_rank in the configuration, the low rank is whatever the file's tensors have
    folder = write_tiny("A", str(tmp_path))
    raw, tensors = load_folder(folder)
    for layer in raw["layers"]:
        layer["mixer"].pop("decay_rank", None)
    _, spec2 = spec_of(raw)
    match_tensors(named_params_of_spec(spec2), tensors, source="test")
    m2 = Model(spec2, torch.float32, "cpu")
    m2.load_tensors(tensors)
    assert m2.layers[1].mixer.rank == 5 and m2.layers[4].mixer.rank == 3
    del tensors["l1.mix.w0"]
    with pytest.raises(WeightError):
        match_tensors(named_params_of_spec(spec2), tensors, source="test")


def test_plain_embedding_rows():
    table, pair, pos = torch.arange(10.0)[:, None] * 100, torch.arange(8.0)[:, None], torch.arange(5.0)[:, None] * 0.01
    x = P.embed([3, 4, 9], table.double(), pair.double(), pos.double(), 7, 5, 2)
    assert x[:, 0].tolist() == pytest.approx([300 + 7, 400 + (3 * 5 + 4 * 2) % 7 + 0.01, 900 + (4 * 5 + 9 * 2) % 7 + 0.02])


def test_plain_delta_rule_by_hand():
    """One channel: S_1 = k v; S_2 = w S_1 - a u (u S_1) + k v with u = k / sqrt(k^2 + 1e-6)."""
    r, k, v = torch.tensor([[1.0], [2.0]]), torch.tensor([[3.0], [0.5]]), torch.tensor([[2.0], [-1.0]])
    w, a = torch.tensor([[0.9], [0.8]]), torch.tensor([[0.3], [0.25]])
    o = P.delta_rule(r.double(), k.double(), v.double(), w.double(), a.double())
    s1 = 6.0
    u2 = 0.5 / math.sqrt(0.25 + 1e-6)
    s2 = 0.8 * s1 - 0.25 * u2 * u2 * s1 + 0.5 * -1.0
    assert o[:, 0].tolist() == pytest.approx([s1, 2 * s2])


def test_plain_gated_recurrence_by_hand():
    q, f, v = torch.tensor([[1.0], [1.0]]), torch.tensor([[0.5], [0.25]]), torch.tensor([[4.0], [8.0]])
    o = P.gated_recurrence(q.double(), f.double(), v.double())
    assert o[:, 0].tolist() == pytest.approx([2.0, 0.25 * 2.0 + 0.75 * 8.0])


def test_plain_routing_weights_the_input():
    h = torch.tensor([[1.0, -2.0]], dtype=torch.float64)
    W = {"router": torch.tensor([[0.0, 0.0], [1.0, 0.0]], dtype=torch.float64)}
    for e in range(2):
        W[f"e{e}.gate"] = W[f"e{e}.up"] = torch.eye(2, dtype=torch.float64) * (e + 1)
        W[f"e{e}.down"] = torch.eye(2, dtype=torch.float64)
    idx, val = P.route(h, W["router"], 1)
    assert idx.tolist() == [[1]] and float(val) == pytest.approx(1 / (1 + math.exp(-1)))
    x = float(val) * h[0] * 2
    assert P.moe_ff(h, W, "", {"router": {"top": 1}})[0].tolist() == pytest.approx((P.silu(x) * x).tolist())
