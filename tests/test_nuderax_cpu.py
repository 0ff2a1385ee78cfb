"""Nuderax without a device: configuration, registry, declared tensors, cache groups, and the
plain implementation's own properties."""
import json
import math

import pytest
import torch

import plain_nuderax as P
from nuderax_configs import CONFIGS, mixer, mlp, random_weights
from bitwise_b200.cache.manager import groups_from_needs
from bitwise_b200.config import ConfigError, NuderaxConfig, NuderaxLayerConfig, architecture_of
from bitwise_b200.models.nuderax import build_nuderax
from bitwise_b200.parts import PagedLatentNeed
from bitwise_b200.weights import WeightError
from bitwise_b200.weights.loader import check_against_specs


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_config_round_trip_and_registry(name):
    cfg = CONFIGS[name]
    raw = json.loads(json.dumps(cfg.to_json()))
    assert raw["architecture"] == "Nuderax"
    arch = architecture_of(raw)
    assert arch.name == "Nuderax"
    assert arch.config_from_json(raw) == cfg


def test_config_errors():
    base = CONFIGS["a"].to_json()
    for change, word in [(lambda d: d["layers"][2]["mixer"].update(kv_from=2), "earlier"),
                         (lambda d: d["layers"][2]["mixer"].update(kv_rank=41), "share"),
                         (lambda d: d["layers"][0]["mixer"].pop("q_rank"), "q_rank"),
                         (lambda d: d["layers"][1].update(type="other"), "unknown type"),
                         (lambda d: d["layers"][1]["mlp"]["router"].update(experts=7), "equal groups"),
                         (lambda d: d["layers"][1]["mlp"]["router"].update(top=5), "choices"),
                         (lambda d: d["layers"][1]["mixer"]["rot"].update(dims=10), "rot.dims"),
                         (lambda d: d.pop("width"), "width")]:
        d = json.loads(json.dumps(base))
        change(d)
        with pytest.raises(ConfigError, match=word):
            NuderaxConfig.from_json(d)


def test_declared_tensors_and_run_order():
    cfg = CONFIGS["a"]
    model = build_nuderax(cfg)
    names = {s.name: s.shape for s in model.param_specs()}
    assert names["embed"] == (131, 72) and names["embed.norm"] == (72,) and names["final.norm"] == (72,)
    assert names["l0.mix.dq"] == (40, 72) and names["l0.mix.dq.norm"] == (40,) and names["l0.mix.uq"] == (2 * 32, 40)
    assert names["l1.mix.q"] == (5 * 24, 72) and names["l1.mix.dkv"] == (48, 72) and names["l1.mix.dkv.norm"] == (40,)
    assert "l2.mix.dkv" not in names and "l2.mix.dkv.norm" not in names and names["l2.mix.uk"] == (80, 40)
    assert names["l1.mlp.e7.down"] == (72, 20) and names["l1.mlp.router"] == (8, 72) and names["l1.mlp.correction"] == (8,)
    assert names["l0.mlp.shared.gate"] == (28, 72)
    # layer 2 reads the entry that layer 1 owns; three layers, two entries
    assert [(r.block, r.cache, r.owns_cache) for r in model.schedule] == [(0, 0, True), (1, 1, True), (2, 1, False)]
    needs = model.cache_needs()
    assert needs == [PagedLatentNeed(48, 16), PagedLatentNeed(40, 8)]
    assert [g.entries for g in groups_from_needs(needs)] == [(0, 1)]
    assert model.graph_safe()
    # a layer without feed-forward declares no second norm
    names_b = {s.name for s in build_nuderax(CONFIGS["b"]).param_specs()}
    assert "l1.norm1" in names_b and "l1.norm2" not in names_b and not any(n.startswith("l1.mlp") for n in names_b)
    assert "l0.mlp.shared.gate" not in names_b and "l2.mlp.shared.gate" in names_b


def test_weights_are_checked_against_the_declaration():
    cfg = CONFIGS["b"]
    w = random_weights(cfg, 1)
    specs = build_nuderax(cfg).param_specs()
    check_against_specs({n: tuple(t.shape) for n, t in w.items()}, specs)
    w.pop("l2.mlp.correction")
    w["l0.mix.extra"] = torch.zeros(1)
    w["l0.mix.uk"] = torch.zeros(3, 3)
    with pytest.raises(WeightError) as e:
        check_against_specs({n: tuple(t.shape) for n, t in w.items()}, specs)
    assert e.value.missing == ["l2.mlp.correction"] and e.value.unexpected == ["l0.mix.extra"]
    assert e.value.wrong_shape[0][0] == "l0.mix.uk"


def test_cache_manager_gives_latent_pages_back():
    from bitwise_b200.cache.storage import build_cache
    model = build_nuderax(CONFIGS["a"])
    manager, storage = build_cache(model, 6, 16, 2, torch.float32, "cpu")
    assert storage.k[0].shape == (7, 16, 64) and storage.k[1].shape == (7, 16, 48) and storage.v[0] is None
    manager.begin("x")
    assert manager.ensure("x", 40) and manager.available(0) == 3
    manager.begin("y")
    assert manager.ensure("y", 48) and not manager.ensure("y", 49)
    manager.release("x")
    assert manager.ensure("y", 49)
    manager.release("y")
    assert manager.all_free()
    manager.check_consistency()


# ---- the plain implementation's own properties ----------------------------------------------
def test_plain_rotation_depends_on_the_distance_only():
    g = torch.Generator().manual_seed(0)
    q, k = torch.randn(1, 12, generator=g, dtype=torch.float64), torch.randn(1, 12, generator=g, dtype=torch.float64)
    def score(pq, pk):
        return float((P.rotate_pairs(q, [pq], 50.0, 8) * P.rotate_pairs(k, [pk], 50.0, 8)).sum())
    assert abs(score(9, 4) - score(105, 100)) < 1e-9
    assert abs(score(9, 4) - score(9, 5)) > 1e-3
    # entries beyond the turned ones pass unchanged
    assert torch.equal(P.rotate_pairs(q, [7], 50.0, 8)[:, 8:], q[:, 8:])


def test_plain_route_groups_and_correction():
    # expert 5 has the largest score, but its group (4, 5) loses: the groups count by the sum of
    # their two largest corrected scores, and only experts of the two best groups can be chosen
    z = torch.tensor([[2.0, 1.9, 0.5, 0.4, -3.0, 2.5, 1.0, 1.2]], dtype=torch.float64)
    w = torch.eye(8, dtype=torch.float64)
    r = {"top": 3, "scale": 2.0, "groups": {"count": 4, "keep": 2}}
    chosen, weights = P.route(z, w, torch.zeros(8, dtype=torch.float64), r)
    assert chosen.tolist() == [[0, 1, 7]]
    assert torch.allclose(weights, 2.0 * torch.sigmoid(z[0, [0, 1, 7]]))
    # a correction moves the choice and not the weight
    corr = torch.zeros(8, dtype=torch.float64)
    corr[6] = 0.5
    chosen, weights = P.route(z, w, corr, r)
    assert chosen.tolist() == [[6, 0, 1]] and torch.allclose(weights[0, 0], 2.0 * torch.sigmoid(z[0, 6]))
    # negative corrected scores: an excluded expert never beats an eligible one
    corr = torch.full((8,), -5.0, dtype=torch.float64)
    chosen, _ = P.route(z, w, corr, r)
    assert sorted(chosen[0].tolist()) == [0, 1, 7]


def test_plain_expert_clamps():
    h = torch.tensor([[1.0]], dtype=torch.float64)
    gate, up, down = (torch.tensor([[v]], dtype=torch.float64) for v in (5.0, -7.0, 1.0))
    y = P.expert(h, gate, up, down, 2.0)       # g = min(5, 2) = 2, u = clamp(-7) = -2
    assert abs(float(y) - 2.0 / (1.0 + math.exp(-1.702 * 2.0)) * (-2.0 + 1.0)) < 1e-12
    y = P.expert(h, -gate, up, down, 2.0)      # the gate is clamped from above only
    assert abs(float(y) - (-5.0) / (1.0 + math.exp(1.702 * 5.0)) * (-1.0)) < 1e-12
