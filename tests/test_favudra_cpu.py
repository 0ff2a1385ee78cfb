"""Favudra without a device: configuration, registry, declared tensors, run order, cache needs,
the plain implementation's own properties, and the engine's host side (pages, slots, the
convolution's and the recurrence's state across steps) on the stand-in kernels."""
import json
import math

import numpy as np
import pytest
import torch

import plain_favudra as P
import replay_patterns as R
from cpu_ops import CpuOps
from favudra_configs import CONFIGS, EDGE_CONFIGS, random_weights, tokens
from bitwise_b200 import Model
from bitwise_b200.cache.manager import groups_from_needs
from bitwise_b200.config import ConfigError, FavudraConfig, architecture_of
from bitwise_b200.models.favudra import build_favudra
from bitwise_b200.parts import PagedKVNeed, SlotStateNeed

F64 = torch.float64


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_config_round_trip_and_registry(name):
    cfg = CONFIGS[name]
    raw = json.loads(json.dumps(cfg.to_json()))
    assert raw["architecture"] == "Favudra"
    arch = architecture_of(raw)
    assert arch.name == "Favudra"
    shapes = {s.name: s.shape for s in build_favudra(cfg).param_specs()}
    assert arch.config_from_json(raw).with_tensor_shapes(shapes) == cfg   # the decay's inner size is a tensor's shape


def test_config_errors():
    base = CONFIGS["a"].to_json()
    for change, word in [(lambda d: d["layers"][3]["mixer"].update(kv_from=3), "earlier"),
                         (lambda d: d["layers"][3]["mixer"].update(kv_from=2), "none of its own"),
                         (lambda d: d["layers"][3]["mixer"].update(kv_heads=1), "share"),
                         (lambda d: d["layers"][0]["mixer"]["rot"].update(dims=7), "rot.dims"),
                         (lambda d: d["layers"][0]["mixer"].update(kv_heads=3), "multiple"),
                         (lambda d: d["layers"][2]["mixer"].update(vdim=8), "vdim"),
                         (lambda d: d["layers"][1].update(type="other"), "unknown type"),
                         (lambda d: d["layers"][1]["mixer"].pop("tau"), "tau"),
                         (lambda d: d["layers"][0]["mlp"].update(kind="moe"), "dense"),
                         (lambda d: d.pop("width"), "width")]:
        d = json.loads(json.dumps(base))
        change(d)
        with pytest.raises(ConfigError, match=word):
            FavudraConfig.from_json(d)


def test_declared_tensors_run_order_and_cache_needs():
    cfg = CONFIGS["a"]
    model = build_favudra(cfg)
    names = {s.name: s.shape for s in model.param_specs()}
    assert names["embed"] == (101, 64) and names["head"] == (101, 64) and names["final.norm"] == (64,)
    assert names["l0.mix.q"] == (64, 64) and names["l0.mix.k"] == (32, 64) and names["l0.mix.v"] == (48, 64)
    assert names["l0.mix.q.conv"] == (64, 3) and names["l0.mix.v.conv"] == (48, 3) and names["l0.mix.k.norm"] == (16,)
    assert names["l0.mix.o"] == (64, 96) and names["l0.mlp.gate"] == (96, 64) and names["l0.norm2b"] == (64,)
    assert names["l1.mix.a1"] == (4, 64) and names["l1.mix.a2"] == (16, 4) and names["l1.mix.a2.b"] == (16,)
    assert names["l1.mix.norm"] == (16,) and names["l1.mix.g"] == (32, 64) and "l1.norm2" not in names
    assert names["l2.mix.k"] == (32, 64) and "l2.mix.v" not in names and "l2.mix.q.conv" not in names
    assert "l3.mix.k" not in names and "l3.mix.v.conv" not in names and names["l3.mix.q.conv"] == (64, 3)
    # layer 3 reads the pages that layer 0 owns and keeps a convolution state of its own
    runs = [(r.block, r.cache, r.owns_cache, r.state) for r in model.schedule]
    assert runs == [(0, 0, True, 1), (1, 2, True, None), (2, 3, True, None), (3, 0, False, 4), (4, 5, True, None)]
    needs = model.cache_needs()
    assert needs[0] == PagedKVNeed(2, 16, None, v_dim=24) and needs[1] == SlotStateNeed((2, 64 + 32 + 48), torch.float32)
    assert needs[2] == SlotStateNeed((2, 8, 16), torch.float32) and needs[3] == PagedKVNeed(2, 16, 20, v_dim=0)
    assert needs[4] == SlotStateNeed((2, 64), torch.float32) and needs[5] == SlotStateNeed((3, 12, 8), torch.float32)
    groups = groups_from_needs(needs)
    assert [(g.window, g.entries) for g in groups] == [(None, (0,)), (20, (3,))]
    assert model.graph_safe()


# -- the plain implementation's own properties -------------------------------------------------
def test_plain_sink_and_cap():
    g = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn(9, 2, 6, generator=g, dtype=F64) for _ in range(3))
    out = P.capped_sink_attention(q, k, v, 0.5, None)
    # position 0 sees itself and the sink: its weight is e^s / (1 + e^s)
    s = float((q[0, 0] * k[0, 0]).sum() * 0.5)
    assert torch.allclose(out[0, 0], v[0, 0] * (math.exp(s) / (1 + math.exp(s))))
    # very negative scores: everything goes to the sink, the output vanishes
    far = P.capped_sink_attention(q.abs(), -1e3 * k.abs(), v, 0.5, None)
    assert far.abs().max() < 1e-12
    # a cap bounds every score: with cap c the weights of n keys lie within e^(+-2c) of uniform
    capped = P.capped_sink_attention(1e3 * q, k, v, 0.5, 0.1)
    uniform = torch.stack([v[:i + 1, 0].sum(0) / (i + 2) for i in range(9)])
    assert (capped[:, 0] - uniform).abs().max() < 0.35 * v.abs().max()


def test_plain_window_and_distance():
    g = torch.Generator().manual_seed(1)
    q, k = torch.randn(12, 2, 4, generator=g, dtype=F64), torch.randn(12, 1, 4, generator=g, dtype=F64)
    out = P.distance_window_attention(q, k, 0.3, 3)
    k2 = k.clone()
    k2[:5] = 99.0                                # positions 7.. see keys 5.. only
    assert torch.allclose(out[7:], P.distance_window_attention(q, k2, 0.3, 3)[7:])
    assert not torch.allclose(out[6], P.distance_window_attention(q, k2, 0.3, 3)[6])
    # with zero queries the weights are softmax(-slope * distance): head 1 of 2 has slope 2^-8
    flat = P.distance_window_attention(torch.zeros_like(q), k, 0.3, None)
    w = torch.softmax(-(2.0 ** -8) * torch.arange(11, -1, -1, dtype=F64), 0)
    assert torch.allclose(flat[11, 1], (w[:, None] * k[:, 0]).sum(0))


def test_plain_convolution_and_recurrence():
    g = torch.Generator().manual_seed(2)
    u, w = torch.randn(7, 3, generator=g, dtype=F64), torch.randn(3, 4, generator=g, dtype=F64)
    y = P.causal_conv(u, w)
    assert torch.allclose(y[0], w[:, 3] * u[0]) and torch.allclose(y[5], sum(w[:, j] * u[2 + j] for j in range(4)))
    q, k, a = (torch.rand(6, 2, 3, generator=g, dtype=F64) for _ in range(3))
    v = torch.randn(6, 2, 5, generator=g, dtype=F64)
    o = P.decayed_recurrence(q, k, v, a)
    # o_t = sum_s (q_t * prod_{s < r <= t} a_r . k_s) v_s
    t = 4
    want = sum(((q[t] * torch.prod(a[s + 1:t + 1], 0) * k[s]).sum(-1, keepdim=True) * v[s]) for s in range(t + 1))
    assert torch.allclose(o[t], want)


# -- the engine's host side on the stand-in kernels ---------------------------------------------
@pytest.mark.parametrize("name", ["a", "b"] + sorted(EDGE_CONFIGS))
def test_every_cut_on_the_stand_in(name):
    cfg = CONFIGS[name] if name in CONFIGS else EDGE_CONFIGS[name]
    W = random_weights(cfg, 3)
    model = Model.from_tensors(cfg, W, dtype="float32", device="cpu", ops=CpuOps("float32"))
    reqs = {f"{name}{i}": tokens(cfg, n, i) for i, n in enumerate([37, 70, 5, 1, 18])}
    want = {rid: P.forward(cfg.to_json(), W, t).numpy() for rid, t in reqs.items()}
    for steps, pool in ((R.whole(reqs), 128), (R.tail_one_by_one(reqs, 9), 128), (R.portions(reqs, sizes=(3, 2, 11, 1)), 128),
                        (R.mixed(reqs, 192, seed=5), 192)):
        got = R.collect(steps, R.run_in_process(model, steps, pool), cfg.vocab)
        for rid in reqs:
            err = np.abs(got[rid] - want[rid]).max() / np.abs(want[rid]).max()
            assert err < 2e-4, (rid, err)
