"""Nizedra without a GPU: configuration, plan, what every run keeps, the distance buckets, and the oracle's parts by hand."""

from __future__ import annotations

import math

import numpy as np
import pytest

import nizedra_util as nu
import plain_nizedra as pn


def test_configuration_round_trip_and_errors():
    from acvram_b200.config import ConfigError, NizedraConfig, family_of
    for which in "ABCD":
        raw = nu.clean(nu.config(which))
        cfg = NizedraConfig.from_dict(raw)
        assert family_of(raw).name == "Nizedra"
        assert NizedraConfig.from_dict(cfg.to_dict()) == cfg
        assert cfg.vocab_size == raw["vocab"] and cfg.hidden_size == raw["width"]
    raw = nu.clean(nu.config("A"))
    for change, word in (
            (lambda c: c["layers"][0].__setitem__("type", "conv"), "mixers built"),
            (lambda c: c["layers"][0]["mixer"].__setitem__("kv_heads", 3), "multiple"),
            (lambda c: c["layers"][1]["mixer"].__setitem__("decay", [0.5]), "decay"),
            (lambda c: c["layers"][2]["mixer"]["rot"].__setitem__("dims", 5), "even"),
            (lambda c: c["layers"][2]["mixer"]["rot"].__setitem__("dims", 10), "at most"),
            (lambda c: c["layers"][0]["mlp"].__setitem__("kind", "moe"), "dense"),
            (lambda c: c["loop"].__setitem__("stop", 9), "stretch")):
        bad = nu.clean(raw)
        change(bad)
        with pytest.raises(ConfigError, match=word):
            NizedraConfig.from_dict(bad)


def test_plan_schedule_and_what_every_run_keeps():
    from acvram_b200.cache.manager import PagedNeed, StateNeed
    from acvram_b200.config import NizedraConfig
    from acvram_b200.models import needs_of_plan
    from acvram_b200.models.decoder import DecoderModel
    from acvram_b200.models.nizedra import nizedra_plan
    raw = nu.clean(nu.config("A"))
    plan = nizedra_plan(NizedraConfig.from_dict(raw))
    # layers 0 and 1 three times, then 2 and 3; every run has a slot of its own; a pass begins with the mix
    assert [(e.layer, e.stream_mix is not None) for e in plan.schedule] == \
        [(l, m) for l, m in pn.run_order(raw)]
    assert [e.cache for e in plan.schedule] == list(range(8))
    assert plan.residual_dtype == "float32" and plan.stream_matrices == {"loop.in": (96, 192)}
    model = DecoderModel(plan)
    needs = model.cache_plan().needs
    assert needs[0] == PagedNeed(2, 16, 0, 24) and needs[0].keeps_all
    assert needs[1] == StateNeed((3, 8, 16), "float32")
    assert needs[6] == PagedNeed(1, 40, 20, 32, 0, 0, True) and not needs[6].keeps_all      # the kept row alone, under the window
    assert needs[6].first_needed(100) == 81
    names = needs_of_plan(plan)
    assert names["l0.mix.rel"].shape == (-1, 4) and names["l0.mix.rel"].fits((12, 4)) and not names["l0.mix.rel"].fits((12, 3))
    assert "l1.norm2" not in names and "l1.mlp.up" not in names and "l1.norm1b" in names      # a layer without feed-forward
    # no loop: no matrix, no mix
    plan_b = nizedra_plan(NizedraConfig.from_dict(nu.clean(nu.config("B"))))
    assert not plan_b.stream_matrices and all(e.stream_mix is None for e in plan_b.schedule)
    assert "loop.in" not in needs_of_plan(plan_b)


@pytest.mark.parametrize("rows,far", [(16, 240.0), (12, 100.0), (2, 64.0), (6, 17.0), (32, 300.0), (8, 24.0), (4, 1000.0)])
def test_distance_buckets_are_the_oracles(rows, far):
    from acvram_b200.kernels.ops import distance_buckets
    table, last = distance_buckets(rows, far)
    table = table.tolist()
    assert last == rows - 1
    for n in range(0, int(far) + 50):
        assert (table[n] if n < len(table) else last) == pn.distance_bucket(n, rows, far), n
    assert pn.distance_bucket(10 ** 6, rows, far) == last
    assert len(table) <= math.ceil(far) + 1 and all(a <= b for a, b in zip(table, table[1:]))


def test_the_oracles_parts_by_hand():
    # the activation: continuous at 0 with slope 1/2 on both sides; its two branches
    z = np.array([-1e-7, 0.0, 1e-7])
    y = pn.xielu(z, 0.3, -0.2)
    assert abs(y[1]) == 0.0 and np.allclose(np.diff(y) / 1e-7, 0.5, atol=1e-5)
    sp = lambda v: math.log1p(math.exp(v))
    assert math.isclose(float(pn.xielu(np.array(2.0), 0.3, -0.2)), sp(0.3) * 4 + 1.0)
    assert math.isclose(float(pn.xielu(np.array(-2.0), 0.3, -0.2)), (0.5 + sp(-0.2)) * (math.exp(-2.0) + 1.0) - 1.0)
    # the recurrence as the sum it unrolls to
    rng = np.random.default_rng(0)
    T, W = 9, 8
    m = {"heads": 1, "dim": 4, "vdim": 3, "decay": [0.8]}
    w = {"q": rng.normal(size=(4, W)), "k": rng.normal(size=(4, W)), "v": rng.normal(size=(3, W)), "g": rng.normal(size=(3, W)),
         "o": np.eye(3), "norm": np.ones(3)}
    h = rng.normal(size=(T, W))
    q, k, v = pn.silu(h @ w["q"].T), pn.silu(h @ w["k"].T), pn.silu(h @ w["v"].T)
    o = np.stack([sum(0.8 ** (t - j) * (q[t] @ k[j]) * v[j] for j in range(t + 1)) for t in range(T)])
    want = pn.rms_norm(o, 1e-6) * pn.sigmoid(h @ w["g"].T)
    assert np.allclose(pn.lightning(h, w, "", m, 1e-6), want)
    # the rotation keeps lengths, leaves the elements behind `dims` alone, and turns pair i by p f_i
    x = rng.normal(size=(5, 2, 6))
    r = pn.rotate_interleaved(x, [0, 1, 2, 3, 40], 4, 100.0)
    assert np.allclose(r[0], x[0]) and np.allclose(r[..., 4:], x[..., 4:])
    assert np.allclose((r[..., :4] ** 2).sum(-1), (x[..., :4] ** 2).sum(-1))
    a = 40 * 100.0 ** (-2.0 / 4)
    assert np.allclose(r[4, 1, 2], x[4, 1, 2] * math.cos(a) - x[4, 1, 3] * math.sin(a))
    assert np.allclose(r[4, 1, 3], x[4, 1, 3] * math.cos(a) + x[4, 1, 2] * math.sin(a))
    # buckets: single distances first, then the logarithm's spread, the last row from `far` on at the latest
    assert [pn.distance_bucket(n, 8, 24.0) for n in (0, 3, 4, 5, 6, 9, 10, 15, 16, 24, 999)] == [0, 3, 4, 4, 4, 5, 6, 6, 7, 7, 7]


def test_pages_of_a_window_over_kept_rows_are_given_back():
    from acvram_b200.cache.manager import CacheManager, CachePlan, PagedNeed, StateNeed
    plan = CachePlan([PagedNeed(1, 40, 20, 32, 0, 0, True), PagedNeed(2, 16, 0, 24), StateNeed((3, 8, 16), "float32")])
    m = CacheManager(plan, 8, 40, 2)
    m.admit("a")
    held = []
    for n in range(1, 120):
        m.grow("a", n)
        m.advance("a", n)
        m.trim("a")
        held.append([len([p for p in g.tables["a"] if p >= 0]) for g in m.paged_groups])
    m.check()
    windowed = max(h[0] for h in held[40:]) if len(held[0]) > 1 else None
    by_need = {g.need.window: i for i, g in enumerate(m.paged_groups)}
    assert max(h[by_need[20]] for h in held) <= 4          # a window of 20 in pages of 8: at most 4 pages at a time
    assert held[-1][by_need[0]] == 15                      # all keys: every page of 119 tokens
    m.release("a")
    m.check()
    assert all(g.pool.num_free == 40 for g in m.paged_groups) and windowed is not None
