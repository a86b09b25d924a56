"""Vadelix without a GPU: configuration, plan, what every layer keeps, and the oracle's mechanisms by hand."""

from __future__ import annotations

import math

import numpy as np
import pytest

import plain_vadelix as pv
import vadelix_util as vu
from acvram_b200.cache.manager import PagedNeed, StateNeed
from acvram_b200.config import ConfigError, VadelixConfig, family_of
from acvram_b200.models import DecoderModel
from acvram_b200.models.vadelix import vadelix_plan


@pytest.mark.parametrize("which", ["A", "B", "C", "D"])
def test_configuration_round_trip(which):
    raw = vu.clean(vu.config(which))
    cfg = VadelixConfig.from_dict(raw)
    assert cfg.to_dict() == raw
    assert family_of(raw).config_cls is VadelixConfig
    assert VadelixConfig.from_dict(cfg.to_dict()) == cfg


def test_configuration_errors_name_the_key():
    def broken(change):
        raw = vu.clean(vu.config("A"))
        change(raw)
        with pytest.raises(ConfigError) as e:
            VadelixConfig.from_dict(raw)
        return str(e.value)

    assert "type" in broken(lambda c: c["layers"][0].update(type="conv"))
    assert "kv_heads" in broken(lambda c: c["layers"][1]["mixer"].update(kv_heads=3))
    assert "groups" in broken(lambda c: c["norm"].update(groups=7))
    assert "choices" in broken(lambda c: c["layers"][1]["mlp"]["router"].update(top=5))       # 2 kept groups of 2 experts
    assert "rot.dims" in broken(lambda c: c["layers"][1]["mixer"]["rot"].update(dims=18))
    assert "v_mix" in broken(lambda c: c["layers"][2]["mixer"].update(vdim=16))                # blended values of two sizes
    assert "canon" in broken(lambda c: c.pop("canon"))
    assert "kind" in broken(lambda c: c["layers"][0]["mlp"].update(kind="glu"))


def test_plan_and_what_every_layer_keeps():
    cfg = VadelixConfig.from_dict(vu.clean(vu.config("A")))
    plan = vadelix_plan(cfg)
    assert plan.residual_dtype == "float32" and [e.layer for e in plan.schedule] == [0, 1, 2, 3]
    kinds = [l.mixer.kind for l in plan.layers]
    assert kinds == ["wkv", "attention", "attention", "attention"]
    roles = [l.mixer.params.get("value_share", {}).get("role") for l in plan.layers]
    assert roles == [None, "source", "mix", "mix"]          # the first blending layer gives, the later ones take
    assert plan.layers[2].mixer.params["sink"] == 0.0 and plan.layers[2].mixer.params["slope_rate"] == 8.0
    assert plan.layers[1].mixer.params["sink"] == "sink" and plan.layers[1].mixer.params["qk_norm_scope"] == "all"
    assert all(l.options["input_conv"] == {"tensor": "canon1", "taps": 3} for l in plan.layers)
    assert plan.layers[2].feed_forward is None and plan.layers[1].feed_forward.params["groups"] == (3, 2)
    model = DecoderModel(plan)
    need = model.blocks[0].cache_need()
    assert need == {"mixer": {"state": StateNeed((3, 16, 16), "float32"), "previous": StateNeed((96,), "float32")},
                    "conv": StateNeed((2, 96), "float32")}
    need = model.blocks[2].cache_need()
    assert need["conv"] == StateNeed((2, 96), "float32") and isinstance(need["mixer"], PagedNeed)
    assert need["mixer"].window == 20 and model.blocks[1].cache_need()["mixer"].window == 0
    cplan = model.cache_plan()
    assert len(cplan.needs if hasattr(cplan, "needs") else cplan.slots) == 3 + 2 + 2 + 2      # what the four layers keep
    names = model.tensor_needs()
    assert "l1.mix.q.norm" in names and names["l1.mix.q.norm"].shape == (64,) and names["l1.mix.vmix"].optional
    assert not names["l2.mix.vmix"].optional and "l2.mix.sink" not in names and "l0.mix.w1" in names


def test_one_tap_and_one_group_are_the_plain_forms():
    x = np.random.default_rng(0).standard_normal((5, 12))
    w = np.ones(12)
    assert np.allclose(pv.grouped_norm(x, w, 1e-6, 1), x / np.sqrt((x * x).mean(-1, keepdims=True) + 1e-6))
    three = pv.grouped_norm(x, w, 0.0, 3)
    assert np.allclose((three.reshape(5, 3, 4) ** 2).mean(-1), 1.0)
    taps = np.full((12, 1), 0.5)
    assert np.allclose(pv.short_conv(x, taps), 0.5 * x)
    taps = np.zeros((12, 3))
    taps[:, 0] = 1.0                                # the oldest tap alone: the row two tokens back
    assert np.allclose(pv.short_conv(x, taps)[2:], x[:-2]) and np.allclose(pv.short_conv(x, taps)[:2], 0.0)


def test_routing_by_groups_by_hand():
    z = np.log(np.array([[0.30, 0.05, 0.10, 0.25, 0.20, 0.10]]))       # three groups of two: worth 0.30, 0.25, 0.20
    chosen, weights = pv.route(z, 2, 3, 2)
    assert chosen.tolist() == [[0, 3]] and np.allclose(weights, [[0.30 / 0.55, 0.25 / 0.55]])
    chosen, _ = pv.route(z, 2, 3, 1)                                     # one group kept: both choices from the best
    assert chosen.tolist() == [[0, 1]]
    chosen, _ = pv.route(z, 3, 1, 1)                                     # one group: the plain top three
    assert chosen.tolist() == [[0, 3, 4]]


def test_sink_and_slopes_by_hand():
    s = np.array([0.0, 0.0])
    v = np.array([[1.0], [3.0]])
    assert np.allclose(pv.sink_softmax_sum(s, [0, 1], 0.0, v), (1.0 + 3.0) / 3.0)       # the sink is a third key of score 0
    assert np.allclose(pv.sink_softmax_sum(s, [0, 1], -50.0, v), 2.0)
    assert np.allclose(pv.sink_softmax_sum(s, [1], math.log(3.0), v), 3.0 / 4.0)


def test_wkv_by_hand():
    """One head of two channels, two tokens, mixes that look at the current token only."""
    W = {"mu." + s: np.zeros(2) for s in "rkvgw"}
    eye = np.eye(2)
    W.update({"r": eye, "k": eye, "v": eye, "g": eye, "w1": np.zeros((1, 2)), "w2": np.zeros((2, 1)),
              "w0": np.full(2, math.log(math.log(2.0))), "u": np.array([[0.5, 0.5]]), "norm": np.ones(2), "o": eye})
    W = {"x." + k: v for k, v in W.items()}
    h = np.array([[1.0, 2.0], [3.0, 1.0]])
    # token 0: o = u k (v . )...: (diag(u) k v^T)^T r = v * sum_i u_i k_i r_i = [1, 2] * 2.5; token 1: S = k0 v0^T,
    # o = S^T r + v1 * sum u k r = [1, 2] * (1*3 + 2*1) + [3, 1] * 5
    o = np.array([[2.5, 5.0], [5.0 + 15.0, 10.0 + 5.0]])
    want = pv.unit_rms(o, 1e-6) * pv.silu(h)
    assert np.allclose(pv.wkv(h, W, "x.", {"heads": 1, "dim": 2}, 1e-6), want)
