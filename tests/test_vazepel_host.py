"""Host-side pieces of the Vazepel family that need no GPU: the configuration's checks and tensor list, the registry, and the
oracle's own mechanisms against brute-force loops."""
import math

import pytest
import torch

from oracle import vazepel_oracle as O
from tests import vazepel_util as U


def test_config_lists_the_tensors_of_every_layer_kind():
    from vyomai_b200 import VazepelConfig
    shapes = VazepelConfig(U.small_config()).tensor_shapes()
    assert shapes["l0.mix.q"] == (6 * 10, 40) and shapes["l0.mix.k"] == (3 * 10, 40) and shapes["l0.mix.v.b"] == (3 * 7,)
    assert shapes["l0.mix.talk"] == (6, 6) and shapes["l0.mix.g"] == (6 * 7, 40) and shapes["l0.mix.o.b"] == (40,)
    assert shapes["l0.dwa"] == (2,) and shapes["l4.dwa"] == (6,)
    assert "l2.rg2" not in shapes and "l2.mlp.up" not in shapes and shapes["l2.rg1"] == (40, 40)
    assert shapes["l1.mlp.e5.gate"] == (12, 40) and shapes["l1.mlp.shared.down"] == (40, 20) and "l3.mlp.shared.up" not in shapes
    assert shapes["l3.mlp.router"] == (4, 40) and shapes["final.norm.b"] == (40,)


@pytest.mark.parametrize("bad", ["heads", "kind", "type"])
def test_config_rejects_what_the_design_does_not_have(bad):
    from vyomai_b200 import VazepelConfig
    d = U.small_config()
    if bad == "heads":
        d["layers"][0]["mixer"]["kv_heads"] = 4
    elif bad == "kind":
        d["layers"][0]["mlp"]["kind"] = "gated"
    else:
        d["layers"][0]["type"] = "lightning"
    with pytest.raises(ValueError):
        VazepelConfig(d)


def test_registry_knows_the_architecture():
    from vyomai_b200.registry import architectures
    assert "Vazepel" in architectures()


def test_random_weights_cover_the_tensor_list():
    from vyomai_b200 import VazepelConfig, VazepelForCausalLM
    cfg = VazepelConfig(U.small_config())
    w = VazepelForCausalLM.random_weights(cfg, seed=1)
    assert {k: tuple(v.shape) for k, v in w.items()} == cfg.tensor_shapes()


def test_oracle_route_against_a_loop():
    g = torch.Generator().manual_seed(0)
    z = torch.randn(50, 12, generator=g, dtype=torch.float64)
    idx, wt = O.route(z, top=3, groups=4, keep=2)
    for t in range(50):
        s = [math.exp(v) for v in z[t].tolist()]
        s = [v / sum(s) for v in s]
        gs = [max(s[3 * a:3 * a + 3]) for a in range(4)]
        kept = sorted(range(4), key=lambda a: -gs[a])[:2]
        ok = [e for e in range(12) if e // 3 in kept]
        best = sorted(ok, key=lambda e: -s[e])[:3]
        assert sorted(best) == sorted(idx[t].tolist())
        for e, w in zip(idx[t].tolist(), wt[t].tolist()):
            assert abs(w - s[e]) < 1e-12


def test_oracle_softmax_has_one_more_unit_below():
    s = torch.tensor([[[0.5, -1.0, 2.0]]], dtype=torch.float64)
    p = O.plus_one_softmax(s, torch.ones(1, 3, dtype=torch.bool))
    e = [math.exp(0.5), math.exp(-1.0), math.exp(2.0)]
    assert abs(float(p.sum()) - sum(e) / (1 + sum(e))) < 1e-12
    alone = O.plus_one_softmax(torch.tensor([[[-30.0]]], dtype=torch.float64), torch.ones(1, 1, dtype=torch.bool))
    assert float(alone) < 1e-12   # a token that sees only itself may still attend to (almost) nothing


def test_oracle_rotation_turns_pairs_and_keeps_the_rest():
    x = torch.zeros(3, 1, 6, dtype=torch.float64)
    x[:, 0, 0] = 1.0
    x[:, 0, 5] = 2.0
    y = O.rotate_pairs(x, base=9.0, dims=4, pos0=5)
    for t in range(3):
        assert abs(float(y[t, 0, 0]) - math.cos(5 + t)) < 1e-12 and abs(float(y[t, 0, 1]) - math.sin(5 + t)) < 1e-12
        assert float(y[t, 0, 5]) == 2.0 and float(y[t, 0, 4]) == 0.0


def test_oracle_expert_clamps_before_the_product():
    h = torch.eye(2, dtype=torch.float64)
    gate = torch.tensor([[5.0, -5.0]], dtype=torch.float64)
    up = torch.tensor([[9.0, -9.0]], dtype=torch.float64)
    down = torch.ones(1, 1, dtype=torch.float64)
    y = O.expert(h, gate, up, down, limit=2.0)
    assert abs(float(y[0]) - 2.0 / (1 + math.exp(-1.702 * 2.0)) * 3.0) < 1e-12        # gate capped above at 2, up at 2
    assert abs(float(y[1]) - (-5.0) / (1 + math.exp(1.702 * 5.0)) * (-1.0)) < 1e-12   # gate not capped below, up at -2
