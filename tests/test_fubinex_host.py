"""Host-side pieces of the Fubinex family that need no GPU: the configuration's checks and tensor list, the registry, the cache specs
of its layers (pages, state slots, a layer reading another layer's pages), and the oracle's own mechanisms against brute-force loops
and closed forms."""
import math

import pytest
import torch

from oracle import fubinex_oracle as O
from tests import fubinex_util as U


def test_config_lists_the_tensors_of_every_layer_kind():
    from vyomai_b200 import FubinexConfig
    shapes = FubinexConfig(U.small_config()).tensor_shapes()
    assert shapes["l0.mix.q"] == (3 * 8, 40) and shapes["l0.mix.g"] == (3 * 10, 40) and "l0.mix.norm" not in shapes
    assert shapes["l1.mix.dkv"] == (20 + 6, 40) and shapes["l1.mix.dq"] == (12, 40) and shapes["l1.mix.uq"] == (3 * (8 + 6), 12)
    assert "l3.mix.dkv" not in shapes and "l3.mix.dkv.norm" not in shapes and shapes["l3.mix.uq"] == (2 * (6 + 6), 9) and shapes["l3.mix.uv"] == (2 * 7, 20)
    assert shapes["l2.mix.left.k"] == (2 * 12, 40) and shapes["l2.mix.right.norm"] == (6,) and shapes["l2.mix.right.a2"] == (3 * 8, -1)
    assert "l2.norm2" not in shapes and "l2.mlp.up" not in shapes and shapes["l4.mlp.act"] == (4,)
    assert shapes["final.norm"] == (40,) and shapes["l0.norm1"] == (40,)


@pytest.mark.parametrize("bad", ["forward", "chain", "rank", "kind", "type", "groups", "decay", "not_latent", "kv_heads"])
def test_config_rejects_what_the_design_does_not_have(bad):
    from vyomai_b200 import FubinexConfig
    d = U.small_config()
    if bad == "forward":
        d["layers"][1]["mixer"]["kv_from"] = 3
    elif bad == "chain":
        d["layers"].append(U.layer("latent_attention", U.latent(kv_from=3, scaling=U.STRETCH), None))
    elif bad == "rank":
        d["layers"][3]["mixer"]["kv_rank"] = 21
    elif bad == "kind":
        d["layers"][0]["mlp"]["kind"] = "moe"
    elif bad == "type":
        d["layers"][0]["type"] = "lightning"
    elif bad == "groups":
        d["norm"]["groups"] = 3
    elif bad == "decay":
        d["layers"][0]["mixer"]["decay"] = [0.9]
    elif bad == "not_latent":
        d["layers"][3]["mixer"]["kv_from"] = 0
    else:
        d["layers"][2]["mixer"]["left"]["kv_heads"] = 3
    with pytest.raises(ValueError):
        FubinexConfig(d)


def test_registry_knows_the_architecture():
    from vyomai_b200.registry import architectures
    assert "Fubinex" in architectures()


def test_layers_declare_pages_slots_and_shared_rows():
    """Built on the CPU (no kernel runs): what each layer asks of the cache manager."""
    from vyomai_b200 import FubinexConfig, FubinexForCausalLM
    from vyomai_b200.paged import HybridCacheManager
    cfg = FubinexConfig(U.small_config())
    model = FubinexForCausalLM(cfg, FubinexForCausalLM.random_weights(cfg, low_rank=5), dtype=torch.float32, device="cpu")
    specs = model.cache_specs()
    assert specs[0] == [{"pages": None, "states": {"S": (3, 8, 10)}}]
    assert specs[1][0]["pages"] == (1, 26, 0) and specs[3][0]["pages_from"] == (1, 0) and specs[3][0]["pages"] is None
    assert specs[2][0]["pages"] == (2, 12, 10) and specs[2][1] == {"pages": None, "states": {"S": (3, 8, 6)}}
    mgr = HybridCacheManager(model, max_tokens=16, block_size=4, max_seqs=2, device="cpu")
    assert mgr.views[3][0] is mgr.views[1][0] and mgr.views[1][0].k_pool.shape[1:] == (4, 1, 26) and mgr.views[1][0].v_pool is None
    assert mgr.views[2][0].v_pool.shape[1:] == (4, 2, 10) and mgr.views[2][1].states["S"].shape == (2, 3, 8, 6)
    assert mgr.views[5][0].states["S"].shape == (2, 1, 6, 6)


def test_oracle_chunk_mask_by_enumeration():
    m = O.chunk_mask(11, 4)
    for i in range(11):
        for j in range(11):
            assert bool(m[i, j]) == (j <= i and i // 4 == j // 4)
    assert torch.equal(O.chunk_mask(6, 1), torch.eye(6, dtype=torch.bool)) and torch.equal(O.chunk_mask(6, 100), O.causal_mask(6))


@pytest.mark.parametrize("layout", ["half", "pairs"])
def test_oracle_rotation_is_relative_and_partial(layout):
    """Scores of rotated vectors depend on the distance only; entries past rot.dims pass; pair partners per layout."""
    rot = {"base": 20.0, "dims": 4}
    g = torch.Generator().manual_seed(0)
    a, b = torch.randn(1, 6, generator=g, dtype=torch.float64), torch.randn(1, 6, generator=g, dtype=torch.float64)
    s = [float((O.rotate(a, rot, layout, pos0=p + 3) * O.rotate(b, rot, layout, pos0=p)).sum()) for p in (0, 5, 40)]
    assert abs(s[0] - s[1]) < 1e-12 and abs(s[0] - s[2]) < 1e-12
    r = O.rotate(a, rot, layout, pos0=7)
    assert torch.equal(r[:, 4:], a[:, 4:])
    u, v = (0, 2) if layout == "half" else (0, 1)
    ang = 7.0
    assert abs(float(r[0, u]) - (float(a[0, u]) * math.cos(ang) - float(a[0, v]) * math.sin(ang))) < 1e-12
    assert abs(float(r[0, v]) - (float(a[0, v]) * math.cos(ang) + float(a[0, u]) * math.sin(ang))) < 1e-12


def test_oracle_recurrence_equals_the_unrolled_sum():
    g = torch.Generator().manual_seed(1)
    T, H, d, dv = 7, 2, 3, 4
    q, k, v = (torch.randn(T, H, n, generator=g, dtype=torch.float64) for n in (d, d, dv))
    decay = torch.rand(T, H, d, generator=g, dtype=torch.float64)
    got = O.decayed_recurrence(q, k, v, decay)
    for t in range(T):
        want = torch.zeros(H, dv, dtype=torch.float64)
        for j in range(t + 1):
            w = torch.ones(H, d, dtype=torch.float64)
            for s in range(j + 1, t + 1):
                w = w * decay[s]
            want += torch.einsum("hd,hv->hv", q[t] * w * k[j], v[j])
        assert float((got[t] - want).abs().max()) < 1e-12


def test_oracle_polynomial_activation_on_a_constant_row():
    """All entries c: every normalised power is sign^p (eps aside), so the result is a + b + c3 + e for c > 0 and -a + b - c3 + e for c < 0."""
    coef = (0.5, 0.25, 2.0, -1.0)
    assert float((O.poly_norm(torch.full((1, 9), 3.0, dtype=torch.float64), coef, 0.0) - 1.75).abs().max()) < 1e-12
    assert float((O.poly_norm(torch.full((1, 9), -3.0, dtype=torch.float64), coef, 0.0) + 3.25).abs().max()) < 1e-12


def test_oracle_grouped_norm_groups_are_independent():
    x = torch.randn(3, 12, generator=torch.Generator().manual_seed(2), dtype=torch.float64)
    w = torch.linspace(0.5, 1.5, 12, dtype=torch.float64)
    y = O.grouped_norm(x, w, 3, 1e-6)
    x2 = x.clone()
    x2[:, 4:8] *= 100.0
    y2 = O.grouped_norm(x2, w, 3, 1e-6)
    assert float((y[:, :4] - y2[:, :4]).abs().max()) == 0.0 and float((y[:, 8:] - y2[:, 8:]).abs().max()) == 0.0
    assert float((y[:, 4:8] - y2[:, 4:8]).abs().max()) < 1e-5   # scale-free but for eps
    assert float(((y[:, :4] / w[:4]) ** 2).mean(-1).sub(1.0).abs().max()) < 1e-5
