"""Shared pieces of the Fubinex tests: small configurations (none of them a shipped model's sizes), float64 copies of seeded
weights for the oracle, an engine builder (tests/hybrid_util.py has the feeding helpers)."""
from __future__ import annotations

from typing import Dict, Optional

import torch


def latent(heads=3, dim=8, rot_dim=6, vdim=10, rank=20, q_rank=12, scale=0.3, base=100.0, kv_from: Optional[int] = None, scaling=None, rot_dims=None):
    rot = {"base": base, "dims": rot_dim if rot_dims is None else rot_dims}
    if scaling:
        rot["scaling"] = dict(scaling)
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "q_rank": q_rank, "scale": scale, "rot": rot}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


STRETCH = {"factor": 3.0, "original": 24, "fast": 8.0, "slow": 1.0}   # original length below the test sequences: every branch of the ramp comes up


def left(heads=4, kv_heads=2, dim=12, vdim=10, chunk=7, scale=0.35, base=300.0, rot_dims=6):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "mask": {"size": chunk}, "rot": {"base": base, "dims": rot_dims}}


def right(heads=3, dim=8, vdim=6, tau=4.0):
    return {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau}


def parallel(l=None, r=None, left_scale=0.7, right_scale=1.4):
    return {"left": l or left(), "right": r or right(), "left_scale": left_scale, "right_scale": right_scale}


def retention(heads=3, dim=8, vdim=10, decay=(0.6, 0.93, 0.999), base=50.0, rot_dims=4):
    return {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay), "rot": {"base": base, "dims": rot_dims}}


def dense(ff=44):
    return {"kind": "dense", "ff": ff}


def layer(kind, mixer, mlp):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


def config(layers, width=40, vocab=97, eps=1e-5, groups=2, emb_scale=1.3) -> dict:
    return {"architecture": "Fubinex", "vocab": vocab, "width": width, "embedding": {"scale": emb_scale}, "norm": {"eps": eps, "groups": groups},
            "layers": layers}


def small_config() -> dict:
    """Odd sizes throughout, every mixer, a sharing layer with its own head count that is not next to its owner, a layer without
    feed-forward, stretched and plain frequencies, rotation of part of a head and of a whole head."""
    return config([
        layer("retention", retention(), dense()),
        layer("latent_attention", latent(scaling=STRETCH), dense(ff=36)),
        layer("parallel", parallel(), None),
        layer("latent_attention", latent(heads=2, dim=6, vdim=7, scale=0.2, q_rank=9, kv_from=1, scaling=STRETCH), dense()),
        layer("parallel", parallel(left(heads=3, kv_heads=3, dim=6, vdim=9, chunk=16, rot_dims=6), right(heads=1, dim=10, vdim=12, tau=1.0), 1.0, 0.5), dense(ff=20)),
        layer("retention", retention(heads=1, dim=6, vdim=6, decay=(0.97,), rot_dims=6), dense()),
    ], groups=5)


def aligned_config(width=128) -> dict:
    """Sizes the tensor-core products take (multiples of 8 and 32), for the bfloat16 path."""
    la = dict(heads=4, dim=32, rot_dim=16, vdim=24, rank=48, q_rank=40, scale=0.15, base=10000.0, scaling={"factor": 2.0, "original": 32, "fast": 16.0, "slow": 2.0})
    return config([
        layer("latent_attention", latent(**la), dense(ff=192)),
        layer("parallel", parallel(left(heads=4, kv_heads=2, dim=32, vdim=24, chunk=24, scale=0.18, base=1000.0, rot_dims=16), right(heads=2, dim=24, vdim=32, tau=8.0)),
              dense(ff=160)),
        layer("latent_attention", latent(**{**la, "heads": 2, "vdim": 40}, kv_from=0), dense(ff=192)),
        layer("retention", retention(heads=4, dim=16, vdim=32, decay=(0.9, 0.97, 0.99, 0.999), base=1000.0, rot_dims=16), dense(ff=128)),
    ], width=width, vocab=203, groups=4)


def many_heads_config() -> dict:
    """8 and 16 query heads over one key / value row: single tokens take the heads-as-rows attention with the keys split over CTAs."""
    return config([
        layer("parallel", parallel(left(heads=8, kv_heads=1, dim=8, vdim=12, chunk=70, rot_dims=4), right()), dense(ff=48)),
        layer("latent_attention", latent(heads=8, dim=8, rot_dim=4, vdim=12, rank=20, base=50.0), dense(ff=48)),
        layer("parallel", parallel(left(heads=16, kv_heads=2, dim=8, vdim=12, chunk=33, rot_dims=8), right(heads=2)), None),
        layer("latent_attention", latent(heads=16, dim=8, rot_dim=4, vdim=12, rank=20, base=50.0, kv_from=1), dense(ff=48)),
    ], width=48, vocab=101, groups=3)


def f64(weights: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    return {k: v.double() for k, v in weights.items()}


def build(cfg_dict: dict, dtype=torch.float32, seed=0, weights=None, low_rank=5, **kw):
    """(model on the GPU, float64 weights)."""
    from vyomai_b200 import FubinexConfig, FubinexForCausalLM
    cfg = FubinexConfig(cfg_dict)
    w = weights if weights is not None else FubinexForCausalLM.random_weights(cfg, seed=seed, low_rank=low_rank)
    return FubinexForCausalLM(cfg, w, dtype=dtype, device="cuda", **kw), f64(w)


def random_config(seed: int) -> dict:
    """A configuration drawn from the design's whole space: 3-6 layers of the three mixers in any order, latent owners and sharers,
    head counts from 1 to 12, unrelated channel counts, chunks shorter and longer than the test sequences, norm groups 1-4."""
    g = torch.Generator().manual_seed(seed)
    pick = lambda xs: xs[int(torch.randint(0, len(xs), (1,), generator=g))]  # noqa: E731
    groups = pick([1, 2, 4])
    width = pick([48, 64, 96, 160])
    layers, owners = [], []
    for i in range(pick([3, 4, 5, 6])):
        kind = pick(["latent_attention", "parallel", "retention"])
        if kind == "latent_attention":
            own = not owners or pick([True, False])
            if own:
                rd = pick([2, 4, 8, 16, 32])
                geo = dict(rank=pick([12, 16, 40, 64, 96]), rot_dim=rd, base=pick([10.0, 1000.0, 250000.0]),
                           scaling=pick([None, {"factor": pick([2.0, 4.0, 8.0]), "original": pick([16, 64, 4096]), "fast": pick([4.0, 32.0]), "slow": pick([0.5, 1.0, 2.0])}]))
                owners.append((i, geo))
                src = None
            else:
                src, geo = pick(owners)
            m = latent(heads=pick([1, 2, 3, 4, 6, 8, 12]), dim=pick([4, 8, 16, 24, 32]), vdim=pick([4, 8, 20, 32, 48]), q_rank=pick([8, 24, 56]),
                       scale=pick([0.1, 0.25, 0.5]), kv_from=src, **geo)
        elif kind == "parallel":
            kvh = pick([1, 2, 3])
            d = pick([8, 16, 24, 32])
            m = parallel(left(heads=kvh * pick([1, 2, 4, 8]), kv_heads=kvh, dim=d, vdim=pick([4, 8, 20, 32]), chunk=pick([1, 3, 17, 50, 200]),
                              scale=pick([0.1, 0.25, 0.5]), base=pick([10.0, 1000.0, 250000.0]), rot_dims=pick([0, 2, d // 2, d])),
                         right(heads=pick([1, 2, 5]), dim=pick([4, 8, 16, 40]), vdim=pick([4, 8, 24]), tau=pick([1.0, 2.0, 16.0])),
                         pick([0.5, 1.0, 1.25]), pick([0.5, 1.0, 2.0]))
        else:
            h = pick([1, 2, 4, 6])
            d = pick([4, 8, 16, 32])
            m = retention(heads=h, dim=d, vdim=pick([4, 8, 16, 40]), decay=[pick([0.5, 0.9, 0.99, 0.999]) for _ in range(h)], base=pick([10.0, 10000.0]),
                          rot_dims=pick([0, 2, d]))
        layers.append(layer(kind, m, pick([None, dense(ff=pick([24, 64, 100]))])))
    return config(layers, width=width, vocab=pick([50, 131, 256]), eps=pick([1e-6, 1e-5]), groups=groups, emb_scale=pick([0.5, 1.0, 3.0]))
