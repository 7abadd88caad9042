"""Shared pieces of the Vazepel tests: small configurations (none of them a shipped model's sizes), float64 copies of seeded
weights for the oracle, a model builder."""
from __future__ import annotations

import random
from typing import Dict, Optional

import torch


def attn(heads=6, kv_heads=3, dim=10, vdim=7, scale=0.3, softcap=4.0, base=100.0, rot_dims=None):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "softcap": softcap,
            "rot": {"base": base, "dims": dim if rot_dims is None else rot_dims}}


def dense(ff=44):
    return {"kind": "dense", "ff": ff}


def moe(experts=6, top=2, ff=12, limit=1.2, groups=(3, 2), shared_ff: Optional[int] = 20, shared_limit=0.8):
    f = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top, "groups": {"count": groups[0], "keep": groups[1]}}}
    if shared_ff:
        f["shared"] = {"ff": shared_ff, "limit": shared_limit}
    return f


def layer(mixer, mlp):
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


def config(layers, width=40, vocab=97, eps=1e-5) -> dict:
    return {"architecture": "Vazepel", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}


def small_config() -> dict:
    """Odd sizes (nothing a multiple of 4 but what must be even), partial rotation, a layer without feed-forward, experts with and
    without a shared one, every head its own key/value head, one key/value head for all."""
    return config([
        layer(attn(), dense()),
        layer(attn(heads=2, kv_heads=2, dim=6, vdim=9, scale=0.2, rot_dims=4), moe()),
        layer(attn(heads=5, kv_heads=1, dim=8, vdim=6, base=7.0, softcap=1.5), None),
        layer(attn(heads=4, kv_heads=2, dim=6, vdim=5, rot_dims=2), moe(experts=4, top=1, ff=9, groups=(4, 1), shared_ff=None)),
        layer(attn(heads=3, kv_heads=3, dim=12, vdim=5), moe(experts=4, top=4, ff=6, groups=(2, 2), shared_ff=5, limit=0.5, shared_limit=3.0)),
    ])


def aligned_config(width=128) -> dict:
    """Sizes the tensor-core products take (multiples of 8 and 32), for the bfloat16 path."""
    a = dict(heads=8, kv_heads=2, dim=32, vdim=24, scale=0.15, softcap=10.0, base=1000.0, rot_dims=16)
    return config([
        layer(attn(**a), dense(ff=192)),
        layer(attn(**{**a, "heads": 4, "kv_heads": 4, "vdim": 40}), moe(experts=6, top=2, ff=32, groups=(3, 2), shared_ff=64)),
        layer(attn(**a), moe(experts=4, top=3, ff=40, groups=(1, 1), shared_ff=None)),
    ], width=width, vocab=203)


def wide_config() -> dict:
    """Heads and channels beyond one 64-row block of the tiled attention: 24 heads (two blocks of rows), 72 value channels (two column
    passes), 40 heads (four blocks), and 72 heads or 136 value channels (the tiled form does not apply: every step takes the one-query
    form)."""
    return config([layer(attn(heads=24, kv_heads=4, dim=12, vdim=72, rot_dims=8), dense(ff=48)),
                   layer(attn(heads=40, kv_heads=8, dim=8, vdim=6), None),
                   layer(attn(heads=72, kv_heads=8, dim=8, vdim=6), None),
                   layer(attn(heads=16, kv_heads=8, dim=20, vdim=136, rot_dims=20), dense(ff=32))], width=48, vocab=101)


def random_config(seed: int, experts: bool = True) -> dict:
    r = random.Random(1000 + seed)
    width = r.choice([24, 40, 48, 64])
    layers = []
    for _ in range(r.randint(2, 5)):
        G = r.choice([1, 2, 3, 4])
        H = G * r.choice([1, 2, 3])
        d = r.choice([4, 6, 8, 10, 16])
        m = attn(heads=H, kv_heads=G, dim=d, vdim=r.choice([3, 5, 8, 12, 16]), scale=r.choice([0.1, 0.35, 1.0]), softcap=r.choice([0.7, 3.0, 30.0]),
                 base=r.choice([5.0, 100.0, 1e4]), rot_dims=r.choice([d, d - 2, 2]))
        kind = r.choice(["dense", "moe", "moe", None]) if experts else r.choice(["dense", "dense", None])
        if kind == "moe":
            cnt = r.choice([1, 2, 3])
            per = r.choice([1, 2, 3])
            keep = r.randint(1, cnt)
            f = moe(experts=cnt * per, top=r.randint(1, keep * per), ff=r.choice([5, 8, 12]), limit=r.choice([0.5, 1.5, 7.0]), groups=(cnt, keep),
                    shared_ff=r.choice([None, 6, 16]), shared_limit=r.choice([0.4, 2.0]))
        else:
            f = dense(ff=r.choice([16, 40])) if kind else None
        layers.append(layer(m, f))
    return config(layers, width=width, vocab=r.choice([61, 97, 128]))


def f64(weights: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    return {k: v.double() for k, v in weights.items()}


def build(cfg_dict: dict, dtype=torch.float32, seed=0, weights=None, **kw):
    """(model on the GPU, float64 weights)."""
    from vyomai_b200 import VazepelConfig, VazepelForCausalLM
    cfg = VazepelConfig(cfg_dict)
    w = weights if weights is not None else VazepelForCausalLM.random_weights(cfg, seed=seed)
    kw.setdefault("sorted_min_rows", 8)   # both forms of the experts' sum come up at test sizes
    kw.setdefault("force_sorted", True)
    return VazepelForCausalLM(cfg, w, dtype=dtype, device="cuda", **kw), f64(w)
