"""Plain float64 statement of the Fubinex decoder's mechanisms, one function per mechanism, written from the equations and
sharing no code with vyomai_b200: grouped RMS norm, the two rotation layouts and the stretched frequencies, latent attention
with a query latent and latent sharing between layers, block-local ("chunked") grouped-query attention with weightless RMS
division of q and k, gated linear attention with a per-channel decay, retention with a fixed decay per head, and the
polynomial feed-forward activation. Every function takes a WHOLE sequence from position 0 (time along dim 0); the tests
compare the CUDA path (whole prompts, portions, single-token decoding, mixed batches) against these.

Notation: T tokens, H heads, G key / value heads, d / dv query-key / value sizes per head, R latent size.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Tuple

import torch

F64 = torch.float64


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def grouped_norm(x: torch.Tensor, w: torch.Tensor, groups: int, eps: float) -> torch.Tensor:
    """x [T, W]: W is cut into `groups` consecutive parts, each divided by its own root mean square; w covers all of W."""
    T, W = x.shape
    return rms(x.reshape(T, groups, W // groups), eps).reshape(T, W) * w


def frequencies(rot: dict) -> Tuple[torch.Tensor, float]:
    """(f [dims / 2], factor on cos and sin). Unscaled: f_i = base^(-2i / dims), factor 1. With rot["scaling"] the slow
    frequencies are divided by `factor` behind a linear ramp over the pair index, and the factor grows with ln(factor)."""
    dims, base = int(rot["dims"]), float(rot["base"])
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F64)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, orig = float(sc["factor"]), float(sc["original"])

    def index_of(turns: float) -> float:   # the (fractional) pair index whose wavelength makes `turns` turns over the original length
        return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(index_of(float(sc["fast"]))), 0)
    hi = min(math.ceil(index_of(float(sc["slow"]))), dims - 1)
    ramp = ((torch.arange(half, dtype=F64) - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(x: torch.Tensor, rot: dict, layout: str, pos0: int = 0) -> torch.Tensor:
    """x [T, ..., n]: the first rot["dims"] entries of the last axis turn by position p = pos0 + t; the others pass. layout "half"
    pairs entry i with entry i + dims / 2, "pairs" entry 2i with 2i + 1; the pair (u, v) becomes (u c - v s, v c + u s)."""
    T, dims = x.shape[0], int(rot["dims"])
    half = dims // 2
    f, m = frequencies(rot)
    a = (torch.arange(T, dtype=F64) + pos0)[:, None] * f[None, :]
    shape = [T] + [1] * (x.dim() - 2) + [half]
    c, s = (torch.cos(a) * m).view(shape), (torch.sin(a) * m).view(shape)
    out = x.clone()
    if layout == "half":
        u, v = x[..., :half], x[..., half:dims]
        out[..., :half] = u * c - v * s
        out[..., half:dims] = v * c + u * s
    else:
        u, v = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2] = u * c - v * s
        out[..., 1:dims:2] = v * c + u * s
    return out


def causal_mask(T: int) -> torch.Tensor:
    i = torch.arange(T)
    return i[:, None] >= i[None, :]


def chunk_mask(T: int, size: int) -> torch.Tensor:
    """[T, T] bool: query i sees key j iff j <= i and both lie in the same block of `size` positions counted from 0."""
    i = torch.arange(T)
    return (i[:, None] >= i[None, :]) & ((i[:, None] // size) == (i[None, :] // size))


def softmax_attention(scores: torch.Tensor, values: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
    """scores [H, T, T] (already scaled), values [H, T, dv], mask [T, T]."""
    return torch.softmax(scores.masked_fill(~mask[None], float("-inf")), -1) @ values


def latent_kv(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float):
    """What a layer with a down-projection caches: the latent c [T, R] (RMS-normed, plain weight) and the rotated key part kr [T, dr]
    that all heads share."""
    R = m["kv_rank"]
    d = h @ w["dkv"].T
    return rms(d[:, :R], eps) * w["dkv.norm"], rotate(d[:, R:], m["rot"], "pairs")


def latent_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, c: torch.Tensor, kr: torch.Tensor, eps: float) -> torch.Tensor:
    """h [T, W] -> [T, W]: this layer's queries (through their own normed latent) against keys / values expanded from (c, kr)."""
    T = h.shape[0]
    H, dn, dr, dv = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    cq = rms(h @ w["dq"].T, eps) * w["dq.norm"]
    q = (cq @ w["uq"].T).view(T, H, dn + dr)
    qn, qr = q[..., :dn], rotate(q[..., dn:], m["rot"], "pairs")
    kn = (c @ w["uk"].T).view(T, H, dn)
    v = (c @ w["uv"].T).view(T, H, dv)
    s = (torch.einsum("thd,jhd->htj", qn, kn) + torch.einsum("thd,jd->htj", qr, kr)) * m["scale"]
    o = softmax_attention(s, v.transpose(0, 1), causal_mask(T))            # [H, T, dv]
    return o.transpose(0, 1).reshape(T, H * dv) @ w["o"].T


def chunked_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float) -> torch.Tensor:
    """Grouped-query attention inside blocks of mask.size positions; q and k are rotated (half layout), then divided by their root
    mean square per head."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rms(rotate((h @ w["q"].T).view(T, H, d), m["rot"], "half"), eps)
    k = rms(rotate((h @ w["k"].T).view(T, G, d), m["rot"], "half"), eps)
    v = (h @ w["v"].T).view(T, G, dv)
    rep = H // G
    k, v = k.repeat_interleave(rep, 1), v.repeat_interleave(rep, 1)        # query head a reads key / value head a // rep
    s = torch.einsum("thd,jhd->htj", q, k) * m["scale"]
    o = softmax_attention(s, v.transpose(0, 1), chunk_mask(T, m["mask"]["size"]))
    return o.transpose(0, 1).reshape(T, H * dv) @ w["o"].T


def decayed_recurrence(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay: torch.Tensor) -> torch.Tensor:
    """q, k [T, H, d], v [T, H, dv], decay [T, H, d] (per key channel) -> o [T, H, dv]: S_t = diag(decay_t) S_(t-1) + k_t v_t^T,
    o_t = S_t^T q_t, S_0 = 0, token by token."""
    T, H, d = q.shape
    S = torch.zeros(H, d, v.shape[-1], dtype=F64)
    out = []
    for t in range(T):
        S = decay[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        out.append(torch.einsum("hdv,hd->hv", S, q[t]))
    return torch.stack(out)


def gated_linear_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = (h @ w["q"].T).view(T, H, d) * d ** -0.5
    k = (h @ w["k"].T).view(T, H, d)
    v = (h @ w["v"].T).view(T, H, dv)
    z = (h @ w["a1"].T) @ w["a2"].T + w["a2.b"]
    alpha = (torch.sigmoid(z) ** (1.0 / m["tau"])).view(T, H, d)
    o = rms(decayed_recurrence(q, k, v, alpha), eps) * w["norm"]           # per head, one weight [dv] for all heads
    return (o.reshape(T, H * dv) * torch.nn.functional.silu(h @ w["g"].T)) @ w["o"].T


def retention(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = rotate((h @ w["q"].T).view(T, H, d), m["rot"], "half")
    k = rotate((h @ w["k"].T).view(T, H, d), m["rot"], "half") * d ** -0.5
    v = (h @ w["v"].T).view(T, H, dv)
    decay = torch.tensor(m["decay"], dtype=F64)[None, :, None].expand(T, H, d)
    o = rms(decayed_recurrence(q, k, v, decay), eps)                       # per head, no weight
    return (o.reshape(T, H * dv) * torch.nn.functional.silu(h @ w["g"].T)) @ w["o"].T


def poly_norm(z: torch.Tensor, coef, eps: float) -> torch.Tensor:
    a, b, c, e = (float(x) for x in coef)
    return a * rms(z, eps) + b * rms(z * z, eps) + c * rms(z * z * z, eps) + e


def feed_forward(h: torch.Tensor, w: Dict[str, torch.Tensor], eps: float) -> torch.Tensor:
    return poly_norm(h @ w["up"].T, w["act"].tolist(), eps) @ w["down"].T


def sub(weights: Dict[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}


def forward(cfg: dict, weights: Dict[str, torch.Tensor], tokens: List[int], residuals: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of a whole sequence; `residuals` collects the stream after every layer."""
    eps, groups = cfg["norm"]["eps"], cfg["norm"].get("groups", 1)
    x = weights["embed"][torch.tensor(tokens)] * cfg.get("embedding", {}).get("scale", 1.0)
    cached = {}
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        h = grouped_norm(x, weights[p + "norm1"], groups, eps)
        if L["type"] == "latent_attention":
            w = sub(weights, p + "mix.")
            j = m.get("kv_from")
            if j is None:
                cached[i] = latent_kv(h, w, m, eps)
            c, kr = cached[i if j is None else j]
            y = latent_attention(h, w, m, c, kr, eps)
        elif L["type"] == "parallel":
            y = m["left_scale"] * chunked_attention(h, sub(weights, p + "mix.left."), m["left"], eps) \
                + m["right_scale"] * gated_linear_attention(h, sub(weights, p + "mix.right."), m["right"], eps)
        elif L["type"] == "retention":
            y = retention(h, sub(weights, p + "mix."), m, eps)
        else:
            raise ValueError(L["type"])
        x = x + y
        if L.get("mlp"):
            x = x + feed_forward(grouped_norm(x, weights[p + "norm2"], groups, eps), sub(weights, p + "mlp."), eps)
        if residuals is not None:
            residuals.append(x.clone())
    return grouped_norm(x, weights["final.norm"], groups, eps) @ weights["head"].T
