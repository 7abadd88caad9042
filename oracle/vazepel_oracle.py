"""Plain float64 statement of the Vazepel decoder's mechanisms, one function per mechanism, written from the equations and
sharing no code with vyomai_b200: layer norm with weight and bias, interleaved partial rotation, grouped-query attention
with biased projections, tanh-capped scores, a head-mixing matrix applied to the scores before the softmax, a softmax with
one extra unit in its denominator, a per-channel sigmoid output gate, the tanh-GELU feed-forward, the softmax-routed mixture
of clamped gated experts with group-limited choice and a shared expert, sigmoid-gated parallel sublayers and the weighted
average over all earlier layer results. Every function takes a WHOLE sequence from position 0 (time along dim 0); the tests
compare the CUDA path (whole prompts, portions, single-token decoding, mixed batches) against these.

Notation: T tokens, W model width, H query heads, G key/value heads, d query/key size per head, dv value size per head,
E experts, k experts per token.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F64 = torch.float64


def layer_norm(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor, eps: float) -> torch.Tensor:
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w + b


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rotate_pairs(x: torch.Tensor, base: float, dims: int, pos0: int = 0) -> torch.Tensor:
    """x [T, heads, n]: entries (2i, 2i + 1), i < dims / 2, of the last axis turn by the angle p * base^(-2i / dims) at position
    p = pos0 + t; entries from `dims` on pass."""
    T = x.shape[0]
    out = x.clone()
    for t in range(T):
        p = float(pos0 + t)
        for i in range(dims // 2):
            a = p * base ** (-2.0 * i / dims)
            c, s = math.cos(a), math.sin(a)
            u, v = x[t, :, 2 * i], x[t, :, 2 * i + 1]
            out[t, :, 2 * i] = u * c - v * s
            out[t, :, 2 * i + 1] = v * c + u * s
    return out


def capped(s: torch.Tensor, cap: float) -> torch.Tensor:
    return cap * torch.tanh(s / cap)


def mix_heads(s: torch.Tensor, talk: torch.Tensor) -> torch.Tensor:
    """s [H, T, T]: head a's new scores are sum_b talk[a, b] * s[b]."""
    return torch.einsum("ab,bij->aij", talk, s)


def plus_one_softmax(s: torch.Tensor, visible: torch.Tensor) -> torch.Tensor:
    """s [H, T, T], visible [T, T] bool -> weights exp(s_j) / (1 + sum over visible j of exp(s_j))."""
    s = s.masked_fill(~visible[None], float("-inf"))
    m = torch.clamp(s.max(-1, keepdim=True).values, min=0.0)
    e = torch.exp(s - m)
    return e / (torch.exp(-m) + e.sum(-1, keepdim=True))


def attention(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict) -> torch.Tensor:
    """h [T, W] -> [T, W]."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w["q"].T + w["q.b"]).view(T, H, d)
    k = (h @ w["k"].T + w["k.b"]).view(T, G, d)
    v = (h @ w["v"].T + w["v.b"]).view(T, G, dv)
    q = rotate_pairs(q, m["rot"]["base"], m["rot"]["dims"])
    k = rotate_pairs(k, m["rot"]["base"], m["rot"]["dims"])
    per = H // G
    s = torch.stack([q[:, a] @ k[:, a // per].T for a in range(H)]) * m["scale"]   # [H, T, T]
    s = mix_heads(capped(s, m["softcap"]), w["talk"])
    causal = torch.arange(T)[:, None] >= torch.arange(T)[None, :]
    p = plus_one_softmax(s, causal)
    o = torch.stack([p[a] @ v[:, a // per] for a in range(H)], 1).reshape(T, H * dv)
    o = o * torch.sigmoid(h @ w["g"].T)
    return o @ w["o"].T + w["o.b"]


def dense_ff(h: torch.Tensor, w: Dict[str, torch.Tensor]) -> torch.Tensor:
    return gelu_tanh(h @ w["up"].T) @ w["down"].T


def expert(h: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor, limit: float) -> torch.Tensor:
    g = torch.clamp(h @ gate.T, max=limit)
    u = torch.clamp(h @ up.T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ down.T


def route(z: torch.Tensor, top: int, groups: int, keep: int):
    """z [T, E] router logits -> (chosen [T, top] indices, their weights [T, top]): softmax scores over all experts; a group of
    E / groups neighbours scores as its best member, only members of the `keep` best groups are eligible; the weights are the
    chosen scores themselves."""
    T, E = z.shape
    s = torch.softmax(z, -1)
    per = E // groups
    gs = s.view(T, groups, per).max(-1).values
    kept = gs.topk(keep, -1).indices                                  # [T, keep]
    ok = torch.zeros(T, groups, dtype=torch.bool)
    ok.scatter_(1, kept, True)
    ok = ok[:, :, None].expand(T, groups, per).reshape(T, E)
    idx = s.masked_fill(~ok, -1.0).topk(top, -1).indices
    return idx, s.gather(1, idx)


def moe_ff(h: torch.Tensor, w: Dict[str, torch.Tensor], f: dict) -> torch.Tensor:
    r = f["router"]
    E = r["experts"]
    g = r.get("groups") or {"count": 1, "keep": 1}
    idx, wt = route(h @ w["router"].T, r["top"], g["count"], g["keep"])
    out = torch.zeros(h.shape[0], w["e0.down"].shape[0], dtype=h.dtype)
    for e in range(E):
        y = expert(h, w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"], f["expert"]["limit"])
        out = out + y * (wt * (idx == e)).sum(-1, keepdim=True)
    if f.get("shared"):
        out = out + expert(h, w["shared.gate"], w["shared.up"], w["shared.down"], f["shared"]["limit"])
    return out


def sub(w: Dict[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v for k, v in w.items() if k.startswith(prefix)}


def layer(stack: List[torch.Tensor], x: torch.Tensor, i: int, spec: dict, w: Dict[str, torch.Tensor], eps: float) -> torch.Tensor:
    """x: what layer i reads; stack: X_0 .. X_i (the embedding output and the earlier layers' own results). Appends X_(i+1) and
    returns the weighted average over the stack that the next layer reads."""
    p = f"l{i}."
    h = layer_norm(x, w[p + "norm1"], w[p + "norm1.b"], eps)
    y = attention(h, sub(w, p + "mix."), spec["mixer"]) * torch.sigmoid(h @ w[p + "rg1"].T + w[p + "rg1.b"])
    f = spec.get("mlp")
    if f:
        z = dense_ff(h, sub(w, p + "mlp.")) if f["kind"] == "dense" else moe_ff(h, sub(w, p + "mlp."), f)
        y = y + z * torch.sigmoid(h @ w[p + "rg2"].T + w[p + "rg2.b"])
    stack.append(x + y)
    return sum(w[p + "dwa"][j] * X for j, X in enumerate(stack))


def forward(tokens: List[int], w: Dict[str, torch.Tensor], cfg: dict, residuals: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of a whole sequence; `residuals` collects what every layer hands on."""
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.tensor(tokens, dtype=torch.long)]
    stack = [x]
    for i, spec in enumerate(cfg["layers"]):
        x = layer(stack, x, i, spec, w, eps)
        if residuals is not None:
            residuals.append(x)
    return layer_norm(x, w["final.norm"], w["final.norm.b"], eps) @ w["head"].T
