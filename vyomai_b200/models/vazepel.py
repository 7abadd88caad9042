"""Vazepel: a decoder-only language model of parallel layers. Layers are listed in the configuration; each norms its input once
(layer norm with weight and bias), runs its mixer and its feed-forward side by side on that normed input, multiplies each result
by a sigmoid gate that is itself a biased projection of the normed input, and adds both to the residual. What a layer hands on is
not its own result but a learned weighted sum over the embedding output and the results of all layers so far. The mixer is
grouped-query attention whose heads exchange scores before the softmax (layers/mixers.py TalkingHeadsAttention: biased
projections, pair rotation on the leading entries of each head, tanh-capped scores, head-mixing matrix, a softmax with one extra
unit in the denominator, per-channel output gate); the feed-forward is dense (tanh-GELU) or a softmax-routed mixture of clamped
gated experts with group-limited choice, unnormalised weights and a shared expert (layers/mixers.py MoEFeedForward). The reference
package has no such model; it is served by the same pieces as the other packed-step decoders here (models/gelutar.py,
models/zugunex.py): a configuration object read from config.json, weights loaded by tensor name, the cache manager's pages
(vyomai_b200/paged.py), one `step` over a packed batch that the batching engine, the CUDA-graph capture and the trace replayer all
call, and greedy selection by vy_argmax_rows.

A layer is five kinds of launches: ONE product for everything that reads the normed input (q | k | v | output gate | the two
residual gates | router logits, biases in its epilogue), rotation + page write, attention, the output projection, the feed-forward's
products, and one closing kernel that forms the gated residual, stores the layer's result in the stack of results, takes the weighted
sum over the stack and applies the NEXT layer's norm to it. The residual stream, the stack, norms, rotation angles, attention scores,
gates, router scores and weights are fp32 in both dtypes; with dtype=bfloat16 the projections read bf16 inputs on the tensor cores
(fp32 results), with dtype=float32 they are fp32 FMA.
"""
from __future__ import annotations

import json
import os
from typing import Dict, List, Optional

import torch

from .. import _lib, ops
from ..layers.mixers import DenseMLP, MoEFeedForward, Projection, TalkingHeadsAttention, pack_biases, pack_rows


class VazepelConfig:
    """config.json of the architecture: vocab, width, norm.eps and `layers`, a list of
    {"type": "attention", "mixer": {heads, kv_heads, dim, vdim, scale, softcap, rot: {base, dims}},
     "mlp": null | {"kind": "dense", "ff"} | {"kind": "moe", "expert": {"ff", "limit"}, "router": {"experts", "top", "groups": {"count", "keep"}},
                    "shared": {"ff", "limit"}?}}."""

    architecture = "Vazepel"

    def __init__(self, d: dict):
        if d.get("architecture") != self.architecture:
            raise ValueError(f"not a {self.architecture} configuration: {d.get('architecture')!r}")
        self.raw = d
        self.vocab, self.width = int(d["vocab"]), int(d["width"])
        self.eps = float(d["norm"]["eps"])
        self.layers = list(d["layers"])
        for i, L in enumerate(self.layers):
            if L["type"] != "attention":
                raise ValueError(f"layer {i}: unknown mixer type {L['type']!r}")
            m = L["mixer"]
            if int(m["heads"]) % int(m["kv_heads"]):
                raise ValueError(f"layer {i}: heads must be a multiple of kv_heads")
            f = L.get("mlp")
            if f and f.get("kind", "dense") not in ("dense", "moe"):
                raise ValueError(f"layer {i}: unknown feed-forward kind {f.get('kind')!r}")

    @classmethod
    def from_dir(cls, path: str) -> "VazepelConfig":
        with open(os.path.join(path, "config.json")) as f:
            return cls(json.load(f))

    def tensor_shapes(self) -> Dict[str, tuple]:
        """Name -> shape of every weight the configuration implies (what a checkpoint must hold; also the recipe for random
        initialisation)."""
        W = self.width
        out: Dict[str, tuple] = {"embed": (self.vocab, W), "final.norm": (W,), "final.norm.b": (W,), "head": (self.vocab, W)}
        for i, L in enumerate(self.layers):
            p, m = f"l{i}.", L["mixer"]
            H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
            out.update({p + "norm1": (W,), p + "norm1.b": (W,), p + "mix.q": (H * d, W), p + "mix.q.b": (H * d,), p + "mix.k": (G * d, W),
                        p + "mix.k.b": (G * d,), p + "mix.v": (G * dv, W), p + "mix.v.b": (G * dv,), p + "mix.talk": (H, H), p + "mix.g": (H * dv, W),
                        p + "mix.o": (W, H * dv), p + "mix.o.b": (W,), p + "rg1": (W, W), p + "rg1.b": (W,), p + "dwa": (i + 2,)})
            f = L.get("mlp")
            if not f:
                continue
            out.update({p + "rg2": (W, W), p + "rg2.b": (W,)})
            if f.get("kind", "dense") == "dense":
                out.update({p + "mlp.up": (f["ff"], W), p + "mlp.down": (W, f["ff"])})
            else:
                ff = int(f["expert"]["ff"])
                for e in range(int(f["router"]["experts"])):
                    out.update({p + f"mlp.e{e}.gate": (ff, W), p + f"mlp.e{e}.up": (ff, W), p + f"mlp.e{e}.down": (W, ff)})
                out[p + "mlp.router"] = (int(f["router"]["experts"]), W)
                if f.get("shared"):
                    sf = int(f["shared"]["ff"])
                    out.update({p + "mlp.shared.gate": (sf, W), p + "mlp.shared.up": (sf, W), p + "mlp.shared.down": (W, sf)})
        return out


class _Layer:
    def __init__(self, idx: int, spec: dict, w: Dict[str, torch.Tensor], cfg: VazepelConfig, act_dtype, tensor_cores: bool, kv_dtype,
                 sorted_min_rows: int, force_sorted: bool):
        p = f"l{idx}."
        sub = lambda pre: {k[len(pre):]: v for k, v in w.items() if k.startswith(pre)}  # noqa: E731
        self.eps, self.act_dtype = cfg.eps, act_dtype
        self.norm_w, self.norm_b = w[p + "norm1"].contiguous(), w[p + "norm1.b"].contiguous()
        self.mixer = TalkingHeadsAttention(spec["mixer"], sub(p + "mix."), cfg.eps, act_dtype, tensor_cores, kv_dtype, sink="zero")
        self.coef = w[p + "dwa"].to(torch.float32).contiguous()
        self.depth = idx + 2
        blocks = list(self.mixer.input_weights()) + [w[p + "rg1"]]
        biases = list(self.mixer.input_biases()) + [w[p + "rg1.b"]]
        self.n_mix = len(self.mixer.input_weights())
        self.mlp, self.moe = None, False
        f = spec.get("mlp")
        if f:
            blocks.append(w[p + "rg2"])
            biases.append(w[p + "rg2.b"])
            if f.get("kind", "dense") == "dense":
                self.mlp = DenseMLP(sub(p + "mlp."), act_dtype, tensor_cores, act="gelu_tanh")
            else:
                r = f["router"]
                g = r.get("groups") or {}
                self.mlp = MoEFeedForward(sub(p + "mlp."), r["experts"], r["top"], 1.0, act_dtype, tensor_cores, shared=bool(f.get("shared")),
                                          sorted_min_rows=sorted_min_rows, force_sorted=force_sorted, router="softmax",
                                          groups=(g.get("count", 0), g.get("keep", 0)), normalize=False, form="glu", limit=float(f["expert"].get("limit", 0.0)),
                                          shared_limit=float((f.get("shared") or {}).get("limit", 0.0)), router_logits=False)
                self.moe = True
                blocks.append(self.mlp.router_weight)
                biases.append(None)
        packed, self.spans = pack_rows(blocks)
        self.inp = Projection(packed, tensor_cores)   # every matrix that reads the normed input, as one product
        self.inp_bias = pack_biases(self.spans, packed.shape[0], biases, packed)

    def cache_specs(self):
        return [self.mixer.cache_spec()]

    def forward(self, x: torch.Tensor, h: torch.Tensor, batch: ops.PackedBatch, caches, stack: torch.Tensor, mixed: torch.Tensor,
                nxt: Optional["_Layer"], h_next: Optional[torch.Tensor]) -> None:
        """x: the fp32 rows this layer reads; h: their layer norm in the activation dtype. Stores the layer's own result as slice
        `depth - 1` of `stack`, the weighted sum over the stack in `mixed` (may be x) and, when another layer follows, that layer's
        norm of the sum in h_next."""
        P = self.inp(h, bias=self.inp_bias)
        parts = [P[:, o:o + n] for o, n in self.spans]
        y1 = self.mixer.forward(parts[:self.n_mix], batch, caches[0])
        g1 = parts[self.n_mix]
        y2 = g2 = None
        if self.mlp is not None:
            g2 = parts[self.n_mix + 1]
            y2 = self.mlp.forward(h, batch, logits=parts[self.n_mix + 2]) if self.moe else self.mlp.forward(h)
        ops.depth_mix(x, y1, g1, y2, g2, stack=stack, depth=self.depth, coef=self.coef, mixed=mixed,
                      norm_weight=nxt.norm_w if nxt is not None else None, norm_bias=nxt.norm_b if nxt is not None else None, eps=self.eps,
                      norm_out=h_next if nxt is not None else None)


class VazepelForCausalLM:
    """The model: `step(ids, batch, caches, want_rows)` runs the step's packed tokens through every layer, writing the sequences' keys
    and values into their pages in `caches` (one entry per layer: a list with the mixer's cache view), and returns fp32 logits
    [len(want_rows), vocab] of the requested rows."""

    config_class = VazepelConfig

    def __init__(self, config: VazepelConfig, weights: Dict[str, torch.Tensor], dtype: torch.dtype = torch.bfloat16,
                 device: Optional[torch.device] = None, tensor_cores: bool = True, kv_dtype: torch.dtype = torch.float32,
                 sorted_min_rows: int = 128, force_sorted: bool = False):
        if dtype not in (torch.bfloat16, torch.float32):
            raise _lib.VyomError("VazepelForCausalLM runs in bfloat16 or float32")
        self.config, self.dtype = config, dtype
        self.device = torch.device(device or "cuda")
        need = config.tensor_shapes()
        missing = [k for k in need if k not in weights]
        if missing:
            raise KeyError(f"checkpoint lacks {missing[:5]}{' ...' if len(missing) > 5 else ''}")
        for k, shp in need.items():
            if tuple(weights[k].shape) != tuple(shp):
                raise ValueError(f"{k}: shape {tuple(weights[k].shape)}, the configuration implies {tuple(shp)}")
        w = {k: v.to(device=self.device, dtype=dtype) for k, v in weights.items() if k in need}
        self.embed = w["embed"].contiguous()
        self.final_w, self.final_b = w["final.norm"].contiguous(), w["final.norm.b"].contiguous()
        self.head = Projection(w["head"], tensor_cores)
        self.layers = [_Layer(i, L, w, config, dtype, tensor_cores, kv_dtype, sorted_min_rows, force_sorted) for i, L in enumerate(config.layers)]
        self.debug_residuals: Optional[list] = None   # set to [] to collect what every layer hands on

    @classmethod
    def from_pretrained(cls, path: str, dtype: torch.dtype = torch.bfloat16, device=None, **kw) -> "VazepelForCausalLM":
        from ..checkpoint import load_safetensors
        return cls(VazepelConfig.from_dir(path), load_safetensors(os.path.join(path, "model.safetensors")), dtype=dtype, device=device, **kw)

    @staticmethod
    def random_weights(config: VazepelConfig, seed: int = 0) -> Dict[str, torch.Tensor]:
        """Seeded bf16 weights of the right shapes (tests, benchmarks): projections ~ N(0, 1/in), embeddings ~ N(0, 1), norm weights around
        1, biases small, head-mixing matrices near the identity with off-diagonal entries that matter, stack coefficients positive and
        summing to about 1 with most of the weight on the newest result, routers small enough that softmax scores stay apart."""
        g = torch.Generator().manual_seed(seed)
        out = {}
        for k, shp in config.tensor_shapes().items():
            leaf = k.split(".")[-1]
            if leaf == "embed":
                t = torch.randn(shp, generator=g)
            elif leaf == "talk":
                t = torch.eye(shp[0]) + 0.3 * torch.randn(shp, generator=g) / (shp[0] ** 0.5)
            elif leaf == "dwa":
                t = 0.5 * torch.rand(shp, generator=g) / shp[0]
                t[-1] += 0.75
            elif leaf == "router":
                t = torch.randn(shp, generator=g) * 2.0 / (shp[1] ** 0.5)
            elif len(shp) == 2:
                t = torch.randn(shp, generator=g) / (shp[1] ** 0.5)
            elif leaf == "b":
                t = 0.1 * torch.randn(shp, generator=g)
            else:   # norm weights
                t = 1.0 + 0.1 * torch.randn(shp, generator=g)
            out[k] = t.to(torch.bfloat16)
        return out

    def cache_specs(self):
        return [L.cache_specs() for L in self.layers]

    @torch.no_grad()
    def step(self, ids: torch.Tensor, batch: ops.PackedBatch, caches, want_rows: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        cfg, n = self.config, len(self.layers)
        rows = ids.numel()
        # the embedding output and every layer's own result: what each layer's closing sum reads
        stack = torch.empty((n + 1, rows, cfg.width), device=self.device, dtype=torch.float32)
        ops.embed_rows(ids, self.embed, 1.0, torch.float32, out=stack[0])
        x = stack[0]
        mixed = torch.empty((rows, cfg.width), device=self.device, dtype=torch.float32)
        h = ops.layer_norm(x, self.layers[0].norm_w, self.layers[0].norm_b, eps=cfg.eps, out_dtype=self.dtype) if n else None
        h_next = torch.empty_like(h) if n > 1 else None
        for i, (L, c) in enumerate(zip(self.layers, caches)):
            nxt = self.layers[i + 1] if i + 1 < n else None
            L.forward(x, h, batch, c, stack, mixed, nxt, h_next)
            x = mixed
            h, h_next = h_next, h
            if self.debug_residuals is not None:
                self.debug_residuals.append(x.clone())
        if want_rows is None or want_rows.numel() == 0:
            return None
        hn = ops.layer_norm(x, self.final_w, self.final_b, eps=cfg.eps, row_index=want_rows, out_dtype=self.dtype)
        return self.head(hn)
