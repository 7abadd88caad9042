"""Fubinex: a hybrid decoder-only language model. Layers are listed in the configuration; each is pre-norm
(x += mixer(norm1 x); x += ff(norm2 x)) with RMS norms taken over `norm.groups` equal consecutive parts of the vector, each part
divided by its own root mean square, and a plain weight over the whole vector. Three mixers:

  * `latent_attention` (layers/mixers.py LatentAttention): causal softmax attention over a cached low-rank latent plus one rotated
    key part per token; queries go through a latent of their own; adjacent-pair rotation with stretched frequencies and a factor on
    cos / sin (rot.scaling); a layer with `kv_from: j` owns no down-projection and attends over layer j's cached rows.
  * `parallel`: two mixers read the same normed input and their outputs are added with configured weights: grouped-query attention
    limited to the query's own block of positions, with half-split rotation and weightless RMS division of q and k (RotaryAttention),
    beside gated linear attention with a learned per-channel decay (GatedLinearAttention).
  * `retention` (RetentionMixer): linear attention with a fixed decay per head over rotated q / k, per-head RMS division, silu gate.

The feed-forward is W_down act(W_up h) with the polynomial activation of normalised powers (PolyNormMLP). Embeddings are scaled on
the way in. The reference package has no such model; it is served by the same pieces as the other packed-step decoders here
(models/gelutar.py, models/zugunex.py, models/vazepel.py): a configuration object read from config.json, weights loaded by tensor
name, the cache manager's pages and state slots (vyomai_b200/paged.py; a sharing layer is given the owner's pool), one `step` over a
packed batch that the batching engine, the CUDA-graph capture and the trace replayer all call, and greedy selection by vy_argmax_rows.

The residual stream, norms, rotation angles, attention scores, decays and recurrent state are fp32 in both dtypes; with
dtype=bfloat16 the projections read bf16 inputs on the tensor cores (fp32 results), with dtype=float32 they are fp32 FMA.
"""
from __future__ import annotations

import json
import os
from typing import Dict, List, Optional

import torch

from .. import _lib, ops
from ..layers.mixers import GatedLinearAttention, LatentAttention, PolyNormMLP, Projection, RetentionMixer, RotaryAttention, pack_rows

MIXER_TYPES = ("latent_attention", "parallel", "retention")


class FubinexConfig:
    """config.json of the architecture: vocab, width, embedding.scale, norm.{eps, groups} and `layers`, a list of
    {"type": "latent_attention", "mixer": {heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, rot: {base, dims, scaling?}, kv_from?}} |
    {"type": "parallel", "mixer": {"left": {heads, kv_heads, dim, vdim, scale, rot: {base, dims}, mask: {size}}, "left_scale",
                                   "right": {heads, dim, vdim, tau}, "right_scale"}} |
    {"type": "retention", "mixer": {heads, dim, vdim, decay: [per head], rot: {base, dims}}},
    each with "mlp": null | {"kind": "dense", "ff"}."""

    architecture = "Fubinex"

    def __init__(self, d: dict):
        if d.get("architecture") != self.architecture:
            raise ValueError(f"not a {self.architecture} configuration: {d.get('architecture')!r}")
        self.raw = d
        self.vocab, self.width = int(d["vocab"]), int(d["width"])
        self.embedding_scale = float((d.get("embedding") or {}).get("scale", 1.0))
        self.eps = float(d["norm"]["eps"])
        self.groups = int(d["norm"].get("groups", 1))
        if self.groups < 1 or self.width % self.groups:
            raise ValueError(f"norm.groups {self.groups} does not divide the width {self.width}")
        self.layers = list(d["layers"])
        for i, L in enumerate(self.layers):
            if L["type"] not in MIXER_TYPES:
                raise ValueError(f"layer {i}: unknown mixer type {L['type']!r}")
            m = L["mixer"]
            if L["type"] == "latent_attention":
                j = m.get("kv_from")
                if j is not None:
                    j = int(j)
                    if not 0 <= j < i or self.layers[j]["type"] != "latent_attention" or self.layers[j]["mixer"].get("kv_from") is not None:
                        raise ValueError(f"layer {i}: kv_from {j} must name an earlier latent-attention layer that owns its latent")
                    o = self.layers[j]["mixer"]
                    if (o["kv_rank"], o["rot_dim"], o.get("rot")) != (m["kv_rank"], m["rot_dim"], m.get("rot")):
                        raise ValueError(f"layer {i}: kv_rank / rot_dim / rot differ from layer {j}'s, whose latent it reads")
            elif L["type"] == "parallel":
                if int(m["left"]["heads"]) % int(m["left"]["kv_heads"]):
                    raise ValueError(f"layer {i}: heads must be a multiple of kv_heads")
            elif len(m["decay"]) != int(m["heads"]):
                raise ValueError(f"layer {i}: one decay per head expected")
            f = L.get("mlp")
            if f and f.get("kind", "dense") != "dense":
                raise ValueError(f"layer {i}: unknown feed-forward kind {f.get('kind')!r}")

    @classmethod
    def from_dir(cls, path: str) -> "FubinexConfig":
        with open(os.path.join(path, "config.json")) as f:
            return cls(json.load(f))

    def tensor_shapes(self) -> Dict[str, tuple]:
        """Name -> shape of every weight the configuration implies (what a checkpoint must hold; also the recipe for random
        initialisation). -1 stands for a size only the checkpoint knows (the rank of the decay's factored projection)."""
        W = self.width
        out: Dict[str, tuple] = {"embed": (self.vocab, W), "final.norm": (W,), "head": (self.vocab, W)}
        for i, L in enumerate(self.layers):
            p, m = f"l{i}.", L["mixer"]
            out[p + "norm1"] = (W,)
            if L["type"] == "latent_attention":
                H, dn, dr, dv, R, Q = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
                out.update({p + "mix.dq": (Q, W), p + "mix.dq.norm": (Q,), p + "mix.uq": (H * (dn + dr), Q), p + "mix.uk": (H * dn, R),
                            p + "mix.uv": (H * dv, R), p + "mix.o": (W, H * dv)})
                if m.get("kv_from") is None:
                    out.update({p + "mix.dkv": (R + dr, W), p + "mix.dkv.norm": (R,)})
            elif L["type"] == "parallel":
                a, r = m["left"], m["right"]
                q = p + "mix.left."
                out.update({q + "q": (a["heads"] * a["dim"], W), q + "k": (a["kv_heads"] * a["dim"], W), q + "v": (a["kv_heads"] * a["vdim"], W),
                            q + "o": (W, a["heads"] * a["vdim"])})
                q = p + "mix.right."
                out.update({q + "q": (r["heads"] * r["dim"], W), q + "k": (r["heads"] * r["dim"], W), q + "v": (r["heads"] * r["vdim"], W),
                            q + "g": (r["heads"] * r["vdim"], W), q + "o": (W, r["heads"] * r["vdim"]), q + "norm": (r["vdim"],),
                            q + "a1": (-1, W), q + "a2": (r["heads"] * r["dim"], -1), q + "a2.b": (r["heads"] * r["dim"],)})
            else:
                H, dk, dv = m["heads"], m["dim"], m["vdim"]
                out.update({p + "mix.q": (H * dk, W), p + "mix.k": (H * dk, W), p + "mix.v": (H * dv, W), p + "mix.g": (H * dv, W),
                            p + "mix.o": (W, H * dv)})
            f = L.get("mlp")
            if f:
                out.update({p + "norm2": (W,), p + "mlp.up": (f["ff"], W), p + "mlp.down": (W, f["ff"]), p + "mlp.act": (4,)})
        return out


class _Layer:
    def __init__(self, idx: int, spec: dict, w: Dict[str, torch.Tensor], cfg: FubinexConfig, act_dtype, tensor_cores: bool, kv_dtype):
        p = f"l{idx}."
        sub = lambda pre: {k[len(pre):]: v for k, v in w.items() if k.startswith(pre)}  # noqa: E731
        self.kind = spec["type"]
        self.eps, self.groups, self.act_dtype = cfg.eps, cfg.groups, act_dtype
        self.norm1 = w[p + "norm1"].contiguous()
        m = spec["mixer"]
        if self.kind == "latent_attention":
            j = m.get("kv_from")
            self.mixers = [LatentAttention(m, sub(p + "mix."), cfg.eps, act_dtype, tensor_cores, kv_dtype, shared_from=None if j is None else int(j))]
            self.out_scales = [1.0]
        elif self.kind == "parallel":
            self.mixers = [RotaryAttention(m["left"], sub(p + "mix.left."), cfg.eps, act_dtype, tensor_cores, kv_dtype, layout="half", unit_rms=True,
                                           mask_kind="chunk"),
                           GatedLinearAttention(m["right"], sub(p + "mix.right."), cfg.eps, act_dtype, tensor_cores)]
            self.out_scales = [float(m.get("left_scale", 1.0)), float(m.get("right_scale", 1.0))]
        else:
            self.mixers = [RetentionMixer(m, sub(p + "mix."), cfg.eps, act_dtype, tensor_cores)]
            self.out_scales = [1.0]
        blocks: List[torch.Tensor] = []
        self.counts = []
        for mx in self.mixers:
            ws = mx.input_weights()
            self.counts.append(len(ws))
            blocks += ws
        packed, self.spans = pack_rows(blocks)
        self.inp = Projection(packed, tensor_cores)   # every matrix that reads norm1(x), as one product
        self.mlp = None
        if spec.get("mlp"):
            self.norm2 = w[p + "norm2"].contiguous()
            self.mlp = PolyNormMLP(sub(p + "mlp."), cfg.eps, act_dtype, tensor_cores)

    def cache_specs(self):
        return [m.cache_spec() for m in self.mixers]

    def forward(self, x: torch.Tensor, batch: ops.PackedBatch, caches) -> None:
        """x: the fp32 residual, updated in place (every output projection adds into it in its epilogue)."""
        h = ops.rms_norm(x, self.norm1, eps=self.eps, w_mode="plain", groups=self.groups, w_full=True, out_dtype=self.act_dtype)
        P = self.inp(h)
        parts = [P[:, o:o + n] for o, n in self.spans]
        at = 0
        for m, cnt, c, sc in zip(self.mixers, self.counts, caches, self.out_scales):
            if sc == 0.0:   # a mixer whose weight in the sum is zero: nothing reads its output, and only itself its state
                at += cnt
                continue
            if self.kind == "latent_attention":
                m.forward(parts[at:at + cnt], batch, c, x_residual=x)
            else:
                m.forward(parts[at:at + cnt], batch, c, x_residual=x, out_scale=sc)
            at += cnt
        if self.mlp is not None:
            h2 = ops.rms_norm(x, self.norm2, eps=self.eps, w_mode="plain", groups=self.groups, w_full=True, out_dtype=self.act_dtype)
            self.mlp.forward(h2, x)


class FubinexForCausalLM:
    """The model: `step(ids, batch, caches, want_rows)` runs the step's packed tokens through every layer, updating the sequences'
    pages and state slots in `caches` (one entry per layer: a list with one cache view per mixer; a sharing layer's view IS its
    owner's), and returns fp32 logits [len(want_rows), vocab] of the requested rows."""

    config_class = FubinexConfig

    def __init__(self, config: FubinexConfig, weights: Dict[str, torch.Tensor], dtype: torch.dtype = torch.bfloat16,
                 device: Optional[torch.device] = None, tensor_cores: bool = True, kv_dtype: torch.dtype = torch.float32):
        if dtype not in (torch.bfloat16, torch.float32):
            raise _lib.VyomError("FubinexForCausalLM runs in bfloat16 or float32")
        self.config, self.dtype = config, dtype
        self.device = torch.device(device or "cuda")
        need = config.tensor_shapes()
        missing = [k for k in need if k not in weights]
        if missing:
            raise KeyError(f"checkpoint lacks {missing[:5]}{' ...' if len(missing) > 5 else ''}")
        for k, shp in need.items():
            got = tuple(weights[k].shape)
            if len(got) != len(shp) or any(a != b for a, b in zip(got, shp) if b >= 0):
                raise ValueError(f"{k}: shape {got}, the configuration implies {tuple(shp)}")
            if k.endswith("mix.right.a1") and weights[k[:-1] + "2"].shape[1] != got[0]:
                raise ValueError(f"{k}: rank {got[0]} does not match {k[:-1]}2")
        w = {k: v.to(device=self.device, dtype=dtype) for k, v in weights.items() if k in need}
        self.embed = w["embed"].contiguous()
        self.final_norm = w["final.norm"].contiguous()
        self.head = Projection(w["head"], tensor_cores)
        self.layers = [_Layer(i, L, w, config, dtype, tensor_cores, kv_dtype) for i, L in enumerate(config.layers)]
        self.debug_residuals: Optional[list] = None   # set to [] to collect the residual stream after every layer

    @classmethod
    def from_pretrained(cls, path: str, dtype: torch.dtype = torch.bfloat16, device=None, **kw) -> "FubinexForCausalLM":
        from ..checkpoint import load_safetensors
        return cls(FubinexConfig.from_dir(path), load_safetensors(os.path.join(path, "model.safetensors")), dtype=dtype, device=device, **kw)

    @staticmethod
    def random_weights(config: FubinexConfig, seed: int = 0, low_rank: int = 16) -> Dict[str, torch.Tensor]:
        """Seeded bf16 weights of the right shapes (tests, benchmarks): projections ~ N(0, 1/in), embeddings ~ N(0, 1), norm weights
        around 1, decay biases in the range that gives per-channel decays between ~0.8 and ~1, activation numbers of order 1."""
        g = torch.Generator().manual_seed(seed)
        out = {}
        for k, shp in config.tensor_shapes().items():
            leaf = k.split(".")[-1]
            shp = tuple(low_rank if n < 0 else n for n in shp)
            if leaf == "embed":
                t = torch.randn(shp, generator=g)
            elif leaf == "act":
                t = torch.tensor([0.9, 0.5, 0.3, 0.1]) + 0.1 * torch.randn(shp, generator=g)
            elif k.endswith("a2.b"):
                t = 1.0 + 2.0 * torch.rand(shp, generator=g)
            elif len(shp) == 2:
                t = torch.randn(shp, generator=g) / (shp[1] ** 0.5)
            else:   # norm weights
                t = 1.0 + 0.1 * torch.randn(shp, generator=g)
            out[k] = t.to(torch.bfloat16)
        return out

    def cache_specs(self):
        return [L.cache_specs() for L in self.layers]

    @torch.no_grad()
    def step(self, ids: torch.Tensor, batch: ops.PackedBatch, caches, want_rows: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        cfg = self.config
        x = ops.embed_rows(ids, self.embed, cfg.embedding_scale, torch.float32)
        for L, c in zip(self.layers, caches):
            L.forward(x, batch, c)
            if self.debug_residuals is not None:
                self.debug_residuals.append(x.clone())
        if want_rows is None or want_rows.numel() == 0:
            return None
        hn = ops.rms_norm(x, self.final_norm, eps=cfg.eps, w_mode="plain", groups=cfg.groups, w_full=True, row_index=want_rows, out_dtype=self.dtype)
        return self.head(hn)
