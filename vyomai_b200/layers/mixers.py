"""Sequence mixers and feed-forwards of the packed-step decoder families (models/gelutar.py, models/zugunex.py, models/vazepel.py,
models/fubinex.py), on the packed-batch kernels of csrc/seqmix.cu, csrc/latent.cu, csrc/talking_attn.cu, csrc/parallel_block.cu and
csrc/rowwise.cu. Each mixer is built from its config block and its weights, declares what it keeps per sequence
(`cache_spec`: pages of keys / values, recurrent state slots) and maps the normed layer input h [rows, width] to its
output; the constants of a mechanism (window, kept tokens, scale, sink, decay, taps, head counts) are constructor
arguments, so another architecture can reuse a mixer with other values.

Precision: projections run on the tensor cores in bf16 with fp32 accumulation and fp32 results (`Projection`), or in true
fp32 when the model is built with dtype float32; everything between two projections (norms, scores, softmax, gates,
convolutions, decays, recurrences, the residual) is fp32, and only a projection's INPUT is rounded to bf16.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from .. import _lib, ops


def _round_up(n: int, m: int) -> int:
    return (n + m - 1) // m * m


class Projection:
    """y = act(x W^T + bias) * scale + addend for a weight stored [out, in]. bf16 weights with 16-byte-aligned rows go to the
    tcgen05 / small-batch GEMM (vy_gemm, fp32 result); fp32 weights and every other shape go to the fp32-FMA kernel."""

    def __init__(self, weight: torch.Tensor, tensor_cores: bool = True):
        # a column slice of a wider matrix (unit column stride, 16-byte aligned rows) is used in place, not copied
        view_ok = weight.dim() == 2 and weight.stride(1) == 1 and (weight.stride(0) * weight.element_size()) % 16 == 0 and weight.data_ptr() % 16 == 0
        self.weight = weight if view_ok else weight.contiguous()
        self.out_features, self.in_features = weight.shape
        self.tensor_cores = bool(tensor_cores) and weight.dtype == torch.bfloat16 and self.in_features % 8 == 0 and self.in_features >= 32 \
            and self.out_features >= 16

    def __call__(self, x: torch.Tensor, *, act: Optional[str] = None, bias: Optional[torch.Tensor] = None, scale: float = 1.0,
                 addend: Optional[torch.Tensor] = None, out_dtype: torch.dtype = torch.float32, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        N = self.out_features
        if addend is not None and scale != 1.0:   # the two kernels order the scale and the addend differently
            raise _lib.VyomError("Projection: a scale together with an addend is not defined; fold the scale into the input")
        if out is None:
            out = torch.empty((x.shape[0], _round_up(N, 8)), device=x.device, dtype=out_dtype)[:, :N]
        tc = self.tensor_cores and x.dtype == torch.bfloat16 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 \
            and act in (None, "none", "relu2", "gelu_tanh")
        if tc:
            ops.gemm(x, self.weight, bias=bias, act=act, addend=addend, out=out, out_scale=scale, swap_ab=x.shape[0] <= 32)
        else:
            ops.linear_plain(x, self.weight, bias=bias, act=act, scale=scale, addend=addend, out=out)
        return out


def pack_rows(tensors: List[torch.Tensor], align: int = 8) -> Tuple[torch.Tensor, List[Tuple[int, int]]]:
    """Stacks weights that read the same input into one [sum out, in] matrix (each block padded with zero rows to a multiple
    of `align` outputs, so every block of the product starts at an aligned column). Returns the matrix and (offset, rows)
    of each block."""
    K = tensors[0].shape[1]
    spans, off = [], 0
    for t in tensors:
        spans.append((off, t.shape[0]))
        off += _round_up(t.shape[0], align)
    w = torch.zeros((off, K), dtype=tensors[0].dtype, device=tensors[0].device)
    for t, (o, n) in zip(tensors, spans):
        w[o:o + n] = t
    return w, spans


def pack_biases(spans: List[Tuple[int, int]], total: int, biases: List[Optional[torch.Tensor]], like: torch.Tensor) -> Optional[torch.Tensor]:
    """The bias of a packed projection: each block's bias at the block's offset, zero where a block has none (None when no block has one)."""
    if not any(b is not None for b in biases):
        return None
    out = torch.zeros(total, dtype=like.dtype, device=like.device)
    for (o, n), b in zip(spans, biases):
        if b is not None:
            out[o:o + n] = b
    return out


def rotary_frequencies(rot: dict, dims: int, device) -> Tuple[torch.Tensor, float]:
    """(inv_freq fp32 [dims / 2], factor on cos and sin) of a rotation block {"base", "dims", "scaling"?}. Without scaling
    f_i = base^(-2i / dims) and the factor is 1. scaling = {"factor", "original", "fast", "slow"} stretches the slow frequencies
    (YaRN): with n(t) = dims ln(original / (2 pi t)) / (2 ln base), lo = max(floor(n(fast)), 0), hi = min(ceil(n(slow)), dims - 1) and
    ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), the frequency is f_i / factor where the ramp is 1, f_i where it is 0, their
    blend between, and cos / sin are multiplied by 0.1 ln(factor) + 1."""
    import math
    base = float(rot.get("base", 10000.0))
    half = dims // 2
    f = [base ** (-2.0 * i / dims) for i in range(half)] or [0.0]
    factor_out = 1.0
    sc = rot.get("scaling")
    if sc and half:
        factor, orig = float(sc["factor"]), float(sc["original"])
        turns = lambda t: dims * math.log(orig / (2.0 * math.pi * t)) / (2.0 * math.log(base))  # noqa: E731
        lo = max(math.floor(turns(float(sc["fast"]))), 0)
        hi = min(math.ceil(turns(float(sc["slow"]))), dims - 1)
        for i in range(half):
            ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
            f[i] = f[i] / factor * ramp + f[i] * (1.0 - ramp)
        factor_out = 0.1 * math.log(factor) + 1.0
    return torch.tensor(f, dtype=torch.float64).to(torch.float32).to(device), factor_out


class Mixer:
    """Common surface: `cache_spec()` -> {"pages": (kv_heads, dim, vdim) | None, "states": {name: per-slot shape}};
    `input_weights()` -> the [out, in] matrices that read the layer input (packed by the layer into one projection), `input_biases()` ->
    their biases (None entries for none); `forward(parts, batch, cache)` with `parts` the list of product blocks in the same order.
    Mixers that can stand beside another one in a layer also take `x_residual` (the fp32 residual their output projection adds into in
    its epilogue) and `out_scale` (the mixer's weight in the layer's sum, multiplied in fp32 into what the output projection reads,
    before that is rounded)."""

    def cache_spec(self) -> dict:
        return {"pages": None, "states": {}}

    def input_biases(self):
        return [None] * len(self.input_weights())


class LightningMixer(Mixer):
    """Linear attention with one fixed decay per head: q, k, v = silu(projections), S_t = decay_h S_(t-1) + k_t v_t^T,
    o_t = S_t^T q_t; the heads' outputs are RMS-normed together, gated by sigmoid(W_g h) and projected."""

    def __init__(self, cfg: dict, w: Dict[str, torch.Tensor], eps: float, act_dtype: torch.dtype, tensor_cores: bool):
        self.heads, self.dim, self.vdim = int(cfg["heads"]), int(cfg["dim"]), int(cfg["vdim"])
        if len(cfg["decay"]) != self.heads:
            raise ValueError("lightning mixer: one decay per head expected")
        self.eps, self.act_dtype = eps, act_dtype
        dev = w["q"].device
        self.decay = torch.tensor([float(d) for d in cfg["decay"]], dtype=torch.float32, device=dev)
        self._in = [w["q"], w["k"], w["v"], w["g"]]
        self.norm = w["norm"].contiguous()
        self.o = Projection(w["o"], tensor_cores)

    def input_weights(self):
        return self._in

    def cache_spec(self):
        return {"pages": None, "states": {"S": (self.heads, self.dim, self.vdim)}}

    def forward(self, parts, batch, cache, x_residual: Optional[torch.Tensor] = None):
        q, k, v, g = parts
        o = ops.linear_attn(batch, q, k, v, self.decay, cache.states["S"], heads=self.heads, dim=self.dim, vdim=self.vdim, in_act="silu")
        og = ops.rms_norm(o, self.norm, eps=self.eps, w_mode="plain", gate=g, gate_act="sigmoid", out_dtype=self.act_dtype)
        if x_residual is not None:  # x += W_o(...) in the projection's epilogue
            return self.o(og, addend=x_residual, out=x_residual)
        return self.o(og)


class WindowSinkAttention(Mixer):
    """Softmax attention without rotation: whole-projection RMS norm of q and k (plain weights), score = q.k * scale, causal
    sliding window that also keeps the first tokens, a learned per-head sink in the denominator, and a per-head sigmoid
    output gate read from the layer input. Keys / values live in pages."""

    def __init__(self, cfg: dict, w: Dict[str, torch.Tensor], eps: float, act_dtype: torch.dtype, tensor_cores: bool,
                 kv_dtype: torch.dtype = torch.float32):
        self.heads, self.kv_heads = int(cfg["heads"]), int(cfg["kv_heads"])
        self.dim, self.vdim = int(cfg["dim"]), int(cfg["vdim"])
        if self.heads % self.kv_heads:
            raise ValueError("attention: heads must be a multiple of kv_heads")
        mask = cfg.get("mask") or {}
        self.window, self.keep_first = int(mask.get("size", 0)), int(mask.get("keep_first", 0))
        self.scale = float(cfg["scale"])
        self.eps, self.act_dtype, self.kv_dtype = eps, act_dtype, kv_dtype
        self._in = [w["q"], w["k"], w["v"], w["g"]]
        self.q_norm, self.k_norm = w["q.norm"].contiguous(), w["k.norm"].contiguous()
        self.sink = w["sink"].contiguous() if "sink" in w else None
        self.o = Projection(w["o"], tensor_cores)

    def input_weights(self):
        return self._in

    def cache_spec(self):
        return {"pages": (self.kv_heads, self.dim, self.vdim), "states": {}, "kv_dtype": self.kv_dtype}

    def forward(self, parts, batch, cache):
        q, k, v, g = parts
        qn = ops.rms_norm(q, self.q_norm, eps=self.eps, w_mode="plain", out_dtype=torch.float32)
        kn = ops.rms_norm(k, self.k_norm, eps=self.eps, w_mode="plain", out_dtype=torch.float32)
        ops.kv_page_write(batch, kn, v, cache.k_pool, cache.v_pool)
        a = ops.window_attn(batch, qn, cache.k_pool, cache.v_pool, heads=self.heads, kv_heads=self.kv_heads, dim=self.dim, vdim=self.vdim,
                            scale=self.scale, window=self.window, keep_first=self.keep_first, sink=self.sink, gate=g,
                            out_dtype=self.act_dtype)
        return self.o(a)


class GatedDeltaMixer(Mixer):
    """Gated delta rule: q / k / v pass a short causal depthwise convolution and silu, q and k become unit vectors per head
    (q also times dim^-1/2), a per-channel decay exp(-exp(A_log) softplus(W_a2 W_a1 h + dt_bias)) shrinks the state, a
    sigmoid write strength scales the delta update; the read-out is RMS-normed per head, gated by sigmoid(W_g2 W_g1 h) and
    projected."""

    def __init__(self, cfg: dict, w: Dict[str, torch.Tensor], eps: float, act_dtype: torch.dtype, tensor_cores: bool):
        self.heads, self.kv_heads = int(cfg["heads"]), int(cfg["kv_heads"])
        self.dim, self.vdim, self.taps = int(cfg["dim"]), int(cfg["vdim"]), int(cfg["conv"])
        if self.heads % self.kv_heads:
            raise ValueError("delta mixer: heads must be a multiple of kv_heads")
        self.eps, self.act_dtype = eps, act_dtype
        # q | k | v are adjacent blocks of the packed product (widths are multiples of the packing alignment or the last block),
        # so one convolution call covers all three when their channel counts need no padding; otherwise three calls
        self._in = [w["q"], w["k"], w["v"], w["b"], w["a1"], w["g1"]]
        self.conv_w = [w["q.conv"].contiguous(), w["k.conv"].contiguous(), w["v.conv"].contiguous()]
        self.a2 = Projection(w["a2"], False)  # contractions over the low rank: fp32 activations straight from the a1 / g1 blocks
        self.g2 = Projection(w["g2"], False)
        self.dt_bias = w["dt_bias"].contiguous()
        self.a_log = w["A_log"].contiguous()
        self.norm = w["norm"].contiguous()
        self.o = Projection(w["o"], tensor_cores)

    def input_weights(self):
        return self._in

    def cache_spec(self):
        qk, vv = self.kv_heads * self.dim, self.heads * self.vdim
        st = {"S": (self.heads, self.dim, self.vdim)}
        if self.taps > 1:
            st.update({"conv_q": (qk, self.taps - 1), "conv_k": (qk, self.taps - 1), "conv_v": (vv, self.taps - 1)})
        return {"pages": None, "states": st}

    def forward(self, parts, batch, cache):
        q, k, v, b, a1, g1 = parts
        dummy = cache.states["S"]
        qc = ops.causal_conv(batch, q, self.conv_w[0], cache.states.get("conv_q", dummy), act="silu", out_dtype=torch.float32)
        kc = ops.causal_conv(batch, k, self.conv_w[1], cache.states.get("conv_k", dummy), act="silu", out_dtype=torch.float32)
        vc = ops.causal_conv(batch, v, self.conv_w[2], cache.states.get("conv_v", dummy), act="silu", out_dtype=torch.float32)
        a = self.a2(a1, bias=self.dt_bias)
        g = self.g2(g1)
        o = ops.delta_rule(batch, qc, kc, vc, a, b, self.a_log, cache.states["S"], heads=self.heads, kv_heads=self.kv_heads, dim=self.dim,
                           vdim=self.vdim, unit_eps=1e-6)
        on = ops.rms_norm(o, self.norm, eps=self.eps, w_mode="plain", groups=self.heads, gate=g, gate_act="sigmoid", out_dtype=self.act_dtype)
        return self.o(on)


class RetentionMixer(Mixer):
    """Linear attention with one fixed decay per head and rotated queries / keys, no softmax and no denominator: q, k turn by position
    (entry i paired with entry i + rot.dims / 2 on the leading rot.dims entries of each head), k is then scaled by dim^-1/2,
    S_t = decay_h S_(t-1) + k_t v_t^T, o_t = S_t^T q_t; each head's read-out is divided by its root mean square (no weight), the heads
    are gated by silu(W_g h) and projected. The state is fp32 per sequence slot."""

    def __init__(self, cfg: dict, w: Dict[str, torch.Tensor], eps: float, act_dtype: torch.dtype, tensor_cores: bool):
        self.heads, self.dim, self.vdim = int(cfg["heads"]), int(cfg["dim"]), int(cfg["vdim"])
        if len(cfg["decay"]) != self.heads:
            raise ValueError("retention: one decay per head expected")
        rot = cfg.get("rot") or {}
        self.rot_dims = int(rot.get("dims", 0))
        if self.rot_dims > self.dim or self.rot_dims % 2:
            raise ValueError("retention: rot.dims must be even and at most dim")
        self.eps, self.act_dtype = eps, act_dtype
        dev = w["q"].device
        self.inv_freq, self.rot_scale = rotary_frequencies(rot, self.rot_dims, dev)
        self.decay = torch.tensor([float(d) for d in cfg["decay"]], dtype=torch.float32, device=dev)
        self._in = [w["q"], w["k"], w["v"], w["g"]]
        self.o = Projection(w["o"], tensor_cores)

    def input_weights(self):
        return self._in

    def cache_spec(self):
        return {"pages": None, "states": {"S": (self.heads, self.dim, self.vdim)}}

    def forward(self, parts, batch, cache, x_residual: Optional[torch.Tensor] = None, out_scale: float = 1.0):
        q, k, v, g = parts
        ops.rope_kv_write(batch, q, k, None, self.inv_freq, None, None, heads=self.heads, kv_heads=self.heads, dim=self.dim, vdim=self.vdim,
                          rot_dims=self.rot_dims, layout="half", rot_scale=self.rot_scale, k_scale=self.dim ** -0.5, k_out=k)
        o = ops.linear_attn(batch, q, k, v, self.decay, cache.states["S"], heads=self.heads, dim=self.dim, vdim=self.vdim, in_act=None)
        og = ops.rms_norm(o, None, eps=self.eps, groups=self.heads, gate=g, gate_act="silu", coef=out_scale, out_dtype=self.act_dtype)
        return self.o(og, addend=x_residual, out=x_residual)


class GatedLinearAttention(Mixer):
    """Linear attention with a learned decay per key channel and token: q = W_q h dim^-1/2, k = W_k h, v = W_v h,
    alpha = sigmoid(W_a2 W_a1 h + b_a2)^(1 / tau) (heads x dim), S_t = diag(alpha_t) S_(t-1) + k_t v_t^T, o_t = S_t^T q_t; each head's
    read-out is RMS-normed with one weight [vdim] shared by the heads, the heads are gated by silu(W_g h) and projected. Decay logits,
    decays and state are fp32."""

    def __init__(self, cfg: dict, w: Dict[str, torch.Tensor], eps: float, act_dtype: torch.dtype, tensor_cores: bool):
        self.heads, self.dim, self.vdim = int(cfg["heads"]), int(cfg["dim"]), int(cfg["vdim"])
        self.tau = float(cfg.get("tau", 1.0))
        if self.tau <= 0.0:
            raise ValueError("gated linear attention: tau must be positive")
        self.eps, self.act_dtype = eps, act_dtype
        self._in = [w["q"], w["k"], w["v"], w["g"], w["a1"]]
        self.a2 = Projection(w["a2"], False)   # contraction over the low rank: fp32 activations straight from the a1 block
        self.a2_bias = w["a2.b"].contiguous()
        self.norm = w["norm"].contiguous()
        self.o = Projection(w["o"], tensor_cores)

    def input_weights(self):
        return self._in

    def cache_spec(self):
        return {"pages": None, "states": {"S": (self.heads, self.dim, self.vdim)}}

    def forward(self, parts, batch, cache, x_residual: Optional[torch.Tensor] = None, out_scale: float = 1.0):
        q, k, v, g, a1 = parts
        a = self.a2(a1, bias=self.a2_bias)
        o = ops.gated_linear_attn(batch, q, k, v, a, cache.states["S"], heads=self.heads, dim=self.dim, vdim=self.vdim, tau=self.tau,
                                  q_scale=self.dim ** -0.5)
        on = ops.rms_norm(o, self.norm, eps=self.eps, w_mode="plain", groups=self.heads, gate=g, gate_act="silu", coef=out_scale, out_dtype=self.act_dtype)
        return self.o(on, addend=x_residual, out=x_residual)


class RotaryAttention(Mixer):
    """Grouped-query softmax attention with rotated queries / keys over pages: the leading rot.dims entries of each head turn by
    position (`layout` "half": entry i with entry i + rot.dims / 2; "pairs": entries 2i, 2i + 1), then, with `unit_rms`, every head of q
    and k is divided by its root mean square over dim (no weight); score = q . k * scale. mask = {"size": n} limits a query to its own
    block of n consecutive positions counted from position 0 (`mask_kind` "chunk") or to the last n positions ("window"); no mask
    entry = plain causal. Keys (rotated, normed) and values live in pages."""

    def __init__(self, cfg: dict, w: Dict[str, torch.Tensor], eps: float, act_dtype: torch.dtype, tensor_cores: bool,
                 kv_dtype: torch.dtype = torch.float32, layout: str = "half", unit_rms: bool = True, mask_kind: str = "chunk"):
        self.heads, self.kv_heads = int(cfg["heads"]), int(cfg["kv_heads"])
        self.dim, self.vdim = int(cfg["dim"]), int(cfg["vdim"])
        if self.heads % self.kv_heads:
            raise ValueError("attention: heads must be a multiple of kv_heads")
        rot = cfg.get("rot") or {}
        self.rot_dims = int(rot.get("dims", 0))
        if self.rot_dims > self.dim or self.rot_dims % 2:
            raise ValueError("attention: rot.dims must be even and at most dim")
        if mask_kind not in ("chunk", "window"):
            raise ValueError(f"attention: unknown mask kind {mask_kind!r}")
        size = int((cfg.get("mask") or {}).get("size", 0))
        self.chunk, self.window = (size, 0) if mask_kind == "chunk" else (0, size)
        self.scale = float(cfg["scale"])
        self.layout, self.unit_rms = layout, bool(unit_rms)
        self.eps, self.act_dtype, self.kv_dtype = eps, act_dtype, kv_dtype
        self.inv_freq, self.rot_scale = rotary_frequencies(rot, self.rot_dims, w["q"].device)
        self._in = [w["q"], w["k"], w["v"]]
        self.o = Projection(w["o"], tensor_cores)

    def input_weights(self):
        return self._in

    def cache_spec(self):
        return {"pages": (self.kv_heads, self.dim, self.vdim), "states": {}, "kv_dtype": self.kv_dtype}

    def forward(self, parts, batch, cache, x_residual: Optional[torch.Tensor] = None, out_scale: float = 1.0):
        q, k, v = parts
        ops.rope_kv_write(batch, q, k, v, self.inv_freq, cache.k_pool, cache.v_pool, heads=self.heads, kv_heads=self.kv_heads, dim=self.dim,
                          vdim=self.vdim, rot_dims=self.rot_dims, layout=self.layout, rot_scale=self.rot_scale, unit_rms=self.unit_rms, eps=self.eps)
        a = ops.window_attn(batch, q, cache.k_pool, cache.v_pool, heads=self.heads, kv_heads=self.kv_heads, dim=self.dim, vdim=self.vdim,
                            scale=self.scale, window=self.window, keep_first=0, chunk=self.chunk, out_scale=out_scale, out_dtype=self.act_dtype)
        return self.o(a, addend=x_residual, out=x_residual)


class LatentAttention(Mixer):
    """Attention whose keys and values are linear images of a cached low-rank latent: per token the cache holds the RMS-normed
    latent c [rank] and one rotated key part kr [rot_dim] shared by the heads. Head h scores (qn_h . W_uk_h c + qr_h . kr) * scale
    and outputs W_uv_h sum_j p_j c_j, so the kernels never expand keys or values: the unrotated query part is carried into latent
    space once per token (qa_h = W_uk_h^T qn_h) and the attention runs with ONE key/value head over rows [c | kr] (key = the whole
    row, value = its first `rank` entries, both views of one pool), followed by the per-head value expansion. Pair rotation by
    position on the rotated parts (optionally with stretched frequencies and a factor on cos / sin: rot.scaling, see
    rotary_frequencies), sliding window, softmax sink and sigmoid output gate as in WindowSinkAttention, each only when the
    configuration / the weights hold it (`mask`, `sink`, `g`). Queries come from the layer input directly (weight `q`) or through a
    latent of their own (weights `dq`, `dq.norm`, `uq`: q = W_uq RMSnorm(W_dq h)). A mixer built with `shared_from` owns no
    down-projection: it reads the pool of the layer it names with its own W_uk / W_uv / queries.

    Whole prompts (every sequence of the step at position 0, bf16 projections) take the expanded form instead: nothing older
    than the step is visible, so the step's own rows [c | kr] (written packed beside the pages) are expanded by ONE tensor-core
    product against [W_uk_h 0; 0 I] per head and [W_uv 0] into per-head keys [kn_h | kr] and values, and the windowed attention
    runs over that buffer with dim + rot_dim / vdim channels per head (2.6 x fewer fp32 multiply-adds than latent rows at
    64 + 32 / 64 channels against rank 192) and no per-head products. Both forms are the same sum."""

    def __init__(self, cfg: dict, w: Dict[str, torch.Tensor], eps: float, act_dtype: torch.dtype, tensor_cores: bool,
                 kv_dtype: torch.dtype = torch.float32, shared_from: Optional[int] = None):
        self.heads, self.dim, self.rot_dim = int(cfg["heads"]), int(cfg["dim"]), int(cfg["rot_dim"])
        self.vdim, self.rank = int(cfg["vdim"]), int(cfg["kv_rank"])
        rot = cfg.get("rot") or {}
        self.rot_dims = int(rot.get("dims", self.rot_dim)) if self.rot_dim else 0
        if self.rot_dims > self.rot_dim or self.rot_dims % 2:
            raise ValueError("latent attention: rot.dims must be even and at most rot_dim")
        self.window = int((cfg.get("mask") or {}).get("size", 0))
        self.scale = float(cfg["scale"])
        self.eps, self.act_dtype, self.kv_dtype, self.shared_from = eps, act_dtype, kv_dtype, shared_from
        self.tensor_cores = bool(tensor_cores) and w["uk"].dtype == torch.bfloat16
        dev = w["uk"].device
        self.inv_freq, self.rot_scale = rotary_frequencies(rot, self.rot_dims, dev)
        self.row = self.rank + self.rot_dim   # one pool row: [latent | rotated key part]
        if self.row > 256 or self.rank > 256:
            raise ValueError(f"latent attention: kv_rank + rot_dim = {self.row} exceeds the attention kernels' 256 channels per head")
        H, dn, R, dv = self.heads, self.dim, self.rank, self.vdim
        self.q_latent, self.has_gate = "dq" in w, "g" in w
        self._in = [w["dq"] if self.q_latent else w["q"]] + ([] if shared_from is not None else [w["dkv"]]) + ([w["g"]] if self.has_gate else [])
        if self.q_latent:
            self.dq_norm = w["dq.norm"].contiguous()
            self.uq = Projection(w["uq"], tensor_cores)
        self.dkv_norm = None if shared_from is not None else w["dkv.norm"].contiguous()
        self.uk_t = w["uk"].view(H, dn, R).transpose(1, 2).contiguous()   # [H, R, dn]: head h maps qn_h to latent space
        self.uv = w["uv"].view(H, dv, R).contiguous()                       # [H, dv, R]
        self.sink = w["sink"].contiguous() if "sink" in w else None
        self.o = Projection(w["o"], tensor_cores)
        self.expand = None
        hd = dn + self.rot_dim
        if self.tensor_cores and act_dtype == torch.bfloat16 and self.row % 8 == 0 and hd % 4 == 0 and hd <= 256 and dv <= 256:
            wk = torch.zeros((H, hd, self.row), dtype=w["uk"].dtype, device=dev)
            wk[:, :dn, :R] = w["uk"].view(H, dn, R)
            wk[:, dn:, R:] = torch.eye(self.rot_dim, dtype=w["uk"].dtype, device=dev)
            wv = torch.zeros((H * dv, self.row), dtype=w["uv"].dtype, device=dev)
            wv[:, :R] = w["uv"]
            self.expand = Projection(torch.cat([wk.view(H * hd, self.row), wv], 0).contiguous(), tensor_cores)

    def input_weights(self):
        return self._in

    def cache_spec(self):
        if self.shared_from is not None:
            return {"pages": None, "states": {}, "pages_from": (self.shared_from, 0)}
        return {"pages": (1, self.row, 0), "states": {}, "kv_dtype": self.kv_dtype}

    def _per_head(self, x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, x_head: int, out_head: int) -> None:
        """out[:, h * out_head : + N] = x[:, h * x_head : + K] @ w[h].T for every head: tensor-core products per head for prompt-sized
        steps when the slices are aligned for them, one batched fp32-FMA launch otherwise."""
        H, N, K = w.shape
        es_o = out.element_size()
        tc = self.tensor_cores and x.shape[0] > 32 and x.dtype == torch.bfloat16 and K % 8 == 0 and K >= 32 and N >= 16 and x_head % 8 == 0 \
            and (out_head * es_o) % 16 == 0 and (out.stride(0) * es_o) % 16 == 0 and x.stride(0) % 8 == 0
        if not tc:
            ops.head_linear(x, w, out, x_head=x_head, out_head=out_head)
            return
        for h in range(H):
            ops.gemm(x[:, h * x_head:h * x_head + K], w[h], out=out[:, h * out_head:h * out_head + N])

    def forward(self, parts, batch, cache, expanded: Optional[bool] = None, x_residual: Optional[torch.Tensor] = None):
        """expanded: force (True) or forbid (False) the whole-prompt form; None = whenever the step allows it. x_residual: the fp32
        residual the output projection adds into (and returns) in its epilogue."""
        rows, H = parts[0].shape[0], self.heads
        whole = self.expand is not None and ((batch.all_start and batch.max_new >= 16) if expanded is None else bool(expanded))
        q = parts[0]
        g = parts[-1] if self.has_gate else None
        if self.q_latent:   # queries through their own latent: q = W_uq RMSnorm(W_dq h)
            q = self.uq(ops.rms_norm(q, self.dq_norm, eps=self.eps, w_mode="plain", out_dtype=self.act_dtype))
        if self.shared_from is None:
            dkv = parts[1]
            # the step's rows packed in step order, kept on the (shared) cache view for the layers that read this layer's rows
            cache.step_rows = torch.empty((rows, self.row), device=q.device, dtype=self.act_dtype) if whole else None
            ops.latent_kv_write(batch, dkv, self.dkv_norm, self.inv_freq, cache.k_pool, rank=self.rank, rot_dim=self.rot_dim,
                                rot_dims=self.rot_dims, eps=self.eps, copy_out=cache.step_rows, rot_scale=self.rot_scale)
        else:
            whole = whole and getattr(cache, "step_rows", None) is not None and cache.step_rows.shape[0] == rows
        if whole:
            hd = self.dim + self.rot_dim
            kv = self.expand(cache.step_rows)   # fp32 [rows, H (dim + rot_dim) | H vdim]
            ops.rope_split(batch, q, self.inv_freq, heads=H, keep=self.dim, rot_dim=self.rot_dim, rot_dims=self.rot_dims, pass_out=None, rot_out=q,
                           rot_head=hd, rot_col=self.dim, rot_scale=self.rot_scale)   # in place: each thread reads its pair before it writes it
            # the buffer as a one-position-per-page pool in step order: position p of sequence s is row cu_tokens[s] + p
            table = (batch.cu_tokens[:-1, None] + torch.arange(batch.max_new, device=q.device, dtype=torch.int32)[None, :]).contiguous()
            flat = ops.PackedBatch(batch.cu_tokens, batch.pos0, batch.slot, batch.max_new, table, 1)
            a = ops.window_attn(flat, q, kv, kv[:, H * hd:], heads=H, kv_heads=H, dim=hd, vdim=self.vdim, scale=self.scale, window=self.window,
                                keep_first=0, sink=self.sink, gate=g, out_dtype=self.act_dtype, k_row=kv.stride(0), v_row=kv.stride(0))
            return self.o(a, addend=x_residual, out=x_residual)
        Q = torch.empty((rows, H * self.row), device=q.device, dtype=torch.float32)
        qn = torch.empty((rows, H * self.dim), device=q.device, dtype=self.act_dtype)
        ops.rope_split(batch, q, self.inv_freq, heads=H, keep=self.dim, rot_dim=self.rot_dim, rot_dims=self.rot_dims, pass_out=qn, rot_out=Q,
                       rot_head=self.row, rot_col=self.rank, rot_scale=self.rot_scale)
        self._per_head(qn, self.uk_t, Q, self.dim, self.row)
        pool = cache.k_pool
        a = ops.window_attn(batch, Q, pool, pool, heads=H, kv_heads=1, dim=self.row, vdim=self.rank, scale=self.scale, window=self.window,
                            keep_first=0, sink=self.sink, gate=g, out_dtype=self.act_dtype, k_row=self.row, v_row=self.row)
        o = torch.empty((rows, H * self.vdim), device=q.device, dtype=self.act_dtype)
        self._per_head(a, self.uv, o, self.rank, self.vdim)
        return self.o(o, addend=x_residual, out=x_residual)


class TalkingHeadsAttention(Mixer):
    """Grouped-query softmax attention whose heads exchange scores: biased q / k / v projections, pair rotation by position on the
    leading rot.dims entries of every head, score = cap tanh(q.k scale / cap), the scores of all heads mixed through a [heads, heads]
    matrix before the softmax, causal (optionally windowed) mask, a sink in the denominator (`sink`: "zero" = a term of score 0,
    "learned" = the per-head tensor `sink`, None = none), a per-channel sigmoid output gate read from the layer input and a biased
    output projection. Keys (rotated) and values live in pages."""

    def __init__(self, cfg: dict, w: Dict[str, torch.Tensor], eps: float, act_dtype: torch.dtype, tensor_cores: bool,
                 kv_dtype: torch.dtype = torch.float32, sink: Optional[str] = "zero"):
        self.heads, self.kv_heads = int(cfg["heads"]), int(cfg["kv_heads"])
        self.dim, self.vdim = int(cfg["dim"]), int(cfg["vdim"])
        if self.heads % self.kv_heads:
            raise ValueError("attention: heads must be a multiple of kv_heads")
        rot = cfg.get("rot") or {}
        self.rot_dims = int(rot.get("dims", 0))
        if self.rot_dims > self.dim or self.rot_dims % 2:
            raise ValueError("attention: rot.dims must be even and at most dim")
        base = float(rot.get("base", 10000.0))
        f = [base ** (-2.0 * i / self.rot_dims) for i in range(self.rot_dims // 2)] or [0.0]
        dev = w["q"].device
        self.inv_freq = torch.tensor(f, dtype=torch.float64).to(torch.float32).to(dev)
        self.scale, self.softcap = float(cfg["scale"]), float(cfg.get("softcap") or 0.0)
        self.window = int((cfg.get("mask") or {}).get("size", 0))
        self.eps, self.act_dtype, self.kv_dtype = eps, act_dtype, kv_dtype
        self._in = [w["q"], w["k"], w["v"], w["g"]]
        self._in_b = [w.get("q.b"), w.get("k.b"), w.get("v.b"), w.get("g.b")]
        self.talk = w["talk"].to(torch.float32).contiguous() if "talk" in w else None
        self.sink_kind = sink
        self.sink = w["sink"].contiguous() if sink == "learned" else None
        self.o = Projection(w["o"], tensor_cores)
        self.o_bias = w["o.b"].contiguous() if "o.b" in w else None

    def input_weights(self):
        return self._in

    def input_biases(self):
        return self._in_b

    def cache_spec(self):
        return {"pages": (self.kv_heads, self.dim, self.vdim), "states": {}, "kv_dtype": self.kv_dtype}

    def forward(self, parts, batch, cache, form: Optional[str] = None):
        q, k, v, g = parts
        ops.rope_kv_write(batch, q, k, v, self.inv_freq, cache.k_pool, cache.v_pool, heads=self.heads, kv_heads=self.kv_heads, dim=self.dim,
                          vdim=self.vdim, rot_dims=self.rot_dims)
        a = ops.talk_attn(batch, q, cache.k_pool, cache.v_pool, heads=self.heads, kv_heads=self.kv_heads, dim=self.dim, vdim=self.vdim,
                          scale=self.scale, softcap=self.softcap, talk=self.talk, window=self.window, sink=self.sink,
                          zero_sink=self.sink_kind == "zero", gate=g, gate_per_channel=True, out_dtype=self.act_dtype, form=form)
        return self.o(a, bias=self.o_bias)


class DenseMLP:
    """W_down act(W_up h). With `x_residual` the down projection adds into the fp32 residual in its epilogue; without, it
    returns the fp32 result (models that norm a sublayer's OUTPUT)."""

    def __init__(self, w: Dict[str, torch.Tensor], act_dtype: torch.dtype, tensor_cores: bool, act: str = "relu2"):
        self.up, self.down = Projection(w["up"], tensor_cores), Projection(w["down"], tensor_cores)
        self.act_dtype, self.act = act_dtype, act

    def forward(self, h: torch.Tensor, x_residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        u = self.up(h, act=self.act, out_dtype=self.act_dtype)   # activation on the fp32 accumulator in the epilogue, rounded once
        if x_residual is None:
            return self.down(u)
        return self.down(u, addend=x_residual, out=x_residual)


class ReluSquaredMLP(DenseMLP):
    """W_down relu(W_up h)^2."""

    def __init__(self, w: Dict[str, torch.Tensor], act_dtype: torch.dtype, tensor_cores: bool):
        super().__init__(w, act_dtype, tensor_cores, act="relu2")


class PolyNormMLP:
    """W_down act(W_up h) with act = a N(z) + b N(z^2) + c N(z^3) + e over each token's hidden vector z (powers element by element,
    N(u) = u / sqrt(mean(u^2) + eps)); the four numbers are the tensor `act`. The up projection's fp32 result feeds the activation,
    which is rounded once for the down projection."""

    def __init__(self, w: Dict[str, torch.Tensor], eps: float, act_dtype: torch.dtype, tensor_cores: bool):
        self.up, self.down = Projection(w["up"], tensor_cores), Projection(w["down"], tensor_cores)
        self.coef = tuple(float(v) for v in w["act"].to(torch.float32).cpu().tolist())
        if len(self.coef) != 4:
            raise ValueError("PolyNorm: the activation holds four numbers")
        self.eps, self.act_dtype = eps, act_dtype

    def forward(self, h: torch.Tensor, x_residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        u = ops.poly_norm(self.up(h), self.coef, eps=self.eps, out_dtype=self.act_dtype)
        if x_residual is None:
            return self.down(u)
        return self.down(u, addend=x_residual, out=x_residual)


class MoEFeedForward:
    """Mixture of experts with an optional shared expert that runs for every token. Router logits (and the shared gate) are one
    product with fp32 accumulation and an fp32 result (its input is the layer input as the experts read it: bf16-rounded when the
    model's projections are); scores, selection and weights are fp32.

    Router (`router`): "sigmoid" scores or the "softmax" over all experts; with `groups` = (count, keep) only members of the `keep`
    best of `count` runs of neighbouring experts are eligible; the `top` largest eligible scores are kept and, with `normalize`,
    divided by their sum; times `route_scale`.
    Expert (`form`): "plain" = W_down act(W_up h); "glu" = W_down (g sigmoid(alpha g) (u + 1)) with g = min(W_gate h, limit),
    u = clamp(W_up h, +-limit) (the shared expert with `shared_limit`). The shared expert is weighted by sigmoid(w_sg . h) when the
    weights hold `shared.sg`, by 1 otherwise.

    Two exact forms of the same sum. Single tokens and short steps (also every CUDA-graph-captured step: no host decision)
    run ALL experts as two products over the concatenated experts, the hidden activations multiplied by each token's routing
    weight (0 for the experts it did not choose) in between: the weights are read once, as a decode step would anyway.
    Prompt-sized steps sort the (token, choice) pairs by expert on the device, gather the rows, run each expert's two products
    on its own rows, and combine per token in choice order (no atomics, so the result does not depend on the batch). The sorted
    form costs two launches per expert and one host read of the experts' row counts, the all-experts form experts / top times
    the multiply-adds: a step of at least `sorted_min_rows` rows takes the sorted form when its estimated time is the smaller one
    (`force_sorted` skips the estimate)."""

    TC_RATE, FMA_RATE = 1.0e15, 2.0e13   # multiply-add rates the estimate assumes for bf16 tensor-core and fp32 FMA products (FLOP/s)
    LAUNCH_COST = 15e-6                   # host time of one product issued from Python (s): what bounds many small launches

    def __init__(self, w: Dict[str, torch.Tensor], experts: int, top: int, route_scale: float, act_dtype: torch.dtype, tensor_cores: bool,
                 act: str = "relu2", shared: bool = False, sorted_min_rows: int = 128, force_sorted: bool = False, router: str = "sigmoid",
                 groups: Optional[Tuple[int, int]] = None, normalize: bool = True, form: str = "plain", limit: float = 0.0,
                 shared_limit: float = 0.0, alpha: float = 1.702, router_logits: bool = True):
        self.experts, self.top, self.route_scale = int(experts), int(top), float(route_scale)
        self.act_dtype, self.act, self.sorted_min_rows, self.force_sorted = act_dtype, act, int(sorted_min_rows), bool(force_sorted)
        self.router_kind, self.normalize = router, bool(normalize)
        self.groups, self.keep_groups = (int(groups[0]), int(groups[1])) if groups and int(groups[0]) > 1 else (0, 0)
        if self.groups and (self.experts % self.groups or not 0 < self.keep_groups <= self.groups or self.top > self.keep_groups * (self.experts // self.groups)):
            raise ValueError("experts: the groups must divide the experts, and the kept groups hold at least `top` experts")
        if form not in ("plain", "glu"):
            raise ValueError(f"experts: unknown form {form!r}")
        self.glu, self.limit, self.shared_limit, self.alpha = form == "glu", float(limit), float(shared_limit), float(alpha)
        E = self.experts
        self.ff = w["e0.up"].shape[0]
        hid = (lambda pre: torch.cat([w[pre + "gate"], w[pre + "up"]], 0)) if self.glu else (lambda pre: w[pre + "up"])
        ups = [hid(f"e{e}.") for e in range(E)]
        downs = [w[f"e{e}.down"] for e in range(E)]
        self.shared_ff = 0
        self.shared_gated = shared and "shared.sg" in w
        rt = [w["router"]]
        if shared:
            self.shared_ff = w["shared.up"].shape[0]
            ups.append(hid("shared."))
            downs.append(w["shared.down"])
            if self.shared_gated:
                rt.append(w["shared.sg"].reshape(1, -1))
        up_all = torch.cat(ups, 0).contiguous()        # [E ff + S, W]  (glu: [E 2 ff + 2 S, W], per expert [gate | up])
        down_all = torch.cat(downs, 1).contiguous()    # [W, E ff + S]
        self.up_all, self.down_all = Projection(up_all, tensor_cores), Projection(down_all, tensor_cores)
        # the router's rows (+ the shared gate's); a layer that packs them into its input projection hands the logits to forward()
        self.router_weight = torch.cat(rt, 0).contiguous()    # [E (+ 1), W]
        self.router = Projection(self.router_weight, tensor_cores) if router_logits else None
        f, fu = self.ff, self.ff * (2 if self.glu else 1)
        self.up_e = [Projection(up_all[e * fu:(e + 1) * fu], tensor_cores) for e in range(E)]
        self.down_e = [Projection(down_all[:, e * f:(e + 1) * f], tensor_cores) for e in range(E)]
        if shared:
            self.up_s = Projection(up_all[E * fu:], tensor_cores)
            self.down_s = Projection(down_all[:, E * f:], tensor_cores)

    def _sorted_is_faster(self, rows: int) -> bool:
        width = self.down_all.out_features
        rate = self.TC_RATE if self.up_all.tensor_cores and self.act_dtype == torch.bfloat16 else self.FMA_RATE
        per_choice = (6.0 if self.glu else 4.0) * rows * self.ff * width / rate   # up (+ gate) + down multiply-adds of one expert-sized slice over all rows
        moved = 3.0 * rows * self.top * width * 4 / 2.0e12   # gather, per-pair results, combine
        return self.top * per_choice + 2 * self.experts * self.LAUNCH_COST + moved < self.experts * per_choice

    def _hidden(self, proj: Projection, x: torch.Tensor, dense: Optional[torch.Tensor], experts: int, shared_ff: int, sg, wide: bool) -> torch.Tensor:
        """The activated (and, with `dense`, weighted) hidden rows of `experts` experts and / or the shared expert, in the activation dtype."""
        if self.glu:
            u = proj(x)   # fp32 pre-activations: the clamps and the gate see the accumulator, rounded once after the activation
            return ops.moe_glu(u, dense, experts=experts, ff=self.ff, shared_ff=shared_ff, limit=self.limit, shared_limit=self.shared_limit,
                               alpha=self.alpha, out_dtype=self.act_dtype)
        u = proj(x, act=self.act, out_dtype=self.act_dtype if wide else torch.float32)
        if dense is None and sg is None:
            return u if u.dtype == self.act_dtype else ops.unary(u, None, self.act_dtype)
        return ops.moe_scale(u, dense, experts=experts, ff=self.ff if experts else 1, shared_ff=shared_ff, shared_gate=sg, out_dtype=self.act_dtype,
                             out=u if wide else None)

    def forward(self, h: torch.Tensor, batch, logits: Optional[torch.Tensor] = None) -> torch.Tensor:
        """h: the layer input in the activation dtype; logits: the router's fp32 logits (and the shared gate's) when the caller has them
        already. Returns fp32 [rows, width]."""
        E, rows = self.experts, h.shape[0]
        z = logits if logits is not None else self.router(h)
        sorted_form = batch.max_new > 1 and rows >= self.sorted_min_rows and (self.force_sorted or self._sorted_is_faster(rows))
        idx, wt, dense = ops.moe_route(z, E, self.top, self.route_scale, dense=not sorted_form, kind=self.router_kind, groups=self.groups,
                                       keep_groups=self.keep_groups, normalize=self.normalize)
        sg = z[:, E:E + 1] if self.shared_gated else None
        if not sorted_form:
            # few rows: fp32 hidden activations, weighted, rounded once. Prompt-sized steps write them in the activation dtype from
            # the product's epilogue and weight them in place (half the bytes of the step's largest tensor, one more rounding)
            wide = rows > 32 and self.act_dtype != torch.float32
            return self.down_all(self._hidden(self.up_all, h, dense, E, self.shared_ff, sg, wide))
        counts, offsets, perm, inv = ops.moe_sort(idx, E)
        xg = ops.moe_gather(h, perm, self.top, self.act_dtype)
        off = offsets.cpu().tolist()   # the one host decision of a prompt step: how many rows each expert got
        part = torch.empty((rows * self.top, self.down_all.out_features), device=h.device, dtype=torch.float32)
        for e in range(E):
            a, b = off[e], off[e + 1]
            if b > a:
                self.down_e[e](self._hidden(self.up_e[e], xg[a:b], None, 1, 0, None, True), out=part[a:b])
        ys = None
        if self.shared_ff:
            ys = self.down_s(self._hidden(self.up_s, h, None, 0, self.shared_ff, sg, False))
        return ops.moe_combine(part, inv, wt, addend=ys)
