"""Each Fubinex mechanism alone on the GPU against its float64 statement in oracle/fubinex_oracle.py: the grouped norm with a
full-row weight, the polynomial activation, both rotation layouts with RMS division and scales (into pages and packed), block-local
attention as an op (edges, a far key that stands out, many heads per key head) and as a mixer, gated linear attention and retention
as ops and mixers, latent attention with its query latent and stretched frequencies. Packed batches mix sequences that start,
continue and advance by one token, over shuffled pages and slots."""
import math

import pytest
import torch

from oracle import fubinex_oracle as O
from tests import fubinex_util as U
from tests import hybrid_util as HU

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _gen(seed):
    return torch.Generator().manual_seed(seed)


@pytest.mark.parametrize("groups,width,dtype", [(1, 40, torch.float32), (5, 40, torch.float32), (3, 1536, torch.float32), (2, 96, torch.bfloat16), (7, 4200, torch.float32)])
def test_grouped_norm_with_a_weight_over_the_whole_row(groups, width, dtype):
    from vyomai_b200 import ops
    g = _gen(0)
    x = torch.randn(9, width, generator=g) * 3.0
    w = (1.0 + 0.3 * torch.randn(width, generator=g)).to(torch.bfloat16)
    got = ops.rms_norm(x.to(DEV), w.to(DEV), eps=1e-3, w_mode="plain", groups=groups, w_full=True, out_dtype=dtype).float().cpu()
    want = O.grouped_norm(x.double(), w.double(), groups, 1e-3)
    assert HU.rel_err(got, want) < (1e-5 if dtype == torch.float32 else 1e-2)
    # accumulate into an fp32 residual with a bf16 copy, rows picked by index
    idx = torch.tensor([4, 0, 8], dtype=torch.int32, device=DEV)
    got = ops.rms_norm(x.to(DEV), w.to(DEV), eps=1e-3, w_mode="plain", groups=groups, w_full=True, row_index=idx).cpu()
    assert HU.rel_err(got, want[[4, 0, 8]]) < 1e-5


@pytest.mark.parametrize("act", ["silu", "sigmoid", None])
def test_norm_gate_activations(act):
    from vyomai_b200 import ops
    g = _gen(1)
    x, gate = torch.randn(6, 30, generator=g), torch.randn(6, 30, generator=g)
    got = ops.rms_norm(x.to(DEV), None, eps=1e-5, groups=3, gate=gate.to(DEV), gate_act=act, coef=0.7).cpu()
    f = {"silu": torch.nn.functional.silu, "sigmoid": torch.sigmoid, None: lambda t: t}[act]
    want = 0.7 * O.rms(x.double().view(6, 3, 10), 1e-5).reshape(6, 30) * f(gate.double())
    assert HU.rel_err(got, want) < 1e-5


@pytest.mark.parametrize("width,dtype", [(7, torch.float32), (44, torch.float32), (1000, torch.bfloat16), (1500, torch.float32), (9000, torch.float32)])
def test_polynomial_activation(width, dtype):
    from vyomai_b200 import ops
    g = _gen(2)
    z = torch.randn(5, width, generator=g) * 2.0
    z[0] *= 0.0      # a zero row: only eps holds the roots up
    coef = (0.8, -0.45, 0.3, 0.15)
    got = ops.poly_norm(z.to(DEV), coef, eps=1e-6, out_dtype=dtype).float().cpu()
    want = O.poly_norm(z.double(), coef, 1e-6)
    assert HU.rel_err(got, want) < (2e-5 if dtype == torch.float32 else 1e-2)
    assert float((got[0] - 0.15).abs().max()) < (1e-6 if dtype == torch.float32 else 1e-2)


def _freq(rot):
    f, m = O.frequencies(rot)
    return f.float().to(DEV), m


@pytest.mark.parametrize("layout,rot_dims,unit", [("half", 6, True), ("half", 10, False), ("pairs", 4, True), ("half", 0, True)])
def test_rotation_into_pages_with_rms_division(layout, rot_dims, unit):
    from vyomai_b200 import ops
    H, G, d, dv, bs = 4, 2, 10, 6, 4
    lengths, pos0 = [9, 1, 5], [0, 3000, 3]
    batch, table, _, n_blocks, _ = HU.shuffled_batch(lengths, pos0, bs, DEV)
    g = _gen(3)
    n = sum(lengths)
    q, k, v = torch.randn(n, H * d, generator=g), torch.randn(n, G * d + 3, generator=g), torch.randn(n, G * dv, generator=g)
    rot = {"base": 40.0, "dims": rot_dims, "scaling": {"factor": 4.0, "original": 8, "fast": 2.0, "slow": 0.5}} if rot_dims == 10 else {"base": 40.0, "dims": rot_dims}
    f, m = _freq(rot) if rot_dims else (torch.zeros(1, device=DEV), 1.0)
    kp = torch.full((n_blocks, bs, G, d), 7.0, device=DEV)
    vp = torch.full((n_blocks, bs, G, dv), 7.0, device=DEV)
    qd = q.to(DEV)
    ops.rope_kv_write(batch, qd, k.to(DEV)[:, :G * d], v.to(DEV), f, kp, vp, heads=H, kv_heads=G, dim=d, vdim=dv, rot_dims=rot_dims, layout=layout,
                      rot_scale=m, unit_rms=unit, eps=1e-4, q_scale=1.0, k_scale=0.5)
    at = 0
    for s, (ln, p) in enumerate(zip(lengths, pos0)):
        qs, ks = q[at:at + ln].double().view(ln, H, d), k[at:at + ln, :G * d].double().view(ln, G, d)
        if rot_dims:
            qs, ks = O.rotate(qs, rot, layout, pos0=p), O.rotate(ks, rot, layout, pos0=p)
        if unit:
            qs, ks = O.rms(qs, 1e-4), O.rms(ks, 1e-4)
        tol = 2e-3 if p > 1000 else 1e-5     # fp32 angles: 3000 * 2^-24 rad
        assert float((qd[at:at + ln].cpu().double().view(ln, H, d) - qs).abs().max()) < tol
        for i in range(ln):
            blk, off = table[s][(p + i) // bs], (p + i) % bs
            assert float((kp[blk, off].cpu().double() - 0.5 * ks[i]).abs().max()) < tol
            assert torch.equal(vp[blk, off].cpu().view(-1), v[at + i])
        at += ln
    assert int((kp == 7.0).all(-1).all(-1).sum()) == n_blocks * bs - n   # nothing else was written


def test_rotation_of_packed_rows_without_pages():
    from vyomai_b200 import ops
    H, d = 3, 8
    lengths, pos0 = [4, 1, 6], [0, 77, 12]
    batch, *_ = HU.shuffled_batch(lengths, pos0, 4, DEV)
    g = _gen(4)
    n = sum(lengths)
    P = torch.randn(n, 2 * H * d + 8, generator=g).to(DEV)
    ref = P.cpu().double()
    q, k = P[:, :H * d], P[:, H * d + 8:]
    rot = {"base": 30.0, "dims": 4}
    f, _ = _freq(rot)
    ops.rope_kv_write(batch, q, k, None, f, None, None, heads=H, kv_heads=H, dim=d, vdim=0, rot_dims=4, layout="half", k_scale=d ** -0.5, k_out=k)
    at = 0
    for ln, p in zip(lengths, pos0):
        for src, dst, sc in ((ref[at:at + ln, :H * d], q[at:at + ln], 1.0), (ref[at:at + ln, H * d + 8:], k[at:at + ln], d ** -0.5)):
            want = O.rotate(src.view(ln, H, d), rot, "half", pos0=p) * sc
            assert float((dst.cpu().double().view(ln, H, d) - want).abs().max()) < 1e-5
        at += ln
    assert torch.equal(P[:, H * d:H * d + 8].cpu().double(), ref[:, H * d:H * d + 8])


def _attend(q, k, v, mask, scale):
    """q [T, H, d], k [T, G, d], v [T, G, dv] float64 -> [T, H * dv] by the definition."""
    H, G = q.shape[1], k.shape[1]
    k, v = k.repeat_interleave(H // G, 1), v.repeat_interleave(H // G, 1)
    s = torch.einsum("thd,jhd->htj", q, k) * scale
    return O.softmax_attention(s, v.transpose(0, 1), mask).transpose(0, 1).reshape(q.shape[0], -1)


@pytest.mark.parametrize("H,G", [(4, 2), (8, 1), (16, 2), (3, 3)])
@pytest.mark.parametrize("chunk,bs", [(7, 4), (16, 16), (64, 16), (100, 8), (1, 4)])
def test_block_local_attention_over_pages(H, G, chunk, bs):
    """Three sequences in one step: a whole prompt of several blocks, a portion that starts inside a block, a single token at a block's
    last position. In the prompt one key per block is made to stand out, the block's first (just inside for every later query of the
    block, just outside for the block before)."""
    from vyomai_b200 import ops
    d, dv, scale = 8, 6, 0.6
    T = [3 * chunk + 2, 2 * chunk + 3, 2 * chunk] if chunk > 1 else [9, 5, 4]
    new = [T[0], max(T[1] - (chunk // 2 + 1), 1), 1]
    g = _gen(5)
    qs = [torch.randn(t, H, d, generator=g).double() for t in T]
    ks = [torch.randn(t, G, d, generator=g).double() for t in T]
    vs = [torch.randn(t, G, dv, generator=g).double() for t in T]
    for j in range(0, T[0], chunk):     # the block's first key: four times as long, with its own value
        ks[0][j] *= 4.0
        vs[0][j] += 5.0
    pos0 = [t - n for t, n in zip(T, new)]
    batch, table, _, n_blocks, _ = HU.shuffled_batch(new, pos0, bs, DEV, seed=chunk)
    kp = torch.zeros((n_blocks, bs, G, d), device=DEV)
    vp = torch.zeros((n_blocks, bs, G, dv), device=DEV)
    for s in range(3):
        for p in range(T[s]):
            blk, off = table[s][p // bs], p % bs
            kp[blk, off], vp[blk, off] = ks[s][p].float().to(DEV), vs[s][p].float().to(DEV)
    q = torch.cat([qs[s][pos0[s]:].reshape(new[s], H * d) for s in range(3)]).float().to(DEV)
    got = ops.window_attn(batch, q, kp, vp, heads=H, kv_heads=G, dim=d, vdim=dv, scale=scale, window=0, keep_first=0, chunk=chunk, out_scale=0.8).cpu()
    want = torch.cat([0.8 * _attend(qs[s], ks[s], vs[s], O.chunk_mask(T[s], chunk), scale)[pos0[s]:] for s in range(3)])
    assert HU.rel_err(got, want) < 2e-5


def _views(model_like_specs, n_blocks, bs, n_slots):
    from vyomai_b200.paged import LayerCacheView
    view = LayerCacheView()
    spec = model_like_specs
    if spec["pages"]:
        G, dk, dv = spec["pages"]
        view.k_pool = torch.zeros((n_blocks, bs, G, dk), device=DEV)
        if dv:
            view.v_pool = torch.zeros((n_blocks, bs, G, dv), device=DEV)
    for name, shape in spec["states"].items():
        view.states[name] = torch.full((n_slots,) + tuple(shape), 3.0, device=DEV)   # what an earlier owner of the slot left
    return view


def _run_mixer(mix, h, steps, bs=4, view=None, **kw):
    """Feeds h [T, width] (one sequence) to the mixer in portions through real pages and a state slot; returns [T, width]."""
    from vyomai_b200 import ops
    T = h.shape[0]
    n_blocks = (T + bs - 1) // bs + 2
    order = torch.randperm(n_blocks, generator=_gen(5)).tolist()
    view = view or _views(mix.cache_spec(), n_blocks, bs, 3)
    t = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)  # noqa: E731
    outs, at = [], 0
    for n in steps:
        batch = ops.PackedBatch(t([0, n]), t([at]), t([2]), n, t(order).view(1, -1), bs, all_start=at == 0)
        x = h[at:at + n].to(DEV)
        parts = [ops.linear_plain(x, wt.to(DEV).float()) for wt in mix.input_weights()]
        outs.append(mix.forward(parts, batch, view, **kw).float().cpu())
        at += n
    return torch.cat(outs), view


def _weights(shapes, seed, dtype=torch.float32):
    g = _gen(seed)
    w = {}
    for k, s in shapes.items():
        if k.endswith("norm"):
            t = 1.0 + 0.2 * torch.randn(s, generator=g)
        elif k == "a2.b":
            t = 0.5 + 2.0 * torch.rand(s, generator=g)
        else:
            t = torch.randn(s, generator=g) / math.sqrt(s[-1])
        w[k] = t.to(torch.bfloat16)
    return {k: v.to(DEV, dtype) for k, v in w.items()}, {k: v.double() for k, v in w.items()}


STEPS = [[37], [20, 1, 1, 1, 14], [2] * 18 + [1], [16, 21], [1] * 37]


@pytest.mark.parametrize("steps", STEPS)
def test_block_local_attention_mixer(steps):
    from vyomai_b200.layers.mixers import RotaryAttention
    m = U.left(heads=4, kv_heads=2, dim=12, vdim=10, chunk=9, rot_dims=6)
    w, W = _weights({"q": (48, 40), "k": (24, 40), "v": (20, 40), "o": (40, 40)}, 6)
    mix = RotaryAttention(m, w, 1e-5, torch.float32, True)
    h = torch.randn(37, 40, generator=_gen(7))
    got, _ = _run_mixer(mix, h, steps, out_scale=0.6)
    assert HU.rel_err(got, 0.6 * O.chunked_attention(h.double(), W, m, 1e-5)) < 3e-5


@pytest.mark.parametrize("steps", STEPS)
@pytest.mark.parametrize("dim,vdim,tau", [(8, 6, 4.0), (40, 33, 1.0), (5, 70, 16.0)])
def test_gated_linear_attention_mixer(steps, dim, vdim, tau):
    from vyomai_b200.layers.mixers import GatedLinearAttention
    H = 3
    m = U.right(heads=H, dim=dim, vdim=vdim, tau=tau)
    w, W = _weights({"q": (H * dim, 40), "k": (H * dim, 40), "v": (H * vdim, 40), "g": (H * vdim, 40), "a1": (5, 40), "a2": (H * dim, 5), "a2.b": (H * dim,),
                     "norm": (vdim,), "o": (40, H * vdim)}, 8)
    mix = GatedLinearAttention(m, w, 1e-5, torch.float32, True)
    h = torch.randn(37, 40, generator=_gen(9))
    got, view = _run_mixer(mix, h, steps, out_scale=1.3)
    assert HU.rel_err(got, 1.3 * O.gated_linear_attention(h.double(), W, m, 1e-5)) < 3e-5
    assert float((view.states["S"][:2] - 3.0).abs().max()) == 0.0    # other sequences' slots untouched


def test_gated_linear_attention_decays_per_channel_and_forgets():
    """Decay logits of -30 on one channel and +30 on another: the first forgets at once (only the current token's key counts), the
    second never; a logit of 0 halves at tau 1."""
    from vyomai_b200 import ops
    T, d, dv = 12, 3, 2
    g = _gen(10)
    q, k, v = torch.randn(T, d, generator=g), torch.randn(T, d, generator=g), torch.randn(T, dv, generator=g)
    a = torch.tensor([[-30.0, 30.0, 0.0]]).repeat(T, 1)
    batch, *_ = HU.shuffled_batch([T], [0], 4, DEV)
    state = torch.zeros((4, 1, d, dv), device=DEV)
    got = ops.gated_linear_attn(batch, q.to(DEV), k.to(DEV), v.to(DEV), a.to(DEV), state, heads=1, dim=d, vdim=dv, tau=1.0).cpu().double()
    decay = torch.sigmoid(a.double()).view(T, 1, d)
    want = O.decayed_recurrence(q.double().view(T, 1, d), k.double().view(T, 1, d), v.double().view(T, 1, dv), decay).view(T, dv)
    assert HU.rel_err(got, want) < 1e-5
    by_hand = sum(q[-1, c].double() * sum(w(T - 1 - j) * k[j, c].double() * v[j].double() for j in range(T))
                  for c, w in ((0, lambda n: 1.0 if n == 0 else 0.0), (1, lambda n: 1.0), (2, lambda n: 0.5 ** n)))
    assert HU.rel_err(got[-1:], by_hand[None]) < 1e-5


@pytest.mark.parametrize("steps", STEPS)
@pytest.mark.parametrize("dim,vdim,rot_dims", [(8, 10, 4), (32, 40, 32), (6, 70, 0)])
def test_retention_mixer(steps, dim, vdim, rot_dims):
    from vyomai_b200.layers.mixers import RetentionMixer
    H = 3
    m = U.retention(heads=H, dim=dim, vdim=vdim, rot_dims=rot_dims)
    w, W = _weights({"q": (H * dim, 40), "k": (H * dim, 40), "v": (H * vdim, 40), "g": (H * vdim, 40), "o": (40, H * vdim)}, 11)
    mix = RetentionMixer(m, w, 1e-5, torch.float32, True)
    h = torch.randn(37, 40, generator=_gen(12))
    got, _ = _run_mixer(mix, h, steps)
    assert HU.rel_err(got, O.retention(h.double(), W, m, 1e-5)) < 3e-5


@pytest.mark.parametrize("steps", STEPS)
@pytest.mark.parametrize("scaling", [None, U.STRETCH])
def test_latent_attention_with_a_query_latent(steps, scaling):
    from vyomai_b200.layers.mixers import LatentAttention
    m = U.latent(heads=3, dim=8, rot_dim=6, vdim=10, rank=20, q_rank=12, scale=0.4, scaling=scaling)
    w, W = _weights({"dq": (12, 40), "dq.norm": (12,), "uq": (3 * 14, 12), "dkv": (26, 40), "dkv.norm": (20,), "uk": (24, 20), "uv": (30, 20), "o": (40, 30)}, 13)
    mix = LatentAttention(m, w, 1e-5, torch.float32, True)
    h = torch.randn(37, 40, generator=_gen(14))
    c, kr = O.latent_kv(h.double(), W, m, 1e-5)
    got, view = _run_mixer(mix, h, steps)
    assert HU.rel_err(got, O.latent_attention(h.double(), W, m, c, kr, 1e-5)) < 3e-5
    # a second mixer over the first one's rows, with its own head count and queries
    m2 = U.latent(heads=2, dim=5, rot_dim=6, vdim=7, rank=20, q_rank=9, scale=0.3, scaling=scaling, kv_from=0)
    w2, W2 = _weights({"dq": (9, 40), "dq.norm": (9,), "uq": (2 * 11, 9), "uk": (10, 20), "uv": (14, 20), "o": (40, 14)}, 15)
    mix2 = LatentAttention(m2, w2, 1e-5, torch.float32, True, shared_from=0)
    got2, _ = _run_mixer(mix2, h, [37] if steps == [37] else [36, 1], view=view) if steps in ([37], [1] * 37) else (None, None)
    if got2 is not None:
        assert HU.rel_err(got2, O.latent_attention(h.double(), W2, m2, c, kr, 1e-5)) < 3e-5


def test_stretched_frequencies_follow_the_ramp():
    """The table the mixers hand to the kernels against the definition, for a block where every branch comes up: fast pairs untouched,
    slow pairs divided by the factor, a blend between, and the factor on cos / sin."""
    from vyomai_b200.layers.mixers import rotary_frequencies
    rot = {"base": 10000.0, "dims": 32, "scaling": {"factor": 8.0, "original": 64, "fast": 16.0, "slow": 1.0}}
    f, m = rotary_frequencies(rot, 32, DEV)
    want, wm = O.frequencies(rot)
    assert abs(m - wm) < 1e-12 and abs(m - (0.1 * math.log(8.0) + 1.0)) < 1e-12
    assert float((f.cpu().double() - want).abs().max() / want.max()) < 1e-7
    plain = torch.tensor([10000.0 ** (-2.0 * i / 32) for i in range(16)], dtype=torch.float64)
    ratio = want / plain
    assert float(ratio[0]) == 1.0 and abs(float(ratio[-1]) - 1.0 / 8.0) < 1e-12 and bool(((ratio > 0.13) & (ratio < 0.99)).any())
