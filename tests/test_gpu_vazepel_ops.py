"""Each Vazepel mechanism alone on the GPU against its float64 statement in oracle/vazepel_oracle.py: layer norm, the layer's closing
kernel (gated residual, stack of results, weighted sum, fused norm), the gated experts' activation, the softmax router with groups,
rotation + page write, the score-exchanging attention in both of its forms, and the mixture of experts in both of its forms. Packed
batches mix sequences that start, continue and advance by one token, over shuffled pages."""
import math

import pytest
import torch

from oracle import vazepel_oracle as O
from tests import hybrid_util as HU
from tests import vazepel_util as U

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _g(seed):
    return torch.Generator().manual_seed(seed)


@pytest.mark.parametrize("width", [1, 37, 128, 700])
def test_layer_norm_rows(width):
    from vyomai_b200 import ops
    g = _g(width)
    x = torch.randn(9, width + 3, generator=g) * 3 + 50.0   # a mean far from zero: one-pass variance formulas lose digits here
    w, b = torch.randn(width, generator=g), torch.randn(width, generator=g)
    want = O.layer_norm(x[:, :width].double(), w.double(), b.double(), 1e-3)
    got = ops.layer_norm(x.to(DEV)[:, :width], w.to(DEV), b.to(DEV), eps=1e-3)
    assert float((got.cpu().double() - want).abs().max()) < 2e-4
    idx = torch.tensor([8, 0, 0, 3], dtype=torch.int32, device=DEV)
    got = ops.layer_norm(x.to(DEV)[:, :width], w.to(DEV), None, eps=1e-3, row_index=idx, out_dtype=torch.bfloat16)
    assert got.dtype == torch.bfloat16 and float((got.cpu().double() - (want - b.double())[[8, 0, 0, 3]]).abs().max()) < 3e-2


@pytest.mark.parametrize("second,gated,depth,fused", [(True, True, 4, True), (False, True, 1, False), (True, False, 2, True), (True, True, 0, True)])
def test_layer_close(second, gated, depth, fused):
    """depth 0 = no stack: the plain gated residual."""
    from vyomai_b200 import ops
    g = _g(3)
    rows, width = 11, 45
    x, y1, g1, y2, g2 = (torch.randn(rows, width, generator=g) for _ in range(5))
    stack = torch.randn(max(depth, 1) + 1, rows, width, generator=g)
    coef = torch.randn(max(depth, 1), generator=g)
    nw, nb = torch.randn(width, generator=g), torch.randn(width, generator=g)
    r = x.double() + y1.double() * (torch.sigmoid(g1.double()) if gated else 1.0)
    if second:
        r = r + y2.double() * (torch.sigmoid(g2.double()) if gated else 1.0)
    mixed = r
    if depth:
        mixed = sum(coef[j].double() * stack[j].double() for j in range(depth - 1)) + coef[depth - 1].double() * r
    sd = stack.to(DEV)
    before = sd.clone()
    out, h = torch.zeros(rows, width, device=DEV), torch.zeros(rows, width, device=DEV)
    ops.depth_mix(x.to(DEV), y1.to(DEV), g1.to(DEV) if gated else None, y2.to(DEV) if second else None, g2.to(DEV) if second and gated else None,
                  stack=sd if depth else None, depth=depth, coef=coef.to(DEV) if depth else None, mixed=out, norm_weight=nw.to(DEV) if fused else None,
                  norm_bias=nb.to(DEV) if fused else None, eps=1e-5, norm_out=h if fused else None)
    assert float((out.cpu().double() - mixed).abs().max()) < 1e-5
    if depth:
        assert float((sd[depth - 1].cpu().double() - r).abs().max()) < 1e-5
        keep = [j for j in range(sd.shape[0]) if j != depth - 1]
        assert torch.equal(sd[keep], before[keep])   # the other slices are read, not written
    if fused:
        assert float((h.cpu().double() - O.layer_norm(mixed, nw.double(), nb.double(), 1e-5)).abs().max()) < 1e-4


def test_layer_close_in_place():
    from vyomai_b200 import ops
    g = _g(4)
    x, y1 = torch.randn(5, 33, generator=g), torch.randn(5, 33, generator=g)
    xd = x.to(DEV)
    ops.depth_mix(xd, y1.to(DEV), None, None, None, mixed=xd)
    assert float((xd.cpu() - (x + y1)).abs().max()) < 1e-6


@pytest.mark.parametrize("experts,ff,shared_ff", [(3, 5, 7), (1, 8, 0), (0, 1, 6)])
def test_gated_experts_activation(experts, ff, shared_ff):
    from vyomai_b200 import ops
    g = _g(5)
    rows = 6
    h = torch.randn(rows, 2 * (experts * ff + shared_ff), generator=g) * 3
    dense = torch.rand(rows, max(experts, 1), generator=g)
    dense[dense < 0.4] = 0.0
    got = ops.moe_glu(h.to(DEV), dense.to(DEV) if experts else None, experts=experts, ff=ff, shared_ff=shared_ff, limit=1.5, shared_limit=0.6,
                      out_dtype=torch.float32).cpu().double()
    hd = h.double()

    def act(gate, up, lim):
        gate, up = torch.clamp(gate, max=lim), torch.clamp(up, -lim, lim)
        return gate * torch.sigmoid(1.702 * gate) * (up + 1)
    for e in range(experts):
        o = e * 2 * ff
        want = act(hd[:, o:o + ff], hd[:, o + ff:o + 2 * ff], 1.5) * dense[:, e:e + 1].double()
        assert float((got[:, e * ff:(e + 1) * ff] - want).abs().max()) < 1e-5
    if shared_ff:
        o = experts * 2 * ff
        want = act(hd[:, o:o + shared_ff], hd[:, o + shared_ff:], 0.6)
        assert float((got[:, experts * ff:] - want).abs().max()) < 1e-5


@pytest.mark.parametrize("experts,top,groups,keep", [(12, 3, 4, 2), (8, 3, 4, 3), (6, 2, 1, 1), (6, 6, 3, 3), (5, 1, 5, 1), (40, 5, 8, 2)])
def test_softmax_router_with_groups(experts, top, groups, keep):
    from vyomai_b200 import ops
    z = torch.randn(70, experts + 2, generator=_g(experts)) * 2
    idx, wt, dense = ops.moe_route(z.to(DEV)[:, :experts], experts, top, 1.0, kind="softmax", groups=groups, keep_groups=keep, normalize=False)
    ri, rw = O.route(z[:, :experts].double(), top, groups, keep)
    assert torch.equal(idx.cpu().long(), ri)                                     # largest first, as topk orders them
    assert float((wt.cpu().double() - rw).abs().max()) < 1e-6
    want_dense = torch.zeros(70, experts, dtype=torch.float64).scatter_(1, ri, rw)
    assert float((dense.cpu().double() - want_dense).abs().max()) < 1e-6


def test_router_group_choice_beats_a_larger_score_outside():
    """The best single score sits in a group whose best... is still the best: so make the second-best EXPERT sit in a group that is not
    kept, and check that it is skipped for a smaller score inside a kept group."""
    from vyomai_b200 import ops
    # groups of 2: scores by expert: g0 = (9, 8), g1 = (7, 0), g2 = (6, 5); keep 1 group, top 2 -> experts 0 and 1; keep 2, top 3 -> 0, 1, 2
    z = torch.tensor([[9.0, 8.0, 7.0, 0.0, 6.0, 5.0]], device=DEV)
    idx, _, _ = ops.moe_route(z, 6, 2, 1.0, kind="softmax", groups=3, keep_groups=1, normalize=False)
    assert idx.cpu().tolist() == [[0, 1]]
    z = torch.tensor([[9.0, 0.0, 7.0, 6.5, 8.0, 1.0]], device=DEV)   # group bests 9, 7, 8: keep 2 -> groups 0 and 2; expert 2 (7.0) is out
    idx, _, _ = ops.moe_route(z, 6, 3, 1.0, kind="softmax", groups=3, keep_groups=2, normalize=False)
    assert idx.cpu().tolist() == [[0, 4, 5]]


def test_sigmoid_router_is_unchanged_by_the_new_options():
    from vyomai_b200 import ops
    z = torch.randn(20, 7, generator=_g(9))
    idx, wt, _ = ops.moe_route(z.to(DEV), 7, 3, 1.5)
    s = torch.sigmoid(z.double())
    v, i = s.topk(3, -1)
    assert torch.equal(idx.cpu().long(), i) and float((wt.cpu().double() - v / v.sum(-1, keepdim=True) * 1.5).abs().max()) < 1e-6


@pytest.mark.parametrize("rot_dims", [10, 4, 0])
def test_rotation_and_page_write(rot_dims):
    from vyomai_b200 import ops
    H, G, d, dv, bs = 4, 2, 10, 7, 4
    lengths, pos0 = [7, 1, 4], [0, 130, 9]
    batch, table, _, n_blocks, _ = HU.shuffled_batch(lengths, pos0, bs, DEV)
    g = _g(1)
    rows = sum(lengths)
    P = torch.randn(rows, H * d + G * d + G * dv + 5, generator=g)
    Pd = P.to(DEV)
    q, k, v = Pd[:, :H * d], Pd[:, H * d:H * d + G * d], Pd[:, H * d + G * d:H * d + G * d + G * dv]
    f = torch.tensor([50.0 ** (-2.0 * i / max(rot_dims, 2)) for i in range(max(rot_dims, 2) // 2)], dtype=torch.float64).float().to(DEV)
    kp = torch.full((n_blocks, bs, G, d), 7.0, device=DEV)
    vp = torch.full((n_blocks, bs, G, dv), 7.0, device=DEV)
    ops.rope_kv_write(batch, q, k, v, f, kp, vp, heads=H, kv_heads=G, dim=d, vdim=dv, rot_dims=rot_dims)
    at = 0
    for s, (n, p) in enumerate(zip(lengths, pos0)):
        sl = P[at:at + n].double()
        qw = O.rotate_pairs(sl[:, :H * d].reshape(n, H, d), 50.0, rot_dims, pos0=p)
        kw = O.rotate_pairs(sl[:, H * d:H * d + G * d].reshape(n, G, d), 50.0, rot_dims, pos0=p)
        assert float((q[at:at + n].cpu().double().view(n, H, d) - qw).abs().max()) < 3e-5
        for i in range(n):
            blk, off = table[s][(p + i) // bs], (p + i) % bs
            assert float((kp[blk, off].cpu().double() - kw[i]).abs().max()) < 3e-5
            assert torch.equal(vp[blk, off].cpu().view(-1), P[at + i, H * d + G * d:H * d + G * d + G * dv])
        at += n
    assert torch.equal(Pd[:, -5:].cpu(), P[:, -5:]) and int((kp == 7.0).sum()) == kp.numel() - rows * G * d


def _attn_oracle(q, k, v, talk, m, gate, window=0):
    """q [T, H, d], k [T, G, d], v [T, G, dv] already rotated -> [T, H * dv] after the gate."""
    T, H, G = q.shape[0], m["heads"], m["kv_heads"]
    per = H // G
    s = torch.stack([q[:, a] @ k[:, a // per].T for a in range(H)]) * m["scale"]
    if m["softcap"] > 0:   # the kernel's "no cap" value
        s = O.capped(s, m["softcap"])
    if talk is not None:
        s = O.mix_heads(s, talk)
    back = torch.arange(T)[:, None] - torch.arange(T)[None, :]
    p = O.plus_one_softmax(s, (back >= 0) & (back < window) if window else back >= 0)
    o = torch.stack([p[a] @ v[:, a // per] for a in range(H)], 1).reshape(T, -1)
    return o * torch.sigmoid(gate)


def _run_attn(m, q, k, v, talk, gate, steps, form, bs=4, window=0):
    """Feeds one sequence in portions through real (shuffled) pages with the chosen form of the kernel."""
    from vyomai_b200 import ops
    T, H, G, d, dv = q.shape[0], m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    n_blocks = (T + bs - 1) // bs + 2
    order = torch.randperm(n_blocks, generator=_g(5)).tolist()
    kp, vp = torch.zeros((n_blocks, bs, G, d), device=DEV), torch.zeros((n_blocks, bs, G, dv), device=DEV)
    t = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)  # noqa: E731
    outs, at = [], 0
    for n in steps:
        batch = ops.PackedBatch(t([0, n]), t([at]), t([0]), n, t(order).view(1, -1), bs)
        ops.kv_page_write(batch, k[at:at + n].reshape(n, -1).float().to(DEV), v[at:at + n].reshape(n, -1).float().to(DEV), kp, vp)
        outs.append(ops.talk_attn(batch, q[at:at + n].reshape(n, -1).float().to(DEV), kp, vp, heads=H, kv_heads=G, dim=d, vdim=dv, scale=m["scale"],
                                  softcap=m["softcap"], talk=None if talk is None else talk.float().to(DEV), zero_sink=True, window=window,
                                  gate=gate[at:at + n].float().to(DEV), gate_per_channel=True, form=form).cpu())
        at += n
    return torch.cat(outs)


@pytest.mark.parametrize("form", ["rows", "tiled"])
@pytest.mark.parametrize("shape", [dict(heads=6, kv_heads=3, dim=10, vdim=7), dict(heads=8, kv_heads=2, dim=32, vdim=24), dict(heads=3, kv_heads=1, dim=6, vdim=70),
                                   dict(heads=24, kv_heads=4, dim=12, vdim=72), dict(heads=5, kv_heads=5, dim=4, vdim=3), dict(heads=40, kv_heads=8, dim=8, vdim=6),
                                   dict(heads=16, kv_heads=4, dim=64, vdim=64), dict(heads=48, kv_heads=48, dim=64, vdim=8)])
@pytest.mark.parametrize("steps", [[75], [40, 1, 1, 33], [2] * 37 + [1]])
def test_score_exchanging_attention(form, shape, steps):
    """The last shape's key rows of all 48 key/value heads do not fit a 16-key tile: the tiled form refuses it (the automatic choice
    never takes it there) and the one-query form drops to 8 keys per tile."""
    from vyomai_b200._lib import VyomError
    m = U.attn(scale=0.4, softcap=3.0, **shape)
    g = _g(shape["heads"])
    T, H, G, d, dv = 75, m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q, k, v = torch.randn(T, H, d, generator=g), torch.randn(T, G, d, generator=g), torch.randn(T, G, dv, generator=g)
    talk = torch.eye(H) + torch.randn(H, H, generator=g) * 0.5
    gate = torch.randn(T, H * dv, generator=g)
    want = _attn_oracle(q.double(), k.double(), v.double(), talk.double(), m, gate.double())
    if form == "tiled" and H == 48:
        with pytest.raises(VyomError):
            _run_attn(m, q, k, v, talk, gate, steps, form)
        form = None
    got = _run_attn(m, q, k, v, talk, gate, steps, form)
    assert HU.rel_err(got, want) < 2e-5


@pytest.mark.parametrize("form", ["rows", "tiled"])
def test_a_far_key_among_hundreds_is_found(form):
    """One early key is made to stand out for the last query of ONE head, and the mixing matrix carries that score to another head only:
    the output of the receiving head must be that key's value, whichever form and however many tiles lie in between."""
    m = U.attn(heads=4, kv_heads=2, dim=8, vdim=5, scale=1.0, softcap=0.0)
    g = _g(11)
    T = 300
    q, k, v = torch.randn(T, 4, 8, generator=g) * 0.1, torch.randn(T, 2, 8, generator=g) * 0.1, torch.randn(T, 2, 5, generator=g)
    q[-1, 0] = 0.0
    q[-1, 0, 3] = 6.0
    k[17, 0] = 0.0
    k[17, 0, 3] = 5.0                       # head 0, last query, key 17: raw score 30
    talk = torch.eye(4)
    talk[0, 0] = 0.0                        # head 0 gives its score away ...
    talk[3, 0] = 1.0                        # ... to head 3 (key/value head 1)
    gate = torch.full((T, 20), 30.0)        # open gates
    got = _run_attn(m, q, k, v, talk, gate, [T], form)[-1].view(4, 5)
    assert float((got[3] - v[17, 1]).abs().max()) < 1e-4
    want = _attn_oracle(q.double(), k.double(), v.double(), talk.double(), m, gate.double())[-1].view(4, 5)
    assert float((got.double() - want).abs().max()) < 1e-4


@pytest.mark.parametrize("form", ["rows", "tiled"])
def test_the_extra_unit_in_the_denominator(form):
    """With very negative scores the weights sum to almost nothing (the unit dominates); with score 0 on a single visible key the
    weight is exactly one half."""
    from vyomai_b200 import ops
    m = U.attn(heads=2, kv_heads=1, dim=4, vdim=3, scale=1.0, softcap=0.0)
    T = 9
    q, k, v = torch.zeros(T, 2, 4), torch.zeros(T, 1, 4), torch.ones(T, 1, 3)
    gate = torch.full((T, 6), 30.0)
    got = _run_attn(m, q, k, v, None, gate, [T], form)
    for i in range(T):
        assert abs(float(got[i, 0]) - (i + 1) / (i + 2)) < 1e-5   # i + 1 keys of score 0 and the unit
    q[:, :, 0], k[:, :, 0] = 10.0, -10.0
    got = _run_attn(m, q, k, v, None, gate, [T], form)
    assert float(got.abs().max()) < 1e-30 or float(got.abs().max()) < 1e-20


@pytest.mark.parametrize("form", ["rows", "tiled"])
@pytest.mark.parametrize("window,steps", [(5, [60]), (16, [40, 1, 1, 18]), (33, [2] * 30), (64, [59, 1])])
def test_window_option_just_inside_and_just_outside(form, window, steps):
    """The kernel's optional sliding window (0 in Vazepel itself): against the oracle, and the key exactly `window` back does not reach
    the last query while the key `window - 1` back does; in prompts, portions and single tokens, with the edge at and off page and tile
    borders."""
    m = U.attn(heads=4, kv_heads=2, dim=8, vdim=5, scale=0.5, softcap=6.0)
    g = _g(window)
    T = 60
    q, k, v = torch.randn(T, 4, 8, generator=g), torch.randn(T, 2, 8, generator=g), torch.randn(T, 2, 5, generator=g)
    talk = torch.eye(4) + torch.randn(4, 4, generator=g) * 0.3
    gate = torch.randn(T, 20, generator=g)
    want = _attn_oracle(q.double(), k.double(), v.double(), talk.double(), m, gate.double(), window=window)
    got = _run_attn(m, q, k, v, talk, gate, steps, form, window=window)
    assert HU.rel_err(got, want) < 2e-5
    if window < T:
        for back, same in ((window, True), (window - 1, False)):
            k2, v2 = k.clone(), v.clone()
            k2[T - 1 - back] += 3.0
            v2[T - 1 - back] += 3.0
            other = _run_attn(m, q, k2, v2, talk, gate, steps, form, window=window)[-1]
            assert torch.equal(other, got[-1]) == same, (back, same)


def test_single_tokens_split_their_keys_over_ctas():
    """A single-token step with a long context takes several CTAs per token and a merge; same values as one CTA per token."""
    from vyomai_b200 import ops
    m = U.attn(heads=6, kv_heads=3, dim=10, vdim=7, scale=0.4, softcap=3.0)
    g = _g(12)
    T = 700
    q, k, v = torch.randn(T, 6, 10, generator=g), torch.randn(T, 3, 10, generator=g), torch.randn(T, 3, 7, generator=g)
    talk = torch.eye(6) + torch.randn(6, 6, generator=g) * 0.5
    gate = torch.randn(T, 42, generator=g)
    want = _attn_oracle(q.double(), k.double(), v.double(), talk.double(), m, gate.double())
    got = _run_attn(m, q, k, v, talk, gate, [T - 3, 1, 1, 1], None, bs=16)
    assert int(ops._lib.lib().vy_talk_attn_workspace_floats(1, 1, 44, 16, 6, 7)) > 0
    assert HU.rel_err(got, want) < 2e-5


def _mixer(cfg_m, seed, dtype=torch.float32, width=40):
    from vyomai_b200.layers.mixers import TalkingHeadsAttention
    g = _g(seed)
    H, G, d, dv = cfg_m["heads"], cfg_m["kv_heads"], cfg_m["dim"], cfg_m["vdim"]
    shapes = {"q": (H * d, width), "k": (G * d, width), "v": (G * dv, width), "g": (H * dv, width), "o": (width, H * dv)}
    w = {k: (torch.randn(s, generator=g) / math.sqrt(s[1])).to(torch.bfloat16) for k, s in shapes.items()}
    for k, n in (("q.b", H * d), ("k.b", G * d), ("v.b", G * dv), ("o.b", width)):
        w[k] = (0.3 * torch.randn(n, generator=g)).to(torch.bfloat16)
    w["talk"] = (torch.eye(H) + 0.4 * torch.randn(H, H, generator=g)).to(torch.bfloat16)
    mix = TalkingHeadsAttention(cfg_m, {k: v.to(DEV, dtype) for k, v in w.items()}, 1e-5, dtype, True)
    return mix, {k: v.double() for k, v in w.items()}


@pytest.mark.parametrize("steps", [[37], [20, 1, 1, 1, 14], [2] * 18 + [1], [16, 21]])
def test_attention_mixer_with_biases_and_rotation(steps):
    from vyomai_b200 import ops
    from vyomai_b200.paged import LayerCacheView
    m = U.attn(heads=6, kv_heads=2, dim=8, vdim=10, rot_dims=6)
    mix, W = _mixer(m, 2)
    h = torch.randn(37, 40, generator=_g(3))
    want = O.attention(h.double(), W, m)
    bs, T = 4, 37
    n_blocks = (T + bs - 1) // bs + 2
    order = torch.randperm(n_blocks, generator=_g(5)).tolist()
    view = LayerCacheView()
    view.k_pool, view.v_pool = torch.zeros((n_blocks, bs, 2, 8), device=DEV), torch.zeros((n_blocks, bs, 2, 10), device=DEV)
    t = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)  # noqa: E731
    outs, at = [], 0
    for n in steps:
        batch = ops.PackedBatch(t([0, n]), t([at]), t([0]), n, t(order).view(1, -1), bs)
        x = h[at:at + n].to(DEV)
        parts = [ops.linear_plain(x, wt.to(DEV).float(), bias=None if b is None else b.float()) for wt, b in zip(mix.input_weights(), mix.input_biases())]
        outs.append(mix.forward(parts, batch, view).float().cpu())
        at += n
    assert HU.rel_err(torch.cat(outs), want) < 1e-4


@pytest.mark.parametrize("force_sorted", [False, True])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gated_experts_both_forms(force_sorted, dtype):
    from vyomai_b200 import ops
    from vyomai_b200.layers.mixers import MoEFeedForward
    g = _g(7)
    width, E, ff, sf = 64, 6, 32, 48
    f = U.moe(experts=E, top=2, ff=ff, limit=1.0, groups=(3, 2), shared_ff=sf, shared_limit=0.7)
    w = {"router": torch.randn(E, width, generator=g) * 2 / math.sqrt(width)}
    for e in list(range(E)) + ["shared"]:
        pre, n = (f"e{e}.", ff) if e != "shared" else ("shared.", sf)
        w.update({pre + "gate": torch.randn(n, width, generator=g) / math.sqrt(width) * 2, pre + "up": torch.randn(n, width, generator=g) / math.sqrt(width) * 2,
                  pre + "down": torch.randn(width, n, generator=g) / math.sqrt(n)})
    w = {k: v.to(torch.bfloat16) for k, v in w.items()}
    mlp = MoEFeedForward({k: v.to(DEV, dtype) for k, v in w.items()}, E, 2, 1.0, dtype, True, shared=True, sorted_min_rows=8, force_sorted=force_sorted,
                         router="softmax", groups=(3, 2), normalize=False, form="glu", limit=1.0, shared_limit=0.7)
    h = torch.randn(40, width, generator=g).to(torch.bfloat16)
    want = O.moe_ff(h.double(), {k: v.double() for k, v in w.items()}, f)
    batch, *_ = HU.shuffled_batch([40], [0], 16, DEV)
    got = mlp.forward(h.to(DEV, dtype), batch).cpu()
    assert HU.rel_err(got, want) < (1e-4 if dtype == torch.float32 else 2e-2)
