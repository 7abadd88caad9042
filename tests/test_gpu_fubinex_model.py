"""The Fubinex decoder end to end on the GPU: FubinexForCausalLM through HybridBatchEngine / HybridCacheManager (the engine a user
generates with, and the one bin/trace_run drives) against oracle/fubinex_oracle.py's float64 forward of the same seeded weights.
Whole prompts, portions down to two tokens, token-by-token decoding (also through the captured CUDA graph), mixed batches of
unequal requests, pages and state slots that are freed and handed out again, chunk edges in prompts and in decoding, a far key, long
decoding across page borders, other sizes, greedy generation, the replayer's command line. float32 models are held to 2e-4 of the
largest logit at every position, bfloat16 ones to 2e-2, except at the first four positions of a sequence, which are held to 0.2: there
a retention head's read-out is a sum of one to four terms (q_t . k_j) v_j divided by its own root mean square, so when a dot product
happens to be near zero the bf16 rounding of the layer input decides the direction of the normalised result."""
import json
import os
import subprocess

import numpy as np
import pytest
import torch

from oracle import fubinex_oracle as O
from tests import fubinex_util as U
from tests import hybrid_util as HU

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TOL = {torch.float32: 2e-4, torch.bfloat16: 2e-2}


def _check(got, want, dtype, what="", tol=None, pos0=0):
    """got: logits of positions pos0 .. of the sequence whose oracle logits are `want` (from position 0)."""
    want = want[pos0:pos0 + got.shape[0]].double()
    e = (got.double() - want).abs().max(-1).values / want.abs().max()
    tol = tol or TOL[dtype]
    if dtype == torch.bfloat16 and pos0 < 4:
        assert float(e[:4 - pos0].max()) < 0.2, (what, "first positions", float(e[:4 - pos0].max()))
        e = e[4 - pos0:]
    assert e.numel() == 0 or float(e.max()) < tol, (what, float(e.max()))


def test_residual_stream_layer_by_layer():
    cfg = U.small_config()
    model, W = U.build(cfg)
    eng, _ = HU.engine_for(model)
    toks = HU.tokens(23, cfg["vocab"], 1)
    ref_res = []
    ref = O.forward(cfg, W, toks, residuals=ref_res)
    model.debug_residuals = []
    got = eng.feed([("a", toks, list(range(len(toks))))]).float().cpu()
    for i, (x, r) in enumerate(zip(model.debug_residuals, ref_res)):
        assert HU.rel_err(x.cpu(), r) < 1e-4, f"layer {i}"
    model.debug_residuals = None
    assert HU.rel_err(got, ref) < TOL[torch.float32]


@pytest.mark.parametrize("dtype,cfg_name", [(torch.float32, "small"), (torch.float32, "aligned"), (torch.bfloat16, "aligned")])
@pytest.mark.parametrize("cuts", [[44], [2, 2, 2, 30], [1], [17, 3, 5], [33]])
def test_prompt_portions_and_decoding_agree_with_the_oracle(dtype, cfg_name, cuts):
    cfg = U.small_config() if cfg_name == "small" else U.aligned_config()
    model, W = U.build(cfg, dtype=dtype)
    eng, _ = HU.engine_for(model)
    toks = HU.tokens(44, cfg["vocab"], 2)
    _check(HU.feed_in_portions(eng, "s", toks, cuts), O.forward(cfg, W, toks), dtype)


def test_cutting_changes_nothing_beyond_rounding():
    cfg = U.small_config()
    model, _ = U.build(cfg)
    eng, _ = HU.engine_for(model)
    toks = HU.tokens(48, cfg["vocab"], 3)
    whole = HU.feed_in_portions(eng, "w", toks, [48])
    for cuts in ([2] * 24, [1], [5, 9, 2, 20], [47]):
        eng.release(["p"])
        assert HU.rel_err(HU.feed_in_portions(eng, "p", toks, cuts), whole) < 2e-5, cuts


@pytest.mark.parametrize("dtype,cfg_name", [(torch.float32, "small"), (torch.bfloat16, "aligned")])
def test_mixed_batch_equals_each_request_alone(dtype, cfg_name):
    cfg = U.small_config() if cfg_name == "small" else U.aligned_config()
    model, W = U.build(cfg, dtype=dtype)
    eng, _ = HU.engine_for(model, max_seqs=1, max_tokens=16)     # pools and slots must grow under the batch
    lens = {"a": 31, "b": 3, "c": 12, "d": 1}
    toks = {k: HU.tokens(n + 6, cfg["vocab"], 10 + i) for i, (k, n) in enumerate(lens.items())}
    ref = {k: O.forward(cfg, W, t) for k, t in toks.items()}
    got = {k: [] for k in lens}
    # prompts of unequal length in one step, then decode together; "b" and "d" end early and drop out
    out = eng.feed([(k, toks[k][:n], list(range(n))) for k, n in lens.items()]).float().cpu()
    at = 0
    for k, n in lens.items():
        got[k].append(out[at:at + n])
        at += n
    live = list(lens)
    for step in range(6):
        if step == 3:
            eng.release(["b", "d"])
            live = ["a", "c"]
        out = eng.feed([(k, [toks[k][lens[k] + step]], [0]) for k in live]).float().cpu()
        for i, k in enumerate(live):
            got[k].append(out[i:i + 1])
    for k in lens:
        _check(torch.cat(got[k]), ref[k], dtype, k)


def test_pages_and_slots_freed_and_used_again():
    cfg = U.small_config()
    model, W = U.build(cfg)
    eng, mgr = HU.engine_for(model, max_tokens=64, block_size=4, max_seqs=2)
    a, b, c = (HU.tokens(n, cfg["vocab"], s) for n, s in ((37, 5), (29, 6), (41, 7)))
    eng.feed([("a", a, []), ("b", b, [])])
    used, slot = set(eng.active["a"].blocks), eng.active["a"].slot
    eng.release(["a"])
    # "c" gets a's pages and state slot back (the slot still holds a's recurrent state) while "b" keeps decoding beside it
    got_c = eng.feed([("c", c[:30], list(range(30))), ("b", [3], [])]).float().cpu()
    assert used & set(eng.active["c"].blocks) and eng.active["c"].slot == slot
    got_c = torch.cat([got_c, HU.feed_in_portions(eng, "c", c[30:], [4])])
    assert HU.rel_err(got_c, O.forward(cfg, W, c)) < TOL[torch.float32]


def _chunk_layer(chunk, **kw):
    return U.config([U.layer("parallel", U.parallel(U.left(chunk=chunk, **kw), U.right(), 1.0, 0.0), None)])


@pytest.mark.parametrize("decode", [False, True])
@pytest.mark.parametrize("chunk,block,heads", [(5, 4, 4), (16, 16, 4), (17, 4, 16)])
def test_chunk_edge_inside_and_outside(chunk, block, heads, decode):
    """One block-local attention layer (its linear-attention neighbour weighted 0): the logits at the first position of a block depend
    on nothing before it, the logits at its last position on the block's first token and not on the token before that; in a prompt
    and when the last tokens are decoded one by one; with the edge at and off a page border; blocks counted from position 0 although the
    prompt is cut elsewhere."""
    cfg = _chunk_layer(chunk, heads=heads)
    model, W = U.build(cfg)
    n = 3 * chunk          # the last position closes the third block
    base = HU.tokens(n, cfg["vocab"], 11)

    def last_logits(toks, upto=n):
        eng, _ = HU.engine_for(model, block_size=block)
        cut = upto - chunk - 2 if decode else upto
        return HU.feed_in_portions(eng, "s", toks[:upto], [cut])[-1]

    ref = last_logits(base)
    assert HU.rel_err(ref[None], O.forward(cfg, W, base)[-1:]) < TOL[torch.float32]
    first = n - chunk      # first position of the last block
    outside, inside = list(base), list(base)
    outside[first - 1] = (base[first - 1] + 1) % cfg["vocab"]
    inside[first] = (base[first] + 1) % cfg["vocab"]
    assert torch.equal(last_logits(outside), ref)
    assert HU.rel_err(last_logits(inside)[None], ref[None]) > 1e-4
    # the first position of a block sees itself only
    alone = last_logits(base, upto=first + 1)
    other = [(t + 1) % cfg["vocab"] for t in base[:first]] + base[first:]
    assert torch.equal(last_logits(other, upto=first + 1), alone)


def test_a_key_far_back_reaches_through_every_mixer():
    """A change of the very first token of a long prompt must show 300 positions later through the latent attention (no window) and
    through the recurrent states, in a whole prompt and in decoding alike."""
    cfg = U.small_config()
    model, W = U.build(cfg)
    toks = HU.tokens(300, cfg["vocab"], 21)
    ref = O.forward(cfg, W, toks)
    for cuts in ([300], [280]):
        eng, _ = HU.engine_for(model, block_size=16, max_tokens=512)
        _check(HU.feed_in_portions(eng, "s", toks, cuts)[-20:], ref[-20:], torch.float32, str(cuts), tol=4e-4)
    changed = [(toks[0] + 1) % cfg["vocab"]] + toks[1:]
    assert HU.rel_err(O.forward(cfg, W, changed)[-1:], ref[-1:]) > 1e-5


def test_first_tokens_of_a_sequence():
    cfg = U.small_config()
    model, W = U.build(cfg)
    toks = HU.tokens(6, cfg["vocab"], 13)
    ref = O.forward(cfg, W, toks)
    for cuts in ([1], [2], [1, 2], [6]):
        eng, _ = HU.engine_for(model)
        assert HU.rel_err(HU.feed_in_portions(eng, "s", toks, cuts), ref) < TOL[torch.float32], cuts


@pytest.mark.parametrize("dtype,cfg_name", [(torch.float32, "small"), (torch.bfloat16, "aligned"), (torch.float32, "many_heads")])
def test_long_decoding_through_the_captured_step(dtype, cfg_name):
    """150 single-token steps (several chunks, many page borders); from the third step of a shape on they replay a CUDA graph."""
    cfg = {"small": U.small_config, "aligned": U.aligned_config, "many_heads": U.many_heads_config}[cfg_name]()
    model, W = U.build(cfg, dtype=dtype)
    eng, _ = HU.engine_for(model, block_size=8, use_graph=True)
    toks = HU.tokens(160, cfg["vocab"], 14)
    got = HU.feed_in_portions(eng, "s", toks, [10])
    assert eng._graphs, "single-token steps were not captured"
    _check(got, O.forward(cfg, W, toks), dtype, tol=None if dtype == torch.float32 else 3e-2)


def test_values_that_are_one_or_equal():
    """One head everywhere, one norm group, chunk 1 (a token sees only itself) and a chunk longer than the sequence, scales and tau of
    1, rank == dim == vdim == rot_dim, a whole head rotated, width == ff, embedding scale 1."""
    la = dict(heads=1, dim=8, rot_dim=8, vdim=8, rank=8, q_rank=8, scale=1.0)
    cfg = U.config([U.layer("parallel", U.parallel(U.left(heads=1, kv_heads=1, dim=8, vdim=8, chunk=1, scale=1.0, rot_dims=8), U.right(heads=1, dim=8, vdim=8, tau=1.0), 1.0, 1.0),
                            U.dense(ff=16)),
                    U.layer("latent_attention", U.latent(**la), U.dense(ff=16)),
                    U.layer("parallel", U.parallel(U.left(heads=2, kv_heads=2, dim=8, vdim=8, chunk=1000, rot_dims=0), U.right(heads=1, dim=8, vdim=8, tau=1.0), 1.0, 1.0), None),
                    U.layer("latent_attention", U.latent(kv_from=1, **la), None),
                    U.layer("retention", U.retention(heads=1, dim=8, vdim=8, decay=(1.0,), rot_dims=8), U.dense(ff=16))], width=16, vocab=16, groups=1, emb_scale=1.0)
    model, W = U.build(cfg)
    eng, _ = HU.engine_for(model)
    toks = HU.tokens(30, cfg["vocab"], 15)
    assert HU.rel_err(HU.feed_in_portions(eng, "s", toks, [9, 2]), O.forward(cfg, W, toks)) < TOL[torch.float32]


@pytest.mark.parametrize("seed", range(8))
def test_configurations_drawn_at_random(seed):
    """Other layer orders, head counts, channel counts, chunks, constants: a prompt with decoding, portions, and two unequal requests in
    one batch, in fp32 and in bf16 (tensor-core products wherever the drawn sizes allow them) against the oracle."""
    for dtype in (torch.float32, torch.bfloat16):
        cfg = U.random_config(seed)
        toks, other = HU.tokens(70, cfg["vocab"], 40 + seed), HU.tokens(21, cfg["vocab"], 80 + seed)
        model, W = U.build(cfg, dtype=dtype, seed=seed)
        ref, ref_o = O.forward(cfg, W, toks), O.forward(cfg, W, other)
        eng, _ = HU.engine_for(model, block_size=16)
        tol = None if dtype == torch.float32 else 5e-2   # latents of 12 channels and widths of 48 average less bf16 noise away
        _check(HU.feed_in_portions(eng, "w", toks, [40]), ref, dtype, "prompt + decoding", tol)
        _check(HU.feed_in_portions(eng, "p", toks, [19, 2, 30, 7]), ref, dtype, "portions", tol)
        out = eng.feed([("a", toks[:50], list(range(50))), ("b", other[:9], list(range(9)))]).float().cpu()
        _check(out[:50], ref, dtype, "batch a", tol)
        _check(out[50:], ref_o, dtype, "batch b", tol)
        out = eng.feed([("a", toks[50:51], [0]), ("b", other[9:10], [0])]).float().cpu()
        _check(out[:1], ref, dtype, "batch a decoded", tol, pos0=50)
        _check(out[1:], ref_o, dtype, "batch b decoded", tol, pos0=9)


def test_greedy_generation_through_the_engine():
    cfg = U.small_config()
    model, W = U.build(cfg)
    eng, _ = HU.engine_for(model, max_seqs=3)
    prompts = [HU.tokens(n, cfg["vocab"], 20 + n) for n in (9, 2, 17)]
    outs = eng.generate(prompts, max_new_tokens=12)
    for p, o in zip(prompts, outs):
        assert o[:len(p)] == p and len(o) == len(p) + 12
        # every generated token is the oracle's argmax given the tokens before it (ties aside: the margin is checked)
        ref = O.forward(cfg, W, o[:-1])
        for t in range(len(p), len(o)):
            row = ref[t - 1]
            top2 = torch.topk(row, 2).values
            if float(top2[0] - top2[1]) > 1e-3 * float(row.abs().max()):
                assert int(row.argmax()) == o[t], (t, o)


def test_trace_replayer_command_line(tmp_path):
    from vyomai_b200 import FubinexConfig, FubinexForCausalLM
    from vyomai_b200.checkpoint import save_safetensors
    cfg = U.small_config()
    w = FubinexForCausalLM.random_weights(FubinexConfig(cfg), seed=3, low_rank=5)
    mdir, out = tmp_path / "model", tmp_path / "out"
    mdir.mkdir()
    (mdir / "config.json").write_text(json.dumps(cfg))
    save_safetensors(str(mdir / "model.safetensors"), w)
    a, b = HU.tokens(21, cfg["vocab"], 31), HU.tokens(9, cfg["vocab"], 32)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:18], "want": [0, 17]}, {"id": "b", "tokens": b[:7], "want": [6]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[18:19], "want": []}, {"id": "b", "tokens": b[7:8], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": a[19:20], "want": [0]}, {"id": "b", "tokens": b[8:9], "want": [0]}], "end": ["b"]},
             {"step": 3, "entries": [{"id": "a", "tokens": a[20:21], "want": [0]}], "end": ["a"]}]
    for dtype, tol in (("float32", TOL[torch.float32]), ("bfloat16", 5e-2)):
        r = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", str(mdir), "--dtype", dtype, "--out", str(out), "--max-tokens", "64"],
                           input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stderr[-2000:]
        assert [ln for ln in r.stdout.splitlines() if ln.startswith("done")] == ["done 0", "done 1", "done 2", "done 3"]
        W = U.f64(w)
        ra, rb = O.forward(cfg, W, a), O.forward(cfg, W, b)
        V = cfg["vocab"]
        g0 = torch.from_numpy(np.fromfile(out / "0.f32", dtype="<f4").reshape(-1, V))
        g2 = torch.from_numpy(np.fromfile(out / "2.f32", dtype="<f4").reshape(-1, V))
        g3 = torch.from_numpy(np.fromfile(out / "3.f32", dtype="<f4").reshape(-1, V))
        assert not (out / "1.f32").exists()
        assert HU.rel_err(g0, torch.stack([ra[0], ra[17], rb[6]])) < tol
        assert HU.rel_err(g2, torch.stack([ra[19], rb[8]])) < tol
        assert HU.rel_err(g3, ra[20:21]) < tol
