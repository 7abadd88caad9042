"""The Vazepel decoder end to end on the GPU: VazepelForCausalLM through HybridBatchEngine / HybridCacheManager (the engine a user
generates with, and the one bin/trace_run drives) against oracle/vazepel_oracle.py's float64 forward of the same seeded weights.
Whole prompts, portions down to two tokens, token-by-token decoding (also through the captured CUDA graph), mixed batches of
unequal requests, pages that are freed and handed out again, keys far away and at page borders, long decoding, other sizes,
greedy generation, the replayer's command line. float32 models are held to 2e-4 of the largest logit at every position;
bfloat16 ones to 2e-2, except that one position in 40 may be a routing close call (the bf16 noise of the router's input moves a
score across its neighbour's, a discrete change) and is held to 0.2 instead."""
import json
import os
import subprocess

import numpy as np
import pytest
import torch

from oracle import vazepel_oracle as O
from tests import hybrid_util as HU
from tests import vazepel_util as U

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TOL = {torch.float32: 2e-4, torch.bfloat16: 2e-2}


def _check(got, want, dtype, what="", tol=None):
    want = want[:got.shape[0]].double()
    e = (got.double() - want).abs().max(-1).values / want.abs().max()
    tol = tol or TOL[dtype]
    if dtype == torch.float32:
        assert float(e.max()) < tol, (what, float(e.max()))
        return
    over = int((e > tol).sum())
    assert over <= max(1, e.numel() // 40) and float(e.max()) < 0.2, (what, over, float(e.max()))


def test_residual_stream_layer_by_layer():
    cfg = U.small_config()
    model, W = U.build(cfg)
    eng, _ = HU.engine_for(model)
    toks = HU.tokens(23, cfg["vocab"], 1)
    ref_res = []
    ref = O.forward(toks, W, cfg, residuals=ref_res)
    model.debug_residuals = []
    got = eng.feed([("a", toks, list(range(len(toks))))]).float().cpu()
    for i, (x, r) in enumerate(zip(model.debug_residuals, ref_res)):
        assert HU.rel_err(x.cpu(), r) < 1e-4, f"layer {i}"
    model.debug_residuals = None
    assert HU.rel_err(got, ref) < TOL[torch.float32]


@pytest.mark.parametrize("dtype,cfg_name", [(torch.float32, "small"), (torch.float32, "aligned"), (torch.bfloat16, "aligned"), (torch.float32, "wide")])
@pytest.mark.parametrize("cuts", [[44], [2, 2, 2, 30], [1], [17, 3, 5], [33]])
def test_prompt_portions_and_decoding_agree_with_the_oracle(dtype, cfg_name, cuts):
    cfg = {"small": U.small_config, "aligned": U.aligned_config, "wide": U.wide_config}[cfg_name]()
    model, W = U.build(cfg, dtype=dtype)
    eng, _ = HU.engine_for(model)
    toks = HU.tokens(44, cfg["vocab"], 2)
    _check(HU.feed_in_portions(eng, "s", toks, cuts), O.forward(toks, W, cfg), dtype)


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
    eng, _ = HU.engine_for(model, max_seqs=1, max_tokens=16)     # pools must grow under the batch
    lens = {"a": 31, "b": 3, "c": 12, "d": 1}
    toks = {k: HU.tokens(n + 6, cfg["vocab"], 10 + i) for i, (k, n) in enumerate(lens.items())}
    ref = {k: O.forward(t, W, cfg) for k, t in toks.items()}
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


def test_batch_neighbours_do_not_change_a_request():
    cfg = U.small_config()
    model, _ = U.build(cfg)
    a, b = HU.tokens(29, cfg["vocab"], 21), HU.tokens(11, cfg["vocab"], 22)
    eng, _ = HU.engine_for(model)
    alone = eng.feed([("a", a, list(range(29)))]).float().cpu()
    eng2, _ = HU.engine_for(model)
    both = eng2.feed([("b", b, []), ("a", a, list(range(29)))]).float().cpu()
    assert HU.rel_err(both, alone) < 2e-5


def test_pages_freed_and_used_again():
    cfg = U.small_config()
    model, W = U.build(cfg)
    eng, mgr = HU.engine_for(model, max_tokens=64, block_size=4, max_seqs=2)
    a, b, c = (HU.tokens(n, cfg["vocab"], s) for n, s in ((37, 5), (29, 6), (41, 7)))
    eng.feed([("a", a, []), ("b", b, [])])
    used = set(eng.active["a"].blocks)
    eng.release(["a"])
    # "c" gets a's pages back (out of order: the free list is a queue) while "b" keeps decoding beside it
    got_c = eng.feed([("c", c[:30], list(range(30))), ("b", [3], [])]).float().cpu()
    assert used & set(eng.active["c"].blocks)
    got_c = torch.cat([got_c, HU.feed_in_portions(eng, "c", c[30:], [4])])
    assert HU.rel_err(got_c, O.forward(c, W, cfg)) < TOL[torch.float32]


@pytest.mark.parametrize("decode", [False, True])
@pytest.mark.parametrize("block", [4, 16])
def test_every_earlier_token_is_seen_and_no_later_one(block, decode):
    """One attention layer: the last logits change when the FIRST token changes (hundreds of keys and many pages back) and when the
    token just before a page border does; the logits of a position do not change when a LATER token does."""
    cfg = U.config([U.layer(U.attn(), None)])
    model, W = U.build(cfg)
    n = 200
    base = HU.tokens(n, cfg["vocab"], 11)

    def logits(toks):
        eng, _ = HU.engine_for(model, block_size=block)
        return HU.feed_in_portions(eng, "s", toks, [n - 40 if decode else n])

    ref = logits(base)
    assert HU.rel_err(ref, O.forward(base, W, cfg)) < TOL[torch.float32]
    for i in (0, block - 1, block, n - 2):
        other = list(base)
        other[i] = (base[i] + 1) % cfg["vocab"]
        got = logits(other)
        assert torch.equal(got[:i], ref[:i]), i
        assert HU.rel_err(got[-1:], ref[-1:]) > 1e-6, i
        assert HU.rel_err(got, O.forward(other, W, cfg)) < TOL[torch.float32]


def test_first_tokens_of_a_sequence():
    cfg = U.small_config()
    model, W = U.build(cfg)
    toks = HU.tokens(6, cfg["vocab"], 13)
    ref = O.forward(toks, W, cfg)
    for cuts in ([1], [2], [1, 2], [6]):
        eng, _ = HU.engine_for(model)
        assert HU.rel_err(HU.feed_in_portions(eng, "s", toks, cuts), ref) < TOL[torch.float32], cuts


@pytest.mark.parametrize("dtype,cfg_name", [(torch.float32, "small"), (torch.bfloat16, "aligned"), (torch.float32, "wide")])
def test_long_decoding_through_the_captured_step(dtype, cfg_name):
    """150 single-token steps (many page borders, several key tiles, key splits once the table is wide enough); from the third step
    of a shape on they replay a CUDA graph."""
    cfg = {"small": U.small_config, "aligned": U.aligned_config, "wide": U.wide_config}[cfg_name]()
    model, W = U.build(cfg, dtype=dtype)
    eng, _ = HU.engine_for(model, block_size=8, use_graph=True)
    toks = HU.tokens(160, cfg["vocab"], 14)
    got = HU.feed_in_portions(eng, "s", toks, [10])
    assert eng._graphs, "single-token steps were not captured"
    _check(got, O.forward(toks, W, cfg), dtype)


def test_values_that_are_one_or_equal():
    """One head; one expert of one; one group; all groups kept; top == experts; dim == vdim == rotated entries; nothing rotated;
    width == ff; a stack coefficient vector of the shortest length (first layer)."""
    a = dict(heads=1, kv_heads=1, dim=8, vdim=8, scale=1.0)
    cfg = U.config([U.layer(U.attn(**a), U.moe(experts=1, top=1, ff=16, groups=(1, 1), shared_ff=16)),
                    U.layer(U.attn(rot_dims=0, **a), U.dense(ff=16)),
                    U.layer(U.attn(heads=2, kv_heads=2, dim=8, vdim=8, scale=1.0), U.moe(experts=2, top=2, ff=8, groups=(2, 2), shared_ff=None))], width=16, vocab=16)
    model, W = U.build(cfg)
    eng, _ = HU.engine_for(model)
    toks = HU.tokens(30, cfg["vocab"], 15)
    assert HU.rel_err(HU.feed_in_portions(eng, "s", toks, [9, 2]), O.forward(toks, W, cfg)) < TOL[torch.float32]


def test_gates_and_stack_coefficients_matter():
    """Weights chosen so that a dropped gate, a dropped bias or a wrong stack slice shows: strongly negative gate biases on one sublayer,
    stack coefficients that put most weight on OLD results."""
    from vyomai_b200 import VazepelConfig, VazepelForCausalLM
    cfg = U.config([U.layer(U.attn(), U.dense()), U.layer(U.attn(), U.moe()), U.layer(U.attn(), U.dense())])
    w = VazepelForCausalLM.random_weights(VazepelConfig(cfg), seed=4)
    w["l0.rg1.b"] = torch.full_like(w["l0.rg1.b"], -6.0)
    w["l1.rg2.b"] = torch.full_like(w["l1.rg2.b"], 4.0)
    w["l1.dwa"] = torch.tensor([0.9, -0.4, 0.3]).to(torch.bfloat16)
    w["l2.dwa"] = torch.tensor([0.5, 0.25, -0.75, 0.125]).to(torch.bfloat16)
    w["l2.mix.o.b"] = torch.full_like(w["l2.mix.o.b"], 2.0)
    model, W = U.build(cfg, weights=w)
    eng, _ = HU.engine_for(model)
    toks = HU.tokens(25, cfg["vocab"], 16)
    assert HU.rel_err(HU.feed_in_portions(eng, "s", toks, [13]), O.forward(toks, W, cfg)) < TOL[torch.float32]


@pytest.mark.parametrize("seed", range(8))
def test_configurations_drawn_at_random(seed):
    """Other layer orders, head counts, channel counts, constants: a prompt with decoding, portions, and two unequal requests in one
    batch, in fp32 against the oracle; the same in bf16 with the mixtures replaced by dense feed-forwards (with random routers the bf16
    noise of the router's input flips a choice now and then, and a flip changes every later position that sees the token)."""
    for dtype in (torch.float32, torch.bfloat16):
        cfg = U.random_config(seed, experts=dtype == torch.float32)
        toks, other = HU.tokens(70, cfg["vocab"], 40 + seed), HU.tokens(21, cfg["vocab"], 80 + seed)
        model, W = U.build(cfg, dtype=dtype, seed=seed)
        ref, ref_o = O.forward(toks, W, cfg), O.forward(other, W, cfg)
        eng, _ = HU.engine_for(model, block_size=16)
        tol = None if dtype == torch.float32 else 5e-2
        _check(HU.feed_in_portions(eng, "w", toks, [40]), ref, dtype, "prompt + decoding", tol)
        _check(HU.feed_in_portions(eng, "p", toks, [19, 2, 30, 7]), ref, dtype, "portions", tol)
        out = eng.feed([("a", toks[:50], list(range(50))), ("b", other[:9], list(range(9)))]).float().cpu()
        _check(out[:50], ref, dtype, "batch a", tol)
        _check(out[50:], ref_o, dtype, "batch b", tol)
        out = eng.feed([("a", toks[50:51], [0]), ("b", other[9:10], [0])]).float().cpu()
        _check(out[:1], ref[50:51], dtype, "batch a decoded", tol)
        _check(out[1:], ref_o[9:10], dtype, "batch b decoded", tol)


def test_greedy_generation_through_the_engine():
    cfg = U.small_config()
    model, W = U.build(cfg)
    eng, _ = HU.engine_for(model, max_seqs=3)
    prompts = [HU.tokens(n, cfg["vocab"], 20 + n) for n in (9, 2, 17)]
    outs = eng.generate(prompts, max_new_tokens=12)
    for p, o in zip(prompts, outs):
        assert o[:len(p)] == p and len(o) == len(p) + 12
        # every generated token is the oracle's argmax given the tokens before it (ties aside: the margin is checked)
        ref = O.forward(o[:-1], W, cfg)
        for t in range(len(p), len(o)):
            row = ref[t - 1]
            top2 = torch.topk(row, 2).values
            if float(top2[0] - top2[1]) > 1e-3 * float(row.abs().max()):
                assert int(row.argmax()) == o[t], (t, o)


def test_trace_replayer_command_line(tmp_path):
    from vyomai_b200 import VazepelConfig, VazepelForCausalLM
    from vyomai_b200.checkpoint import save_safetensors
    cfg = U.small_config()
    w = VazepelForCausalLM.random_weights(VazepelConfig(cfg), seed=3)
    mdir, out = tmp_path / "model", tmp_path / "out"
    mdir.mkdir()
    (mdir / "config.json").write_text(json.dumps(cfg))
    save_safetensors(str(mdir / "model.safetensors"), w)
    a, b = HU.tokens(21, cfg["vocab"], 31), HU.tokens(9, cfg["vocab"], 32)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:18], "want": [0, 17]}, {"id": "b", "tokens": b[:7], "want": [6]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[18:19], "want": []}, {"id": "b", "tokens": b[7:8], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": a[19:20], "want": [0]}, {"id": "b", "tokens": b[8:9], "want": [0]}], "end": ["b"]},
             {"step": 3, "entries": [{"id": "a", "tokens": a[20:21], "want": [0]}], "end": ["a"]}]
    r = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", str(mdir), "--dtype", "float32", "--out", str(out), "--max-tokens", "64"],
                       input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [ln for ln in r.stdout.splitlines() if ln.startswith("done")] == ["done 0", "done 1", "done 2", "done 3"]
    W = U.f64(w)
    ra, rb = O.forward(a, W, cfg), O.forward(b, W, cfg)
    V = cfg["vocab"]
    g0 = torch.from_numpy(np.fromfile(out / "0.f32", dtype="<f4").reshape(-1, V))
    g2 = torch.from_numpy(np.fromfile(out / "2.f32", dtype="<f4").reshape(-1, V))
    g3 = torch.from_numpy(np.fromfile(out / "3.f32", dtype="<f4").reshape(-1, V))
    assert not (out / "1.f32").exists()
    assert HU.rel_err(g0, torch.stack([ra[0], ra[17], rb[6]])) < TOL[torch.float32]
    assert HU.rel_err(g2, torch.stack([ra[19], rb[8]])) < TOL[torch.float32]
    assert HU.rel_err(g3, ra[20:21]) < TOL[torch.float32]
