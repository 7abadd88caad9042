#!/usr/bin/env python
"""bench.py — headline benchmark of the B200-native VyomAI hot path.

    python bench.py --gpus N --steps K --warmup W            # this repo (sm_100a kernels)
    python bench.py --impl reference --steps K --warmup W    # the reference's CPU path (oracle port)

Metric (BASELINE.json): caption-train samples/s — one step = one full training step (ViT encoder +
RoPE/GQA decoder forward, shifted cross-entropy, backward, gradient all-reduce, global-norm clip,
AdamW) of the image-text fusion captioner `VisionLanguageModel` on one batch of synthetic,
right-padded image/caption pairs, bf16 weights with fp32 master copies. Data-parallel: every rank
processes its own batch of the same size (weak scaling); the only collective is the NCCL gradient
all-reduce. One JSON line is printed by rank 0.
"""
import argparse
import json
import os
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
# stdout carries exactly one JSON line: NCCL's own version / debug prints go to stderr
os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")

WORKLOAD = "captioner_train_vit224p16L4_dec768L8gqa4_rope_rpad_S128"
PER_GPU_BATCH = 64
TEXT_LEN = 127  # + 1 image token = 128 decoder positions
CPU_SAMPLE_BATCH = 8


class TextCfg:
    hidden_size = 768
    num_attention_heads = 12
    num_key_value_heads = 4
    max_position_embeddings = 514
    num_hidden_layers = 8
    vocab_size = 50265
    hidden_dropout_prob = 0.0  # fused path implements p = 0; the reference default is 0.1
    initializer_range = 0.02
    intermediate_size = 3072
    layer_norm_eps = 1e-05
    hidden_act = "gelu"
    pad_token_id = 1


class VitCfg:
    hidden_size = 768
    num_attention_heads = 12
    image_size = (224, 224)
    patch_size = (16, 16)
    num_channels = 3
    num_hidden_layers = 4
    hidden_dropout_prob = 0.0
    initializer_range = 0.02
    intermediate_size = 3072
    layer_norm_eps = 1e-05
    hidden_act = "gelu"


def synth_batch(batch, seed, pin):
    g = torch.Generator().manual_seed(seed)
    pixels = torch.rand((batch, 3, 224, 224), generator=g)
    ids = torch.randint(3, TextCfg.vocab_size, (batch, TEXT_LEN), generator=g)
    lens = torch.randint(8, TEXT_LEN + 1, (batch,), generator=g)
    mask = (torch.arange(TEXT_LEN)[None, :] < lens[:, None]).long()
    ids = torch.where(mask.bool(), ids, torch.full_like(ids, TextCfg.pad_token_id))
    if pin:
        pixels, ids, mask = pixels.pin_memory(), ids.pin_memory(), mask.pin_memory()
    return pixels, ids, mask


# ---- second workload: the notebook-II form of the captioner (Examples/vyom-ai-accelerate-multimodel-2t4.ipynb cell 1) ----
# ViT-base (12 layers) -> all 197 tokens scattered into the <image> slots of a 248-token sequence ([bos, <Caption>] + 197 x
# <image> + caption + eos, right-padded), 8-layer RoPE decoder with the DeBERTa-v3-base widths the notebook takes its config
# from (768 / 12 heads MHA / 3072, vocab 128100 + <image>, LayerNorm eps 1e-7), causal x padding mask, AdamW + clip 1.0.
SLOTS_WORKLOAD = "captioner_II_train_vit224p16L12_197img_in_248tok_dec768L8mha_rope_rpad"
SLOTS_SEQ, SLOTS_IMG, SLOTS_BATCH, SLOTS_IMAGE_TOKEN = 248, 197, 32, 128001


class SlotTextCfg(TextCfg):
    num_key_value_heads = None
    vocab_size = 128101
    layer_norm_eps = 1e-07
    pad_token_id = 0


class SlotVitCfg(VitCfg):
    num_hidden_layers = 12


def synth_slot_batch(batch, seed, pin):
    g = torch.Generator().manual_seed(seed)
    pixels = torch.rand((batch, 3, 224, 224), generator=g)
    n_text = SLOTS_SEQ - 2 - SLOTS_IMG  # 49 caption positions incl. eos
    ids = torch.full((batch, SLOTS_SEQ), SlotTextCfg.pad_token_id, dtype=torch.long)
    ids[:, 0], ids[:, 1] = 1, 5
    ids[:, 2:2 + SLOTS_IMG] = SLOTS_IMAGE_TOKEN
    text = torch.randint(6, 128000, (batch, n_text), generator=g)
    lens = torch.randint(8, n_text + 1, (batch,), generator=g)
    keep = torch.arange(n_text)[None, :] < lens[:, None]
    ids[:, 2 + SLOTS_IMG:] = torch.where(keep, text, torch.full_like(text, SlotTextCfg.pad_token_id))
    mask = (ids != SlotTextCfg.pad_token_id).long()
    if pin:
        pixels, ids, mask = pixels.pin_memory(), ids.pin_memory(), mask.pin_memory()
    return pixels, ids, mask


class ClockSampler(threading.Thread):
    """Samples SM clocks and throttle reasons through NVML while the timed region runs."""

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index, self.stop_flag, self.samples, self.reasons, self.max_mhz = index, False, [], set(), None

    def run(self):
        try:
            import pynvml as nv
            nv.nvmlInit()
            h = nv.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM)
            names = {
                nv.nvmlClocksThrottleReasonHwSlowdown: "hw_slowdown",
                nv.nvmlClocksThrottleReasonHwThermalSlowdown: "hw_thermal_slowdown",
                nv.nvmlClocksThrottleReasonSwThermalSlowdown: "sw_thermal_slowdown",
                nv.nvmlClocksThrottleReasonSwPowerCap: "sw_power_cap",
            }
            while not self.stop_flag:
                self.samples.append(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(h)
                for bit, nm in names.items():
                    if r & bit:
                        self.reasons.add(nm)
                time.sleep(0.1)
        except Exception as e:  # NVML missing: report that instead of inventing clocks
            self.reasons.add(f"nvml_unavailable:{type(e).__name__}")

    def result(self):
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons)}


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d["hbm_gbs"], d["bf16_tflops"], d["bf16_tflops_sustained"], "measured"
    return 6650.0, 1590.0, 1400.0, "fallback"


# ------------------------------------------------------------------------------------------------
# reference arm / cpu baseline: the oracle port of the reference's CPU path
# ------------------------------------------------------------------------------------------------
def oracle_state_dict(TextCfg=TextCfg, VitCfg=VitCfg, head="decoder.lm_head.", head_proj="decoder"):
    """Random-init weights of the bench's captioner for the CPU arm, keyed like the reference's state_dict (the names the
    oracle reads), built with plain torch — none of this repo's modules are involved in the reference arm."""
    g = torch.Generator().manual_seed(0)
    H, V, FF = TextCfg.hidden_size, TextCfg.vocab_size, 4 * TextCfg.hidden_size
    kv = (TextCfg.num_key_value_heads or TextCfg.num_attention_heads) * (H // TextCfg.num_attention_heads)
    sd = {}

    def lin(name, out_f, in_f):
        bound = in_f ** -0.5  # nn.Linear's default init range
        sd[name + ".weight"] = (torch.rand(out_f, in_f, generator=g) * 2 - 1) * bound
        sd[name + ".bias"] = (torch.rand(out_f, generator=g) * 2 - 1) * bound

    def ln(name, n):
        sd[name + ".weight"], sd[name + ".bias"] = torch.ones(n), torch.zeros(n)

    def block(pre, fused_qkv, kv_out):
        if fused_qkv:
            lin(pre + "attention.qkv", 3 * H, H)
        else:
            lin(pre + "attention.query", H, H)
            lin(pre + "attention.key", kv_out, H)
            lin(pre + "attention.value", kv_out, H)
        lin(pre + "attention.out.dense", H, H)
        ln(pre + "attention.out.layernorm", H)
        lin(pre + "feed_forward.intermediate", FF, H)
        lin(pre + "feed_forward.out", H, FF)
        ln(pre + "feed_forward.layernorm", H)

    pdim = VitCfg.num_channels * VitCfg.patch_size[0] * VitCfg.patch_size[1]
    npatch = (VitCfg.image_size[0] // VitCfg.patch_size[0]) * (VitCfg.image_size[1] // VitCfg.patch_size[1])
    sd["encoder.pixel_seq.weight"] = (torch.rand(H, VitCfg.num_channels, *VitCfg.patch_size, generator=g) * 2 - 1) * pdim ** -0.5
    sd["encoder.pixel_seq.bias"] = (torch.rand(H, generator=g) * 2 - 1) * pdim ** -0.5
    sd["encoder.cls_token"] = torch.randn(1, 1, pdim, generator=g)
    sd["encoder.position_embeddings.pos_embeddings"] = torch.randn(1, npatch + 1, pdim, generator=g)
    for i in range(VitCfg.num_hidden_layers):
        block(f"encoder.all_layer.{i}.", True, H)
    sd["decoder.word_embeddings.weight"] = torch.randn(V, H, generator=g)
    for i in range(TextCfg.num_hidden_layers):
        block(f"decoder.all_layer.{i}.", False, kv)
    lin(head + "dense", H, H)
    ln(head + "layer_norm", H)
    sd[head + head_proj + ".weight"] = (torch.rand(V, H, generator=g) * 2 - 1) * H ** -0.5
    sd[head + "bias"] = torch.zeros(V)
    sd = {k: v.requires_grad_(True) for k, v in sd.items()}
    sd[head + head_proj + ".bias"] = sd[head + "bias"]
    return sd


def oracle_train(steps, warmup, batch):
    """Times the reference's algorithm (oracle/vyom_oracle.py restatement, fp32, all host threads) on a
    bounded sample of the same workload: forward + shifted CE + backward + AdamW, `batch` samples/step."""
    from oracle import vyom_oracle as O
    sd = oracle_state_dict()
    params = [v for k, v in sd.items() if v.requires_grad and k != "decoder.lm_head.decoder.bias"]
    opt = torch.optim.AdamW(params, lr=1e-5)
    cfg = O.Cfg(768, 12, 4, 514, 8, 50265, 1e-5, "gelu")
    vcfg = O.Cfg(768, 12, None, 514, 4, 0, 1e-5, "gelu", (224, 224), (16, 16), 3)
    times = []
    for it in range(warmup + steps):
        px, ids, mask = synth_batch(batch, 1000 + it, False)
        labels = ids.masked_fill(mask == 0, -100)
        t0 = time.perf_counter()
        opt.zero_grad(set_to_none=True)
        logits = O.vlm_forward(sd, cfg, vcfg, px, ids, mask, "rope", "gqa")
        loss = O.cross_entropy_shifted(logits[:, 1:], labels)
        loss.backward()
        torch.nn.utils.clip_grad_norm_(params, 1.0)
        opt.step()
        dt = time.perf_counter() - t0
        if it >= warmup:
            times.append(dt)
    return batch / (sum(times) / len(times)), sum(times) / len(times)


def oracle_train_slots(steps, warmup, batch):
    """The same for the notebook-II form: oracle ViT (all 197 tokens) -> slot_vlm_forward (training mask) -> slot_loss -> AdamW."""
    from oracle import vyom_oracle as O
    sd = oracle_state_dict(SlotTextCfg, SlotVitCfg, head="lm_head.", head_proj="vocab")
    params = [v for k, v in sd.items() if v.requires_grad and k != "lm_head.vocab.bias"]
    opt = torch.optim.AdamW(params, lr=1e-5, weight_decay=0.0)
    cfg = O.Cfg(768, 12, None, 514, 8, SlotTextCfg.vocab_size, 1e-7, "gelu")
    vcfg = O.Cfg(768, 12, None, 514, 12, 0, 1e-5, "gelu", (224, 224), (16, 16), 3)
    times = []
    for it in range(warmup + steps):
        px, ids, mask = synth_slot_batch(batch, 2000 + it, False)
        t0 = time.perf_counter()
        opt.zero_grad(set_to_none=True)
        feats = O.vit_forward(sd, vcfg, px, pre="encoder.")
        logits = O.slot_vlm_forward(sd, cfg, feats, ids, mask, True, SLOTS_IMAGE_TOKEN)
        loss = O.slot_loss(logits, ids, mask, SlotTextCfg.pad_token_id, SLOTS_IMAGE_TOKEN)
        loss.backward()
        torch.nn.utils.clip_grad_norm_(params, 1.0)
        opt.step()
        dt = time.perf_counter() - t0
        if it >= warmup:
            times.append(dt)
    return batch / (sum(times) / len(times)), sum(times) / len(times)


def host_threads():
    """All host cores for the CPU arm. torchrun exports OMP_NUM_THREADS=1 to its workers, which made round 1's N > 1 reference
    lines single-threaded: set the intra-op pool explicitly."""
    n = os.cpu_count() or 1
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        pass
    torch.set_num_threads(n)
    return torch.get_num_threads()


def run_reference(args):
    """Reference arm: the reference's CPU path (oracle port: the reference has no setup.py / pyproject, nothing installs
    under baseline/_ref) on ALL host threads, same model / sequence length / per-step batch as one GPU of our arm. If the
    first (warm-up) step shows that K + W steps of 64 samples would not end within ~4.5 minutes on this host, the per-step
    sample is cut to the largest multiple of 8 that does, and the line says so."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = host_threads()
    slots = args.workload == "slots"
    train = oracle_train_slots if slots else oracle_train
    ours_batch = SLOTS_BATCH if slots else PER_GPU_BATCH
    probe_n = 2 if slots else CPU_SAMPLE_BATCH
    batch = ours_batch
    t0 = time.perf_counter()
    train(1, 0, probe_n)  # probe: one small step (also pages the libraries in)
    probe = time.perf_counter() - t0
    est = probe * (batch / probe_n) * (args.steps + args.warmup)
    if est > 270.0:
        batch = max(probe_n, int(batch * 270.0 / est) // probe_n * probe_n)
    v, sec = train(args.steps, args.warmup, batch)
    sample = (f"{batch} samples per step (same model, S={SLOTS_SEQ if slots else TEXT_LEN + 1}, fp32; our arm: {ours_batch} per GPU), {args.steps} timed steps after "
              f"{args.warmup} warm-up, {cores} host threads")
    line = {
        "impl": "reference", "metric": "caption_train_samples_per_s", "value": v, "unit": "samples/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": SLOTS_WORKLOAD if slots else WORKLOAD, "per_gpu_batch": batch, "per_step_samples": batch,
                   "seq_len": SLOTS_SEQ if slots else TEXT_LEN + 1,
                   "host": "cpu oracle port of the reference path (rank 0 only)"},
        "cpu_baseline": {"value": v, "unit": "samples/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": v, "unit": "samples/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# this repo's arm
# ------------------------------------------------------------------------------------------------
FAMILIES = (  # kernel-name fragment -> C-ABI entry point it belongs to (first match wins)
    ("dp_barrier", "vy_dp_barrier (includes the wait for the peers)"), ("dp_reduce", "vy_dp_reduce_shard"), ("dp_adamw", "vy_dp_adamw_shard"),
    ("gemm_kernel", "vy_gemm"), ("splitk_reduce", "vy_gemm"), ("attn_fwd_kernel", "vy_attn_fwd"), ("attn_bwd", "vy_attn_bwd"),
    ("attn_dsum", "vy_attn_bwd"), ("add_layernorm_fwd", "vy_add_layernorm_fwd"), ("add_layernorm_bwd", "vy_add_layernorm_bwd"),
    ("norm_bwd", "vy_add_layernorm_bwd"), ("adamw", "vy_adamw"), ("sqnorm", "vy_sqnorm"), ("xent", "vy_softmax_xent"),
    ("colsum", "vy_colsum"), ("embed_bwd", "vy_embed_bwd"), ("embed_fwd", "vy_embed_fwd"), ("patchify", "vy_patchify"),
    ("cast4d", "vy_cast4d"), ("act_bwd", "vy_act_bwd"), ("scale_by_ptr", "vy_scale_by_ptr"), ("attn_decode", "vy_attn_decode"),
    ("decode_step", "vy_decode_step"), ("argmax", "vy_argmax_rows"), ("nccl", "nccl"), ("Memcpy", "memcpy"), ("Memset", "memset"),
)


def family_of(kernel_name):
    for frag, fam in FAMILIES:
        if frag in kernel_name:
            return fam
    return "torch_glue"


def replay_profile(step, steps=2):
    """Per-family device time of the step AS TIMED (CUDA-graph replays under CUPTI through torch.profiler): {family:
    {"calls": per step, "ms": per step}}. Round 1's table came from an eager step with events around every call, whose small
    kernels were inflated and whose sum exceeded ms_per_step."""
    from collections import defaultdict
    step()
    torch.cuda.synchronize()
    with torch.profiler.profile(activities=[torch.profiler.ProfilerActivity.CUDA]) as prof:
        for _ in range(steps):
            step()
        torch.cuda.synchronize()
    agg = defaultdict(lambda: [0, 0.0])
    for ev in prof.events():
        if ev.device_type != torch.autograd.DeviceType.CUDA:
            continue
        fam = family_of(ev.name)
        agg[fam][0] += 1
        agg[fam][1] += ev.device_time_total
    return {k: {"calls": n / steps, "ms": t / steps / 1e3} for k, (n, t) in agg.items()}


class DecodeCfg:  # BASELINE config 3: GPT-style CLM, kv-cache, prefill 512 + greedy decode 256, batch 32
    hidden_size = 768
    num_attention_heads = 12
    max_position_embeddings = 1024
    num_hidden_layers = 4
    vocab_size = 50265
    hidden_dropout_prob = 0.0
    layer_norm_eps = 1e-05
    hidden_act = "gelu"
    pad_token_id = 1
    eos_token_id = 2


def decode_config3(dev, attn, batch=32, prefill=512, new_tokens=256, base=None, kv_heads=4, tag="decoder_clm_L4"):
    """Prefill + greedy decode of BASELINE config 3 through DecoderModel.generate (static cache, one CUDA-graph replay per
    token). Returns prefill tok/s, decode tok/s (device time of the replayed steps), the HBM roofline fraction of a decode
    step (algorithmic bytes = every weight but the embedding table + the kv-cache rows read, at the mean context) and
    generate()'s wall clock."""
    import io
    from contextlib import redirect_stdout
    from vyomai_b200 import DecoderModel
    base = base or DecodeCfg
    cfg = type("Cfg3", (base,), {"num_key_value_heads": kv_heads})() if attn == "gqa" else base()
    torch.manual_seed(0)
    with redirect_stdout(io.StringIO()):
        model = DecoderModel(cfg, "rope", "gqa" if attn == "gqa" else None)
    model = model.to(dev).to(torch.bfloat16).eval()
    B, P, N = batch, prefill, new_tokens
    ids = torch.randint(3, cfg.vocab_size, (B, P), device=dev)
    mask = torch.ones((B, P), device=dev, dtype=torch.long)
    hkv = kv_heads if attn == "gqa" else cfg.num_attention_heads
    model.generate(ids, mask, max_len=N, use_cache=True, use_static_cache=True)  # warm-up: tunes the GEMMs, captures the graph
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    out = model.generate(ids, mask, max_len=N, use_cache=True, use_static_cache=True)
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
    kv = model._decode_graph_cache
    with torch.no_grad():
        model(ids, mask, use_cache=True, kv_cache=kv, start_pos=0, _logits_last_only=True)  # (one-time tuning / lazy module loads)
        e0.record()
        model(ids, mask, use_cache=True, kv_cache=kv, start_pos=0, _logits_last_only=True)
        e1.record()
        g = model._decode_graph
        g.pos.fill_(P)
        for _ in range(N - 1):
            g.graph.replay()
        e2.record()
    torch.cuda.synchronize()
    pre_ms, step_us = e0.elapsed_time(e1), e1.elapsed_time(e2) * 1e3 / (N - 1)
    n_params = sum(p.numel() for n, p in model.named_parameters() if "word_embeddings" not in n)
    step_bytes = 2.0 * n_params + 2.0 * B * cfg.num_hidden_layers * 2 * hkv * (P + N / 2) * 64
    hbm = peaks()[0]
    return {"workload": f"{tag}_{attn}_B{B}_prefill{P}_decode{N}_bf16_staticcache",
            "prefill_tok_per_s": B * P / (pre_ms / 1e3), "decode_tok_per_s": B / (step_us * 1e-6), "decode_us_per_step": step_us,
            "decode_step_algorithmic_MB": step_bytes / 1e6, "decode_hbm_frac": step_bytes / (step_us * 1e-6) / 1e9 / hbm,
            "generate_tok_per_s_wall": B * N / wall, "tokens_checked": int(out.shape[1]),
            "step_kernel": "vy_decode_step" if getattr(g, "fused", None) is not None else "per-op graph"}

def build_package_model():
    from vyomai_b200 import VisionLanguageModel, Vit
    return VisionLanguageModel(TextCfg(), encoder=Vit(VitCfg()), pos_embedding_type="rope", attention_type="gqa")


def build_slots_model():
    from vyomai_b200 import ImageSlotVisionLanguageModel, Vit
    return ImageSlotVisionLanguageModel(Vit(SlotVitCfg()), SlotTextCfg(), decoder_pos_embedding_type="rope")


def slots_labels(ids, mask):
    from vyomai_b200 import slot_caption_labels
    return slot_caption_labels(ids, mask, SlotTextCfg.pad_token_id, SLOTS_IMAGE_TOKEN)


def workload_of(name):
    from vyomai_b200.trainer import caption_labels
    if name == "slots":
        return {"name": SLOTS_WORKLOAD, "batch": SLOTS_BATCH, "seq": SLOTS_SEQ, "synth": synth_slot_batch, "build": build_slots_model,
                "labels": slots_labels, "wd": 0.0}
    return {"name": WORKLOAD, "batch": PER_GPU_BATCH, "seq": TEXT_LEN + 1, "synth": synth_batch, "build": build_package_model,
            "labels": caption_labels, "wd": 0.01}


def measure_slots(dev, steps, warmup):
    """The notebook-II workload on one GPU, appended to the default line: resident-input training steps (CUDA-graph replays)
    timed with CUDA events, and the oracle port of the same step on the host cores (2 samples per step)."""
    import io
    from contextlib import redirect_stdout
    from vyomai_b200.trainer import Trainer
    wl = workload_of("slots")
    torch.manual_seed(0)
    with redirect_stdout(io.StringIO()):
        model = wl["build"]()
    model = model.to(dev).to(torch.bfloat16).train()
    tr = Trainer(model, lr=1e-5, weight_decay=wl["wd"], max_grad_norm=1.0, use_graph=True)
    px, ids, mask = [t.to(dev) for t in wl["synth"](wl["batch"], 23, False)]
    labels = wl["labels"](ids, mask)
    for _ in range(max(warmup, 3)):
        loss = tr.caption_step(px, ids, mask, labels)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        loss = tr.caption_step(px, ids, mask, labels)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    # the notebook's own per-GPU batch (8: `prep(batch_size=8)`), same model and trainer (the step is re-captured for the new shape)
    px8, ids8, mask8 = [t.to(dev) for t in wl["synth"](8, 29, False)]
    labels8 = wl["labels"](ids8, mask8)
    for _ in range(3):
        tr.caption_step(px8, ids8, mask8, labels8)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(steps):
        tr.caption_step(px8, ids8, mask8, labels8)
    e1.record()
    torch.cuda.synchronize()
    ms8 = e0.elapsed_time(e1) / steps
    cores = host_threads()
    v, sec = oracle_train_slots(1, 1, 2)
    n_params = sum(p.numel() for p in model.parameters())
    return {"workload": wl["name"], "per_gpu_batch": wl["batch"], "seq_len": wl["seq"], "image_tokens": SLOTS_IMG, "ms_per_step": ms,
            "samples_per_s": wl["batch"] / (ms / 1e3), "tokens_per_s": wl["batch"] * wl["seq"] / (ms / 1e3), "params_M": round(n_params / 1e6, 1),
            "final_loss": float(loss), "grad_overwrite": bool(tr.grad_overwrite), "kernels_per_step": tr.graph_kernels,
            "notebook_batch_8": {"ms_per_step": ms8, "samples_per_s": 8 / (ms8 / 1e3)},
            "cpu_port": {"value": v, "unit": "samples/s", "cores": cores, "sample": f"1 timed step of 2 samples after 1 warm-up ({sec:.1f} s/step)"}}


def _timed_graph(fn, iters=20):
    """Device time per call of `fn` replayed from a CUDA graph (3 eager warm-up calls on a side stream first)."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(3):
            fn()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        fn()
    for _ in range(3):
        graph.replay()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def measure_configs_1_2(dev):
    """BASELINE configs[0] and [1] on this GPU with the oracle port timed beside them on the host cores:
    C1 = EncoderModel (default EncoderConfig, RoPE + GQA kv4), 8 x 128 right-padded tokens, forward + backward of (out . G).sum();
    C2 = Vit 224 / patch 16 (4 layers) + Linear(768, 6) on the CLS row, batch 64, forward. FLOPs: SURVEY.md §8(d)."""
    import io
    from contextlib import redirect_stdout
    from oracle import vyom_oracle as O
    from vyomai_b200 import EncoderConfig, EncoderModel, Vit
    tf_sust = peaks()[2]
    out = {}
    cores = host_threads()
    # ---- C1 ----
    cfg = type("C1", (), dict(vars(EncoderConfig()), num_key_value_heads=4, hidden_dropout_prob=0.0))()
    torch.manual_seed(0)
    with redirect_stdout(io.StringIO()):
        enc = EncoderModel(cfg, pos_embedding_type="rope", attention_type="gqa")
    enc = enc.to(dev).to(torch.bfloat16).train()
    g = torch.Generator().manual_seed(3)
    ids = torch.randint(0, cfg.vocab_size, (8, 128), generator=g)
    lens = torch.randint(16, 129, (8,), generator=g)
    lens[0] = 128
    mask = (torch.arange(128)[None, :] < lens[:, None]).long()
    cot = torch.randn(8, 128, cfg.hidden_size, generator=g) * mask[..., None]
    ids_d, mask_d, cot_d = ids.to(dev), mask.to(dev), cot.to(dev).to(torch.bfloat16)

    def c1_step():
        for p in enc.parameters():
            p.grad = None
        (enc(ids_d, mask_d).logits * cot_d).sum().backward()

    try:
        ms, how = _timed_graph(c1_step), "cuda-graph replay"
    except Exception as e:  # capture refused: time eager launches instead and say so
        torch.cuda.synchronize()
        for _ in range(3):
            c1_step()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(20):
            c1_step()
        e1.record()
        torch.cuda.synchronize()
        ms, how = e0.elapsed_time(e1) / 20, f"eager launches (graph capture failed: {type(e).__name__})"
    sd = {k: v.detach().float().cpu().requires_grad_(v.dtype.is_floating_point) for k, v in enc.state_dict().items()}
    ocfg = O.Cfg(cfg.hidden_size, cfg.num_attention_heads, 4, cfg.max_position_embeddings, cfg.num_hidden_layers, cfg.vocab_size,
                 cfg.layer_norm_eps, cfg.hidden_act)
    ts = []
    for _ in range(3):
        t0 = time.perf_counter()
        for v in sd.values():
            v.grad = None
        (O.encoder_forward(sd, ocfg, ids, mask, "rope", "gqa") * cot).sum().backward()
        ts.append(time.perf_counter() - t0)
    cpu_s = min(ts[1:])
    out["C1_encoder_8x128_fwd_bwd"] = {"ms_per_step": ms, "samples_per_s": 8 / (ms / 1e3), "tflops": 159.0 / ms, "frac_of_sustained_bf16": 159.0 / ms / tf_sust,
                                      "algorithmic_gflop_per_step": 159.0, "timed_as": how, "dtype": "bf16",
                                      "cpu_port": {"samples_per_s": 8 / cpu_s, "cores": cores, "dtype": "f32", "sample": "best of 2 steps after 1 warm-up"}}
    del enc
    # ---- C2 ----
    torch.manual_seed(0)
    with redirect_stdout(io.StringIO()):
        vit = Vit(VitCfg())
    head = torch.nn.Linear(768, 6)
    vit, head = vit.to(dev).to(torch.bfloat16).eval(), head.to(dev).to(torch.bfloat16)
    px = torch.rand(64, 3, 224, 224, generator=g)
    px_d = px.to(dev).to(torch.bfloat16)

    def c2_step():
        with torch.no_grad():
            return head(vit(pixel_values=px_d).logits[:, 0])

    try:
        ms2, how2 = _timed_graph(c2_step), "cuda-graph replay"
    except Exception as e:
        torch.cuda.synchronize()
        for _ in range(3):
            c2_step()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(20):
            c2_step()
        e1.record()
        torch.cuda.synchronize()
        ms2, how2 = e0.elapsed_time(e1) / 20, f"eager launches (graph capture failed: {type(e).__name__})"
    vsd = {k: v.detach().float().cpu() for k, v in vit.state_dict().items()}
    vcfg = O.Cfg(768, 12, None, 514, VitCfg.num_hidden_layers, 0, 1e-5, "gelu", (224, 224), (16, 16), 3)
    with torch.no_grad():
        O.vit_forward(vsd, vcfg, px[:8])
        t0 = time.perf_counter()
        O.vit_forward(vsd, vcfg, px[:16])
        cpu2 = time.perf_counter() - t0
    out["C2_vit224p16_L4_b64_fwd"] = {"ms_per_step": ms2, "images_per_s": 64 / (ms2 / 1e3), "tflops": 759.0 / ms2, "frac_of_sustained_bf16": 759.0 / ms2 / tf_sust,
                                     "algorithmic_gflop_per_step": 759.0, "timed_as": how2, "dtype": "bf16",
                                     "cpu_port": {"images_per_s": 16 / cpu2, "cores": cores, "dtype": "f32", "sample": "one 16-image forward after an 8-image warm-up"}}
    return out


C5_VISION = dict(hidden_size=1152, intermediate_size=4304, num_hidden_layers=27, num_attention_heads=16, num_channels=3, image_size=224,
                 patch_size=14, layer_norm_eps=1e-6)
C5_TEXT = dict(vocab_size=257216, hidden_size=2048, intermediate_size=16384, num_hidden_layers=18, num_attention_heads=8,
               num_key_value_heads=1, head_dim=256, max_position_embeddings=8192, rms_norm_eps=1e-6, rope_theta=10000.0)


def measure_config5(dev, batches=(1, 32), new_tokens=50, cpu=True):
    """BASELINE configs[4]: PaliGemma-scale scratch model (SigLIP 27 x 1152 / 14-pixel patches + Gemma 18 x 2048, 8 q heads,
    1 kv head of 256, GeGLU 16384, vocab 257216, tied head), random init, bf16: prefill of 256 image + 8 text tokens, then
    `new_tokens` greedy tokens through a 384-slot static cache — the procedure of Examples/paligemma.ipynb cell 30.
    HBM floor per decoded token: every weight once (5.02 GB incl. the tied table as lm_head) + the kv rows."""
    from vyomai_b200.models.paligemma import PaliGemmaConfig, PaliGemmaForConditionalGeneration, StaticCache
    out = {"workload": "paligemma_scale_siglip27x1152_gemma18x2048_mqa256_prefill264_decode%d_bf16_staticcache384" % new_tokens}
    try:
        cfg = PaliGemmaConfig(vision_config=dict(C5_VISION), text_config=dict(C5_TEXT), image_token_index=257152, vocab_size=257216,
                              projection_dim=2048, hidden_size=2048, pad_token_id=0)
        old = torch.get_default_dtype()
        torch.set_default_dtype(torch.bfloat16)
        try:
            with torch.device(dev):
                torch.manual_seed(0)
                model = PaliGemmaForConditionalGeneration(cfg)
        finally:
            torch.set_default_dtype(old)
        model.tie_weights()
        model.eval()
        with torch.no_grad():
            for n, p in model.named_parameters():  # N(0, 0.02) like a scratch init; norms near identity
                if p.dim() >= 2:
                    p.normal_(0.0, 0.02)
        n_params = sum(p.numel() for p in model.parameters())
        lm_params = sum(p.numel() for n, p in model.language_model.named_parameters())
        out["params_B"] = round(n_params / 1e9, 3)
        hbm = peaks()[0]
        g = torch.Generator().manual_seed(5)
        for B in batches:
            ids = torch.cat([torch.full((B, 256), 257152, dtype=torch.long), torch.randint(2, 250000, (B, 8), generator=g)], dim=1).to(dev)
            mask = torch.ones((B, 264), dtype=torch.long, device=dev)
            px = torch.rand((B, 3, 224, 224), generator=g).to(dev).to(torch.bfloat16)

            from vyomai_b200 import ops
            from vyomai_b200.models.paligemma import PaliGemmaDecodeGraph

            def run(n_new):
                cache = StaticCache(cfg.text_config, batch_size=B, device=dev, dtype=torch.bfloat16, max_cache_len=384)
                ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
                ev[0].record()
                o = model(input_ids=ids, pixel_values=px, attention_mask=mask, past_key_values=cache, use_cache=True, logits_last_only=True)
                first = ops.argmax_rows(o.logits[:, -1])
                ev[1].record()
                g_ = PaliGemmaDecodeGraph(model, cache, mask)
                g_.tok.copy_(first)
                g_.pos.fill_(264)
                g_.capture()  # (one eager warm-up step + the capture: outside the timed region)
                toks = torch.empty((B, n_new - 1), dtype=torch.long, device=dev)
                torch.cuda.synchronize()
                ev[2].record()
                g_.run(first, 264, n_new - 1, toks)
                ev[3].record()
                torch.cuda.synchronize()
                return ev[0].elapsed_time(ev[1]), ev[2].elapsed_time(ev[3]) / (n_new - 1)

            run(4)  # warm-up: weight packing, GEMM tuning, lazy module loads
            pre_ms, step_ms = run(new_tokens)
            kv_bytes = 2.0 * B * 18 * 2 * 1 * (264 + new_tokens / 2) * 256
            step_bytes = 2.0 * lm_params + kv_bytes  # (tied table counted once: it is read as the lm_head)
            out[f"B{B}"] = {"prefill_ms": pre_ms, "prefill_tok_per_s": B * 264 / (pre_ms / 1e3), "decode_ms_per_step": step_ms,
                            "decode_tok_per_s": B / (step_ms / 1e3), "decode_step_algorithmic_GB": step_bytes / 1e9,
                            "decode_hbm_frac": step_bytes / (step_ms / 1e3) / 1e9 / hbm,
                            "timed_as": "prefill: eager launches; decode: one CUDA-graph replay per token; CUDA events"}
        del model
        torch.cuda.empty_cache()
    except Exception as e:  # the headline line must still be printed
        out["error"] = f"{type(e).__name__}: {str(e)[:300]}"
        return out
    if cpu:
        try:
            import psutil
            if psutil.virtual_memory().available < 48e9:
                out["cpu_port"] = {"skipped": "less than 48 GB of free host memory for the fp32 weights (11.7 GB) and activations"}
                return out
            from oracle import vyom_oracle as O
            cores = host_threads()
            t0 = time.perf_counter()
            sd = {}
            gg = torch.Generator().manual_seed(1)

            def w(name, *shape):
                sd[name] = torch.empty(shape).normal_(0.0, 0.02, generator=gg)

            t = C5_TEXT
            w("language_model.model.embed_tokens.weight", t["vocab_size"], t["hidden_size"])
            sd["language_model.lm_head.weight"] = sd["language_model.model.embed_tokens.weight"]
            for i in range(t["num_hidden_layers"]):
                lp = f"language_model.model.layers.{i}."
                w(lp + "self_attn.q_proj.weight", 2048, 2048); w(lp + "self_attn.k_proj.weight", 256, 2048)
                w(lp + "self_attn.v_proj.weight", 256, 2048); w(lp + "self_attn.o_proj.weight", 2048, 2048)
                w(lp + "mlp.gate_proj.weight", 16384, 2048); w(lp + "mlp.up_proj.weight", 16384, 2048); w(lp + "mlp.down_proj.weight", 2048, 16384)
                sd[lp + "input_layernorm.weight"] = torch.zeros(2048); sd[lp + "post_attention_layernorm.weight"] = torch.zeros(2048)
            sd["language_model.model.norm.weight"] = torch.zeros(2048)
            build_s = time.perf_counter() - t0
            cfgd = {"hidden_size": 2048, "image_token_index": 257152, "text": t, "vision": C5_VISION}
            ids = torch.randint(2, 250000, (1, 264), generator=gg)  # text-only prompt of the same length: the decode steps are what is timed
            mask = torch.ones(1, 264, dtype=torch.long)
            cache = ([torch.zeros(1, 1, 384, 256) for _ in range(18)], [torch.zeros(1, 1, 384, 256) for _ in range(18)])
            with torch.no_grad():
                t0 = time.perf_counter()
                lg = O.paligemma_forward(sd, cfgd, ids, None, mask, cache=cache, seen=0, cache_len=384)
                pre_s = time.perf_counter() - t0
                nxt = lg[:, -1].argmax(-1, keepdim=True)
                ts = []
                for s in range(3):
                    mask = torch.cat([mask, torch.ones(1, 1, dtype=mask.dtype)], -1)
                    t0 = time.perf_counter()
                    lg = O.paligemma_forward(sd, cfgd, nxt, None, mask, cache=cache, seen=264 + s, cache_len=384)
                    ts.append(time.perf_counter() - t0)
                    nxt = lg[:, -1].argmax(-1, keepdim=True)
            out["cpu_port"] = {"decode_tok_per_s": 1.0 / min(ts), "prefill_tok_per_s": 264 / pre_s, "cores": cores, "dtype": "f32", "batch": 1,
                               "sample": f"Gemma decoder only (text prompt of 264 tokens), 3 decode steps, best; weights built in {build_s:.0f} s"}
        except Exception as e:
            out["cpu_port"] = {"error": f"{type(e).__name__}: {str(e)[:200]}"}
    return out


def _guarded(fn, *a, **kw):
    """The appended measurements must never cost the headline line: a failure is reported in place of the numbers."""
    try:
        return fn(*a, **kw)
    except Exception as e:  # noqa: BLE001
        torch.cuda.synchronize()
        return {"error": f"{fn.__name__}: {type(e).__name__}: {str(e)[:300]}"}


def run_ours(args):
    import torch.distributed as dist
    from vyomai_b200 import _lib
    from vyomai_b200.trainer import HostPrefetcher, Trainer
    wl = workload_of(args.workload)
    caption_labels = wl["labels"]

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    L = _lib.lib()  # raises if the CUDA library is missing: there is no fallback

    torch.manual_seed(0)
    import io
    from contextlib import redirect_stdout
    with redirect_stdout(io.StringIO()):
        model = wl["build"]()
    model = model.to(dev).to(torch.bfloat16).train()
    trainer = Trainer(model, lr=1e-5, weight_decay=wl["wd"], max_grad_norm=1.0, use_graph=not args.no_graph,
                      grad_overwrite=not args.no_grad_overwrite, overlap=not args.no_overlap, bucket_mb=args.bucket_mb,
                      dp_mode=args.dp_mode)

    B = wl["batch"]
    host = [wl["synth"](B, 17 + 1000 * rank + i, True) for i in range(2)]
    px_d, ids_d, mask_d = [t.to(dev) for t in host[0]]
    labels_d = caption_labels(ids_d, mask_d)

    def sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def step_resident():
        return trainer.caption_step(px_d, ids_d, mask_d, labels_d)

    # end to end: every step's batch comes from pinned host memory (copied on a side stream one step ahead, like a
    # pin_memory DataLoader) and the step's loss is read back to the host before the next step starts
    feeder = HostPrefetcher(host, dev)

    def step_e2e(i):
        px, ids, mask = feeder.next()  # this step's inputs; issues the H2D copy of the next step's batch
        loss = trainer.caption_step(px, ids, mask, caption_labels(ids, mask))
        return float(loss)  # device -> host read of the step's result

    for _ in range(args.warmup):
        step_resident()
    sync()
    sampler = ClockSampler(local)
    sampler.start()
    launches0 = L.vy_launch_count() + trainer.replayed_kernels
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        loss = step_resident()
    e1.record()
    sync()
    ms = e0.elapsed_time(e1)
    launches = L.vy_launch_count() + trainer.replayed_kernels - launches0
    sampler.stop_flag = True
    sampler.join(timeout=2)
    t = torch.tensor([ms], device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t[0])
    value = world * B * args.steps / (ms / 1e3)

    # end to end: pinned host inputs -> H2D every step, loss read back every step
    for i in range(2):
        step_e2e(i)
    sync()
    e0.record()
    for i in range(args.steps):
        last = step_e2e(i)
    e1.record()
    sync()
    t = torch.tensor([e0.elapsed_time(e1)], device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_value = world * B * args.steps / (float(t[0]) / 1e3)
    h2d = sum(x.numel() * x.element_size() for x in host[0])

    # Algorithmic work per kernel family: one instrumented EAGER step (the C-ABI wrappers count FLOPs / bytes per call; its
    # timings are not used). Time per family: CUPTI over the captured step as it is replayed in the timed region.
    _lib.TIMER = _lib.KernelTimer()
    trainer._caption_body(px_d, ids_d, mask_d, labels_d)
    work = _lib.TIMER.summary()
    _lib.TIMER = None
    prof = replay_profile(step_resident) if not args.no_graph else {k: {"calls": v["calls"], "ms": v["ms"]} for k, v in work.items()}
    hbm, tf_burst, tf_sust, src = peaks()
    traffic = None  # DRAM bytes per launch of the dominant kernel from the committed ncu --set full capture
    for tname in ("r02_gemm_traffic.json", "r01_gemm_traffic.json"):  # r02: mean over two whole steps (350 launches); r01: 6 launches
        tpath = os.path.join(ROOT, "profiles", tname)
        if os.path.exists(tpath):
            traffic = json.load(open(tpath)).get("dram_bytes_per_launch_mean")
            break
    # the device barriers of the data-parallel step only wait for the other ranks (and absorb the profiler's skew): not work
    ours = {k: v for k, v in prof.items() if k.startswith("vy_") and not k.startswith("vy_dp_barrier")}
    total_ms = sum(d["ms"] for k, d in prof.items() if not k.startswith("vy_dp_barrier"))
    name, d = max(ours.items(), key=lambda kv: kv[1]["ms"])
    w = work.get(name, {"flops": 0.0, "bytes": 0.0})
    timed_as = "cuda-graph replay (CUPTI)" if not args.no_graph else "eager step (CUDA events per call)"
    if w["flops"] > 0:
        achieved = w["flops"] / (d["ms"] / 1e3) / 1e12
        roof = {"bound": "tensor", "kernel": name, "achieved": achieved, "peak": tf_sust, "unit": "TFLOP/s",
                "frac": achieved / tf_sust, "traffic": traffic if name == "vy_gemm" else None,
                "peak_source": f"{src} (sustained bf16 GEMM)", "timed_as": timed_as,
                "launches_per_step": d["calls"], "share_of_kernel_time": d["ms"] / total_ms}
    else:
        achieved = w["bytes"] / (d["ms"] / 1e3) / 1e9
        roof = {"bound": "hbm", "kernel": name, "achieved": achieved, "peak": hbm, "unit": "GB/s", "frac": achieved / hbm,
                "traffic": None, "peak_source": src, "timed_as": timed_as, "launches_per_step": d["calls"],
                "share_of_kernel_time": d["ms"] / total_ms}
    breakdown = {}
    for k, v in sorted(prof.items(), key=lambda kv: -kv[1]["ms"]):
        wk = work.get(k, {"flops": 0.0, "bytes": 0.0})
        breakdown[k] = {"calls": round(v["calls"], 1), "ms": round(v["ms"], 3),
                        "tflops": round(wk["flops"] / (v["ms"] / 1e3) / 1e12, 1) if wk["flops"] else None,
                        "gbs": round(wk["bytes"] / (v["ms"] / 1e3) / 1e9, 1) if wk["bytes"] else None}

    final_loss = float(loss)
    poisoned = _lib.lib().vy_gemm_poisoned()
    if poisoned != 0:
        raise RuntimeError(f"vy_gemm_poisoned() = {poisoned}: a wait inside a GEMM kernel timed out, the numbers above are void")
    decode = None
    if world == 1 and not args.no_decode:
        # the metric also names decode tok/s: BASELINE config 3, GQA and MHA, on this GPU (inference replicas do not interact,
        # so it is measured at N = 1 only)
        decode = {a: _guarded(decode_config3, dev, a) for a in ("gqa", "mha")}
    small = None
    if world == 1 and args.workload == "package" and not args.no_configs_1_2:
        small = _guarded(measure_configs_1_2, dev)  # BASELINE configs[0], [1]
    c5 = None
    if world == 1 and args.workload == "package" and not args.no_config5:
        c5 = measure_config5(dev, cpu=not args.no_cpu_baseline)  # BASELINE configs[4]
    slots = None
    if world == 1 and args.workload == "package" and not args.no_slots:
        slots = _guarded(measure_slots, dev, args.steps, args.warmup)  # BASELINE configs[3] in its notebook-II form, same GPU
    if rank == 0:
        cpu = None
        if world == 1 and not args.no_cpu_baseline:
            cores = host_threads()
            nb = CPU_SAMPLE_BATCH if args.workload == "package" else 2
            v, sec = (oracle_train if args.workload == "package" else oracle_train_slots)(1, 1, nb)
            cpu = {"value": v, "unit": "samples/s", "cores": cores, "kind": "port",
                   "sample": f"1 timed step of {nb} samples after 1 warm-up step (oracle port, fp32, {sec:.1f} s/step)"}
        line = {
            "metric": "caption_train_samples_per_s", "value": value, "unit": "samples/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": wl["name"], "per_gpu_batch": B, "global_batch": B * world, "seq_len": wl["seq"],
                       "parallelism": f"dp{world}", "dp_step": trainer.dp_mode, "l2": "per-step working set (GBs of activations) exceeds the 126 MB L2",
                       "dropout": 0.0, "optimizer": "AdamW fp32 master + clip 1.0",
                       "cuda_graph": not args.no_graph, "grad_overwrite": bool(trainer.grad_overwrite)},
            "e2e": {"value": e2e_value, "unit": "samples/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4},
            "gpu_launches": int(launches), "clocks": sampler.result(), "roofline": roof, "cpu_baseline": cpu,
            "kernel_breakdown_ms": breakdown, "kernel_breakdown_sum_ms": round(total_ms, 3),
            **({"kernel_breakdown_note": "rank 0 under the profiler; the device barriers' time is the wait for the other ranks (profiling skews "
                                         "them) and is left out of kernel_breakdown_sum_ms and of the roofline's share"} if world > 1 else {}),
            "decode": decode, "notebook_II": slots, "configs_1_2": small, "config_5": c5,
            "final_loss": final_loss, "e2e_last_loss": last,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        # NCCL communicators that were captured into CUDA graphs do not always tear down cleanly
        # (destroy_process_group was seen to hang after the result line was out): synchronise, then leave.
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)



# ------------------------------------------------------------------------------------------------
# --workload hybrid: the Gelutar hybrid decoder beside DecoderModel at equal width / depth / vocabulary
# ------------------------------------------------------------------------------------------------
HYBRID_KERNELS = ("linear_attn_chunk", "linear_attn", "delta_rule", "window_attn", "causal_conv", "rms_norm", "kv_page_write", "qk_norm_write",
                  "linear_plain", "unary", "embed_rows", "gemm_skinny", "gemm_kernel", "attn_fwd", "attn_decode", "add_layernorm", "argmax")


def hybrid_config(width, layers=8, vocab=32768, window=512):
    """A realistic layer stack: three fixed-decay linear-attention layers, then one parallel (windowed softmax + gated delta) layer,
    repeated; 128-wide heads, feed-forward 4 x width."""
    H = width // 128
    lin = {"type": "lightning", "mixer": {"heads": H, "dim": 128, "vdim": 128, "decay": [1.0 - 2.0 ** -(3 + 5 * i / max(H - 1, 1)) for i in range(H)]},
           "mlp": {"kind": "dense", "ff": 4 * width}}
    par = {"type": "parallel", "mixer": {"left": {"heads": H, "kv_heads": max(H // 4, 1), "dim": 128, "vdim": 128, "scale": 128 ** -0.5,
                                                  "mask": {"size": window, "keep_first": 4}},
                                         "right": {"heads": H, "kv_heads": max(H // 2, 1), "dim": 128, "vdim": 128, "conv": 4}},
           "mlp": {"kind": "dense", "ff": 4 * width}}
    return {"architecture": "Gelutar", "vocab": vocab, "width": width, "embedding": {"scale": 1.0}, "norm": {"eps": 1e-6}, "logit_scale": 1.0,
            "layers": [par if i % 4 == 3 else lin for i in range(layers)]}


def _kernel_table(fn, names=HYBRID_KERNELS):
    """Device time per kernel family of one call of fn (CUPTI through torch.profiler): {fragment: {"calls", "ms"}}."""
    from collections import defaultdict
    torch.cuda.synchronize()
    with torch.profiler.profile(activities=[torch.profiler.ProfilerActivity.CUDA]) as prof:
        fn()
        torch.cuda.synchronize()
    agg = defaultdict(lambda: [0, 0.0])
    for ev in prof.events():
        if ev.device_type != torch.autograd.DeviceType.CUDA:
            continue
        fam = next((n for n in names if n in ev.name), "other")
        agg[fam][0] += 1
        agg[fam][1] += ev.device_time_total
    return {k: {"calls": n, "ms": round(t / 1e3, 4)} for k, (n, t) in sorted(agg.items(), key=lambda kv: -kv[1][1])}


def measure_hybrid(dev, width, batch_prefill=4, prompt=2048, batch_decode=32, decode_steps=64, steps=5, warmup=3):
    from vyomai_b200 import GelutarConfig, GelutarForCausalLM, HybridBatchEngine, HybridCacheManager
    cfgd = hybrid_config(width)
    cfg = GelutarConfig(cfgd)
    model = GelutarForCausalLM(cfg, GelutarForCausalLM.random_weights(cfg, seed=0, low_rank=64), dtype=torch.bfloat16, device=dev,
                               kv_dtype=torch.float32)
    hbm, tf_burst, _, src = peaks()
    g = torch.Generator().manual_seed(1)
    flush = torch.empty(160 * 1024 * 1024, dtype=torch.uint8, device=dev)   # > L2, rewritten between timed iterations
    out = {"width": width, "layers": [L["type"] for L in cfgd["layers"]], "vocab": cfg.vocab, "peaks": src}

    # prefill: batch_prefill prompts of `prompt` tokens as one packed step, pinned host ids -> device inside the timed region
    mgr = HybridCacheManager(model, max_tokens=batch_decode * (prompt + decode_steps + 16), block_size=16, max_seqs=batch_decode)
    eng = HybridBatchEngine(model, mgr)
    prompts = [torch.randint(0, cfg.vocab, (prompt,), generator=g).tolist() for _ in range(batch_decode)]

    def prefill(n):
        lg = eng.feed([(i, prompts[i], [prompt - 1]) for i in range(n)])
        return lg

    times = []
    for it in range(warmup + steps):
        flush.fill_(it)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        prefill(batch_prefill)
        e1.record()
        torch.cuda.synchronize()
        eng.release(range(batch_prefill))
        if it >= warmup:
            times.append(e0.elapsed_time(e1))
    pre_ms = sorted(times)[len(times) // 2]
    out["prefill"] = {"batch": batch_prefill, "prompt": prompt, "ms": round(pre_ms, 3), "tok_per_s": round(batch_prefill * prompt / pre_ms * 1e3)}
    out["prefill_kernels"] = _kernel_table(lambda: prefill(batch_prefill))
    # the three sequence mixers are fp32 by definition (scores, weights, state): their roofline is the FMA rate, not the tensor cores'
    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    fp32_tflops = sms * 128 * 2 * 1.965e9 / 1e12          # nominal: 128 FMA lanes per SM at the maximum SM clock
    tokens, lin, par = batch_prefill * prompt, cfgd["layers"][0]["mixer"], cfgd["layers"][3]["mixer"]
    n_lin = sum(1 for L in cfgd["layers"] if L["type"] == "lightning")
    n_par = len(cfgd["layers"]) - n_lin
    W, K = par["left"]["mask"]["size"], par["left"]["mask"]["keep_first"]
    visible = sum(min(p + 1, W) + (min(K, p + 1 - W) if p + 1 > W else 0) for p in range(prompt)) / prompt
    flops = {"linear_attn_chunk": n_lin * tokens * lin["heads"] * (2 * lin["dim"] * lin["vdim"] + 32 * (lin["dim"] + lin["vdim"])) * 2,
             "window_attn": n_par * tokens * par["left"]["heads"] * visible * (par["left"]["dim"] + par["left"]["vdim"]) * 2,
             "delta_rule": n_par * tokens * par["right"]["heads"] * 3 * par["right"]["dim"] * par["right"]["vdim"] * 2}
    out["prefill_fp32_roofline"] = {"fp32_tflops_nominal": round(fp32_tflops, 1)}
    for name, f in flops.items():
        ms = out["prefill_kernels"].get(name, {}).get("ms")
        if ms:
            out["prefill_fp32_roofline"][name] = {"gflop": round(f / 1e9, 1), "tflops": round(f / ms / 1e9, 2), "frac": round(f / ms / 1e9 / fp32_tflops, 3)}
    eng.release(range(batch_prefill))

    # decode: batch_decode sequences at context `prompt`, one token each per step (second step captures the graph)
    prefill(batch_decode)
    nxt = [[int(t)] for t in torch.randint(0, cfg.vocab, (batch_decode,), generator=g)]
    one = lambda: eng.feed([(i, nxt[i], [0]) for i in range(batch_decode)])  # noqa: E731
    for _ in range(4):
        one()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(decode_steps):
        one()
    e1.record()
    torch.cuda.synchronize()
    step_us = e0.elapsed_time(e1) * 1e3 / decode_steps
    cap = next(iter(eng._graphs.values()), None)
    dev_us = None
    if cap is not None:   # device time of the replayed step alone (no host work between replays)
        e0.record()
        for _ in range(8):
            cap.graph.replay()
        e1.record()
        torch.cuda.synchronize()
        dev_us = e0.elapsed_time(e1) * 1e3 / 8
        # (those replays re-ran the last step on the same rows: states moved, bookkeeping did not; the sequences end here)
    n_params = sum(t.numel() for k, t in model_weights_bytes(model))
    state_bytes = sum(v.states[n][0].numel() * 4 * 2 for layer in mgr.views for v in layer for n in v.states) * batch_decode
    win = cfgd["layers"][3]["mixer"]["left"]
    kv_bytes = sum(1 for L in cfgd["layers"] if L["type"] == "parallel") * batch_decode * (win["mask"]["size"] + win["mask"]["keep_first"]) * \
        win["kv_heads"] * (win["dim"] + win["vdim"]) * 4
    step_bytes = 2.0 * n_params + state_bytes + kv_bytes
    out["decode"] = {"batch": batch_decode, "context": prompt, "us_per_step_engine": round(step_us, 1), "us_per_step_device": dev_us and round(dev_us, 1),
                     "tok_per_s": round(batch_decode / step_us * 1e6), "step_algorithmic_MB": round(step_bytes / 1e6, 1),
                     "hbm_frac_device": dev_us and round(step_bytes / (dev_us * 1e-6) / 1e9 / hbm, 3), "graph": cap is not None}
    eng.use_graph = False   # per-kernel times from an eager step: under the graph's dependent launches a kernel's duration includes its wait
    one()
    out["decode_kernels_eager"] = _kernel_table(one)
    eng.release(range(batch_decode))
    del eng, mgr, model
    torch.cuda.empty_cache()

    # the closest existing model at equal width / depth / vocabulary: the RoPE GQA decoder with its static cache and decode graph
    base = type("EqCfg", (DecodeCfg,), {"hidden_size": width, "num_attention_heads": width // 64, "num_hidden_layers": len(cfgd["layers"]),
                                        "vocab_size": cfg.vocab, "max_position_embeddings": prompt + decode_steps + 8})
    out["decoder_model_decode"] = _guarded(decode_config3, dev, "gqa", batch=batch_decode, prefill=prompt, new_tokens=decode_steps, base=base,
                                           kv_heads=max(width // 256, 1), tag=f"decoder_clm_L{len(cfgd['layers'])}_w{width}")
    out["decoder_model_prefill"] = _guarded(decode_config3, dev, "gqa", batch=batch_prefill, prefill=prompt, new_tokens=4, base=base,
                                            kv_heads=max(width // 256, 1), tag=f"decoder_clm_L{len(cfgd['layers'])}_w{width}")
    return out


def model_weights_bytes(model):
    """(name, tensor) of every weight a decode step reads (the embedding table is touched by one row per token)."""
    seen = []
    for L in model.layers:
        seen.append(("inp", L.inp.weight))
        for m in L.mixers:
            for name in ("o", "a2", "g2"):
                if hasattr(m, name):
                    seen.append((name, getattr(m, name).weight))
        if L.mlp is not None:
            seen += [("up", L.mlp.up.weight), ("down", L.mlp.down.weight)]
    seen.append(("head", model.head.weight))
    return seen


def run_hybrid(args):
    from vyomai_b200 import _lib
    if int(os.environ.get("WORLD_SIZE", "1")) > 1 or args.gpus != 1:
        print(json.dumps({"workload": "hybrid", "error": "the hybrid decoder measurement runs on one GPU"}))
        return
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    L = _lib.lib()
    sampler = ClockSampler(0)
    sampler.start()
    n0 = L.vy_launch_count()
    res = [_guarded(measure_hybrid, dev, int(w), steps=max(args.steps // 2, 3), warmup=max(args.warmup, 3)) for w in args.hybrid_sizes.split(",")]
    launches = L.vy_launch_count() - n0
    sampler.stop_flag = True
    sampler.join(timeout=2)
    print(json.dumps({"workload": "hybrid", "metric": "gelutar_prefill_and_decode_tokens_per_s", "n_gpus": 1, "dtype": "bf16 (fp32 residual / scores / state)",
                      "data": "synthetic", "sizes": res, "gpu_launches_total": int(launches), "gemm_poisoned": int(L.vy_gemm_poisoned()),
                      "clocks": sampler.result(), "l2": "160 MB buffer rewritten between timed prefill iterations"}))

# ------------------------------------------------------------------------------------------------
# --workload latent: the Zugunex latent-attention / mixture-of-experts decoder beside the Gelutar hybrid decoder at equal
# width / depth / vocabulary (both run on HybridBatchEngine's packed step)
# ------------------------------------------------------------------------------------------------
LATENT_KERNELS = ("window_attn_tiled", "window_attn_decode", "window_attn_heads_merge", "window_attn_heads", "window_attn", "latent_kv_write", "rope_split", "moe_route", "moe_scale", "moe_sort",
                  "moe_gather", "moe_combine", "linear_tile", "linear_rows", "linear_attn_chunk", "linear_attn", "delta_rule", "delta_prep",
                  "causal_conv", "rms_norm", "kv_page_write", "unary", "embed_rows", "gemm_skinny", "gemm_kernel", "argmax")


def latent_config(width, layers=8, vocab=32768, window=512):
    """A realistic layer stack: 64 + 32 query / key channels and 64 value channels per head, latent rank 192, every second layer
    reading the latent rows of the layer before it, a dense tanh-GELU feed-forward (4 x width) in the first layer and 32 squared-ReLU
    experts of width / 4 (4 chosen) plus a shared expert of width / 2 in the others."""
    H = width // 64
    def mix(i):
        m = {"heads": H, "dim": 64, "rot_dim": 32, "vdim": 64, "kv_rank": 192, "scale": 96 ** -0.5, "mask": {"size": window},
             "rot": {"base": 10000.0, "dims": 32}}
        if i % 2:
            m["kv_from"] = i - 1
        return m
    moe = {"kind": "moe", "expert": {"ff": width // 4}, "router": {"experts": 32, "top": 4, "scale": 2.5}, "shared": {"ff": width // 2}}
    return {"architecture": "Zugunex", "vocab": vocab, "width": width, "norm": {"eps": 1e-6},
            "layers": [{"type": "latent_attention", "mixer": mix(i), "mlp": {"kind": "dense", "ff": 4 * width} if i == 0 else moe} for i in range(layers)]}


def _packed_numbers(dev, model, vocab, batch_prefill, prompt, batch_decode, decode_steps, steps, warmup, kernels=None):
    """Prefill and single-token-step timings of a packed-step model through HybridBatchEngine: prompts from pinned host ids inside the
    timed region with L2 flushed between iterations; decode as CUDA-graph replays; CUPTI kernel tables of one prefill and one eager step."""
    from vyomai_b200 import HybridBatchEngine, HybridCacheManager
    kernels = kernels or LATENT_KERNELS
    g = torch.Generator().manual_seed(1)
    flush = torch.empty(160 * 1024 * 1024, dtype=torch.uint8, device=dev)
    mgr = HybridCacheManager(model, max_tokens=batch_decode * (prompt + decode_steps + 16), block_size=16, max_seqs=batch_decode)
    eng = HybridBatchEngine(model, mgr)
    prompts = [torch.randint(0, vocab, (prompt,), generator=g).tolist() for _ in range(batch_decode)]
    prefill = lambda n: eng.feed([(i, prompts[i], [prompt - 1]) for i in range(n)])  # noqa: E731
    out, times = {}, []
    for it in range(warmup + steps):
        flush.fill_(it)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        prefill(batch_prefill)
        e1.record()
        torch.cuda.synchronize()
        eng.release(range(batch_prefill))
        if it >= warmup:
            times.append(e0.elapsed_time(e1))
    pre_ms = sorted(times)[len(times) // 2]
    out["prefill"] = {"batch": batch_prefill, "prompt": prompt, "ms": round(pre_ms, 3), "tok_per_s": round(batch_prefill * prompt / pre_ms * 1e3)}
    out["prefill_kernels"] = _kernel_table(lambda: prefill(batch_prefill), kernels)
    eng.release(range(batch_prefill))
    prefill(batch_decode)
    nxt = [[int(t)] for t in torch.randint(0, vocab, (batch_decode,), generator=g)]
    one = lambda: eng.feed([(i, nxt[i], [0]) for i in range(batch_decode)])  # noqa: E731
    for _ in range(4):
        one()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(decode_steps):
        one()
    e1.record()
    torch.cuda.synchronize()
    step_us = e0.elapsed_time(e1) * 1e3 / decode_steps
    cap = next(iter(eng._graphs.values()), None)
    dev_us = None
    if cap is not None:
        e0.record()
        for _ in range(8):
            cap.graph.replay()
        e1.record()
        torch.cuda.synchronize()
        dev_us = e0.elapsed_time(e1) * 1e3 / 8
    out["decode"] = {"batch": batch_decode, "context": prompt, "us_per_step_engine": round(step_us, 1), "us_per_step_device": dev_us and round(dev_us, 1),
                     "tok_per_s": round(batch_decode / step_us * 1e6), "graph": cap is not None}
    eng.use_graph = False
    one()
    out["decode_kernels_eager"] = _kernel_table(one, kernels)
    eng.release(range(batch_decode))
    return out


def measure_latent(dev, width, batch_prefill=4, prompt=2048, batch_decode=32, decode_steps=64, steps=5, warmup=3):
    from vyomai_b200 import GelutarConfig, GelutarForCausalLM, ZugunexConfig, ZugunexForCausalLM
    hbm, _, _, src = peaks()
    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    fp32_tflops = sms * 128 * 2 * 1.965e9 / 1e12
    cfgd = latent_config(width)
    cfg = ZugunexConfig(cfgd)
    model = ZugunexForCausalLM(cfg, ZugunexForCausalLM.random_weights(cfg, seed=0), dtype=torch.bfloat16, device=dev)
    out = {"width": width, "vocab": cfg.vocab, "peaks": src, "fp32_tflops_nominal": round(fp32_tflops, 1)}
    z = _packed_numbers(dev, model, cfg.vocab, batch_prefill, prompt, batch_decode, decode_steps, steps, warmup)
    m = cfgd["layers"][0]["mixer"]
    tokens, W = batch_prefill * prompt, m["mask"]["size"]
    visible = sum(min(p + 1, W) for p in range(prompt)) / prompt
    row = m["kv_rank"] + m["rot_dim"]
    # whole prompts attend over per-head expanded keys / values: dim + rot_dim and vdim channels per (query, key, head)
    fl = len(cfgd["layers"]) * tokens * m["heads"] * visible * (m["dim"] + m["rot_dim"] + m["vdim"]) * 2
    ms = z["prefill_kernels"].get("window_attn_tiled", {}).get("ms")
    if ms:
        z["window_attn_tiled_roofline"] = {"gflop": round(fl / 1e9, 1), "tflops": round(fl / ms / 1e9, 2), "frac_of_fp32_nominal": round(fl / ms / 1e9 / fp32_tflops, 3)}
    # single-token attention: the bytes of the visible latent rows, read once per (sequence, layer) if the heads share them through L2
    dk = z["decode_kernels_eager"]   # 8 or more heads per latent row: the heads-as-rows kernel and its merge; else the key-parallel kernel
    ms = sum(dk.get(k, {}).get("ms", 0.0) for k in ("window_attn_heads", "window_attn_heads_merge", "window_attn_decode"))
    if ms:
        by = len(cfgd["layers"]) * batch_decode * min(W, prompt) * row * 4
        dfl = len(cfgd["layers"]) * batch_decode * m["heads"] * min(W, prompt) * (row + m["kv_rank"]) * 2
        z["window_attn_decode_roofline"] = {"MB_rows_once": round(by / 1e6, 1), "frac_of_hbm_rows_once": round(by / (ms * 1e-3) / 1e9 / hbm, 3),
                                            "gflop": round(dfl / 1e9, 2), "tflops": round(dfl / ms / 1e9, 2),
                                            "frac_of_fp32_nominal": round(dfl / ms / 1e9 / fp32_tflops, 3)}
    step_bytes = 2.0 * sum(t.numel() for t in latent_weights(model)) + len(cfgd["layers"]) * batch_decode * min(W, prompt) * row * 4
    if z["decode"]["us_per_step_device"]:
        z["decode"].update(step_algorithmic_MB=round(step_bytes / 1e6, 1),
                           hbm_frac_device=round(step_bytes / (z["decode"]["us_per_step_device"] * 1e-6) / 1e9 / hbm, 3))
    out["zugunex"] = z
    del model
    torch.cuda.empty_cache()
    gd = hybrid_config(width)
    gcfg = GelutarConfig(gd)
    gmodel = GelutarForCausalLM(gcfg, GelutarForCausalLM.random_weights(gcfg, seed=0, low_rank=64), dtype=torch.bfloat16, device=dev)
    gz = _packed_numbers(dev, gmodel, gcfg.vocab, batch_prefill, prompt, batch_decode, decode_steps, steps, warmup)
    par = gd["layers"][3]["mixer"]["left"]
    n_par = sum(1 for L in gd["layers"] if L["type"] == "parallel")
    Wg, K = par["mask"]["size"], par["mask"]["keep_first"]
    vis = sum(min(p + 1, Wg) + (min(K, p + 1 - Wg) if p + 1 > Wg else 0) for p in range(prompt)) / prompt
    fl = n_par * tokens * par["heads"] * vis * (par["dim"] + par["vdim"]) * 2
    ms = gz["prefill_kernels"].get("window_attn_tiled", {}).get("ms")
    if ms:
        gz["window_attn_tiled_roofline"] = {"gflop": round(fl / 1e9, 1), "tflops": round(fl / ms / 1e9, 2), "frac_of_fp32_nominal": round(fl / ms / 1e9 / fp32_tflops, 3)}
    ms = gz["decode_kernels_eager"].get("window_attn_decode", {}).get("ms")
    if ms:
        by = n_par * batch_decode * (Wg + K) * par["kv_heads"] * (par["dim"] + par["vdim"]) * 4
        dfl = n_par * batch_decode * par["heads"] * (Wg + K) * (par["dim"] + par["vdim"]) * 2
        gz["window_attn_decode_roofline"] = {"MB_rows_once": round(by / 1e6, 1), "frac_of_hbm_rows_once": round(by / (ms * 1e-3) / 1e9 / hbm, 3),
                                             "gflop": round(dfl / 1e9, 2), "tflops": round(dfl / ms / 1e9, 2),
                                             "frac_of_fp32_nominal": round(dfl / ms / 1e9 / fp32_tflops, 3)}
    out["gelutar"] = gz
    del gmodel
    torch.cuda.empty_cache()
    return out


def latent_weights(model):
    """Every weight a Zugunex decode step reads (the all-experts form reads every expert once)."""
    seen = []
    for L in model.layers:
        seen += [L.inp.weight, L.mixer.uk_t, L.mixer.uv, L.mixer.o.weight]
        if L.mlp is not None:
            seen += [L.mlp.up_all.weight, L.mlp.down_all.weight, L.mlp.router.weight] if L.moe else [L.mlp.up.weight, L.mlp.down.weight]
    seen.append(model.head.weight)
    return seen


def run_latent(args):
    from vyomai_b200 import _lib
    if int(os.environ.get("WORLD_SIZE", "1")) > 1 or args.gpus != 1:
        print(json.dumps({"workload": "latent", "error": "the latent-attention decoder measurement runs on one GPU"}))
        return
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    L = _lib.lib()
    sampler = ClockSampler(0)
    sampler.start()
    n0 = L.vy_launch_count()
    res = [_guarded(measure_latent, dev, int(w), steps=max(args.steps // 2, 3), warmup=max(args.warmup, 3)) for w in args.hybrid_sizes.split(",")]
    launches = L.vy_launch_count() - n0
    sampler.stop_flag = True
    sampler.join(timeout=2)
    print(json.dumps({"workload": "latent", "metric": "zugunex_prefill_and_decode_tokens_per_s", "n_gpus": 1, "dtype": "bf16 (fp32 residual / scores / router)",
                      "data": "synthetic", "sizes": res, "gpu_launches_total": int(launches), "gemm_poisoned": int(L.vy_gemm_poisoned()),
                      "clocks": sampler.result(), "l2": "160 MB buffer rewritten between timed prefill iterations"}))


# ------------------------------------------------------------------------------------------------
# --workload talking: the Vazepel parallel-layer decoder (score-exchanging attention, gated experts) beside the Zugunex
# latent-attention decoder at equal width / depth / vocabulary (both run on HybridBatchEngine's packed step)
# ------------------------------------------------------------------------------------------------
TALKING_KERNELS = ("talk_attn_tiled", "talk_attn_rows", "talk_attn_merge", "depth_mix_norm", "moe_glu", "rope_kv_write") + LATENT_KERNELS


def talking_config(width, layers=8, vocab=32768):
    """A realistic layer stack: heads of 64 query / key and 64 value channels, 4 query heads per key/value head, all channels rotated, a
    dense tanh-GELU feed-forward (4 x width) in the first layer and 32 gated experts of width / 4 (4 chosen, 8 groups of which 4 are
    kept) plus a shared expert of width / 2 in the others: the same expert sizes as latent_config()."""
    H = width // 64
    mix = {"heads": H, "kv_heads": max(H // 4, 1), "dim": 64, "vdim": 64, "scale": 0.125, "softcap": 30.0, "rot": {"base": 10000.0, "dims": 64}}
    moe = {"kind": "moe", "expert": {"ff": width // 4, "limit": 7.0}, "router": {"experts": 32, "top": 4, "groups": {"count": 8, "keep": 4}},
           "shared": {"ff": width // 2, "limit": 7.0}}
    return {"architecture": "Vazepel", "vocab": vocab, "width": width, "norm": {"eps": 1e-5},
            "layers": [{"type": "attention", "mixer": dict(mix), "mlp": {"kind": "dense", "ff": 4 * width} if i == 0 else moe} for i in range(layers)]}


def talking_weights(model):
    """Every weight a Vazepel decode step reads (the all-experts form reads every expert once)."""
    seen = []
    for L in model.layers:
        seen += [L.inp.weight, L.mixer.o.weight]
        if L.mlp is not None:
            seen += [L.mlp.up_all.weight, L.mlp.down_all.weight] if L.moe else [L.mlp.up.weight, L.mlp.down.weight]
    seen.append(model.head.weight)
    return seen


def measure_talking(dev, width, batch_prefill=4, prompt=2048, batch_decode=32, decode_steps=64, steps=5, warmup=3):
    from vyomai_b200 import VazepelConfig, VazepelForCausalLM, ZugunexConfig, ZugunexForCausalLM
    hbm, _, _, src = peaks()
    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    fp32_tflops = sms * 128 * 2 * 1.965e9 / 1e12
    cfgd = talking_config(width)
    cfg = VazepelConfig(cfgd)
    model = VazepelForCausalLM(cfg, VazepelForCausalLM.random_weights(cfg, seed=0), dtype=torch.bfloat16, device=dev)
    out = {"width": width, "vocab": cfg.vocab, "peaks": src, "fp32_tflops_nominal": round(fp32_tflops, 1)}
    z = _packed_numbers(dev, model, cfg.vocab, batch_prefill, prompt, batch_decode, decode_steps, steps, warmup, kernels=TALKING_KERNELS)
    m = cfgd["layers"][0]["mixer"]
    n_layers, H, G = len(cfgd["layers"]), m["heads"], m["kv_heads"]
    tokens = batch_prefill * prompt
    visible = (prompt + 1) / 2.0
    # prompts: the two contractions (dim + vdim channels per query, key, head) plus the exchange (heads multiply-adds per query, key, head)
    fl = n_layers * tokens * H * visible * (m["dim"] + m["vdim"] + H) * 2
    ms = z["prefill_kernels"].get("talk_attn_tiled", {}).get("ms")
    if ms:
        z["talk_attn_tiled_roofline"] = {"gflop": round(fl / 1e9, 1), "tflops": round(fl / ms / 1e9, 2), "frac_of_fp32_nominal": round(fl / ms / 1e9 / fp32_tflops, 3)}
    dk = z["decode_kernels_eager"]
    ms = sum(dk.get(k, {}).get("ms", 0.0) for k in ("talk_attn_rows", "talk_attn_merge"))
    if ms:
        by = n_layers * batch_decode * prompt * G * (m["dim"] + m["vdim"]) * 4
        dfl = n_layers * batch_decode * H * prompt * (m["dim"] + m["vdim"] + H) * 2
        z["talk_attn_decode_roofline"] = {"MB_rows_once": round(by / 1e6, 1), "frac_of_hbm_rows_once": round(by / (ms * 1e-3) / 1e9 / hbm, 3),
                                          "gflop": round(dfl / 1e9, 2), "tflops": round(dfl / ms / 1e9, 2),
                                          "frac_of_fp32_nominal": round(dfl / ms / 1e9 / fp32_tflops, 3)}
    step_bytes = 2.0 * sum(t.numel() for t in talking_weights(model)) + n_layers * batch_decode * prompt * G * (m["dim"] + m["vdim"]) * 4
    if z["decode"]["us_per_step_device"]:
        z["decode"].update(step_algorithmic_MB=round(step_bytes / 1e6, 1),
                           hbm_frac_device=round(step_bytes / (z["decode"]["us_per_step_device"] * 1e-6) / 1e9 / hbm, 3))
    out["vazepel"] = z
    del model
    torch.cuda.empty_cache()
    # the closest existing model: latent attention over a 512-token window; its attention numbers as --workload latent derives them
    ld = latent_config(width)
    lcfg = ZugunexConfig(ld)
    lmodel = ZugunexForCausalLM(lcfg, ZugunexForCausalLM.random_weights(lcfg, seed=0), dtype=torch.bfloat16, device=dev)
    lz = _packed_numbers(dev, lmodel, lcfg.vocab, batch_prefill, prompt, batch_decode, decode_steps, steps, warmup)
    lm = ld["layers"][0]["mixer"]
    Wn = lm["mask"]["size"]
    vis = sum(min(p + 1, Wn) for p in range(prompt)) / prompt
    fl = len(ld["layers"]) * tokens * lm["heads"] * vis * (lm["dim"] + lm["rot_dim"] + lm["vdim"]) * 2
    ms = lz["prefill_kernels"].get("window_attn_tiled", {}).get("ms")
    if ms:
        lz["window_attn_tiled_roofline"] = {"gflop": round(fl / 1e9, 1), "tflops": round(fl / ms / 1e9, 2), "frac_of_fp32_nominal": round(fl / ms / 1e9 / fp32_tflops, 3)}
    dk = lz["decode_kernels_eager"]
    ms = sum(dk.get(k, {}).get("ms", 0.0) for k in ("window_attn_heads", "window_attn_heads_merge", "window_attn_decode"))
    if ms:
        row = lm["kv_rank"] + lm["rot_dim"]
        by = len(ld["layers"]) * batch_decode * min(Wn, prompt) * row * 4
        dfl = len(ld["layers"]) * batch_decode * lm["heads"] * min(Wn, prompt) * (row + lm["kv_rank"]) * 2
        lz["window_attn_decode_roofline"] = {"MB_rows_once": round(by / 1e6, 1), "frac_of_hbm_rows_once": round(by / (ms * 1e-3) / 1e9 / hbm, 3),
                                             "gflop": round(dfl / 1e9, 2), "tflops": round(dfl / ms / 1e9, 2),
                                             "frac_of_fp32_nominal": round(dfl / ms / 1e9 / fp32_tflops, 3)}
    out["zugunex"] = lz
    del lmodel
    torch.cuda.empty_cache()
    return out


def run_talking(args):
    from vyomai_b200 import _lib
    if int(os.environ.get("WORLD_SIZE", "1")) > 1 or args.gpus != 1:
        print(json.dumps({"workload": "talking", "error": "the parallel-layer decoder measurement runs on one GPU"}))
        return
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    L = _lib.lib()
    sampler = ClockSampler(0)
    sampler.start()
    n0 = L.vy_launch_count()
    res = [_guarded(measure_talking, dev, int(w), steps=max(args.steps // 2, 3), warmup=max(args.warmup, 3)) for w in args.hybrid_sizes.split(",")]
    launches = L.vy_launch_count() - n0
    sampler.stop_flag = True
    sampler.join(timeout=2)
    print(json.dumps({"workload": "talking", "metric": "vazepel_prefill_and_decode_tokens_per_s", "n_gpus": 1, "dtype": "bf16 (fp32 residual / scores / router)",
                      "data": "synthetic", "sizes": res, "gpu_launches_total": int(launches), "gemm_poisoned": int(L.vy_gemm_poisoned()),
                      "clocks": sampler.result(), "l2": "160 MB buffer rewritten between timed prefill iterations"}))

# ------------------------------------------------------------------------------------------------
# --workload fubinex: the Fubinex decoder (latent attention with a query latent, block-local attention beside gated linear
# attention, retention, polynomial feed-forward activation) beside the Gelutar hybrid decoder at equal width / depth / vocabulary
# (both run on HybridBatchEngine's packed step)
# ------------------------------------------------------------------------------------------------
FUBINEX_KERNELS = ("rope_heads", "poly_norm", "gla_prep", "rope_kv_write") + LATENT_KERNELS


def fubinex_config(width, layers=8, vocab=32768, chunk=512):
    """A realistic layer stack, repeated: latent attention (64 + 32 query / key and 64 value channels per head, latent rank 192, query
    latent width / 2), a second latent layer reading the first one's rows, a parallel layer (128-wide heads, 4 query heads per key /
    value head, blocks of `chunk` positions; gated linear attention with 128 x 128 states), a retention layer (128 x 128 states);
    feed-forward 4 x width."""
    H, H2 = width // 64, width // 128
    rot = {"base": 10000.0, "dims": 32, "scaling": {"factor": 8.0, "original": 2048, "fast": 16.0, "slow": 2.0}}
    lat = lambda src: {"heads": H, "dim": 64, "rot_dim": 32, "vdim": 64, "kv_rank": 192, "q_rank": width // 2, "scale": 96 ** -0.5, "rot": rot,  # noqa: E731
                       **({} if src is None else {"kv_from": src})}
    par = {"left": {"heads": H2, "kv_heads": max(H2 // 4, 1), "dim": 128, "vdim": 128, "scale": 128 ** -0.5, "mask": {"size": chunk},
                    "rot": {"base": 10000.0, "dims": 64}}, "left_scale": 0.75,
           "right": {"heads": H2, "dim": 128, "vdim": 128, "tau": 8.0}, "right_scale": 1.25}
    ret = {"heads": H2, "dim": 128, "vdim": 128, "decay": [1.0 - 2.0 ** -(3 + 5 * i / max(H2 - 1, 1)) for i in range(H2)], "rot": {"base": 10000.0, "dims": 128}}
    mlp = {"kind": "dense", "ff": 4 * width}
    out = []
    for i in range(layers):
        kind = i % 4
        if kind == 0:
            out.append({"type": "latent_attention", "mixer": lat(None), "mlp": mlp})
        elif kind == 1:
            out.append({"type": "latent_attention", "mixer": lat(i - 1), "mlp": mlp})
        elif kind == 2:
            out.append({"type": "parallel", "mixer": par, "mlp": mlp})
        else:
            out.append({"type": "retention", "mixer": ret, "mlp": mlp})
    return {"architecture": "Fubinex", "vocab": vocab, "width": width, "embedding": {"scale": 1.0}, "norm": {"eps": 1e-6, "groups": 2}, "layers": out}


def _roof(table, names, flop=None, byts=None, fp32_tflops=None, hbm=None):
    """Achieved rate of the kernel families `names` of a CUPTI table against the fp32 FMA rate and / or the measured copy bandwidth."""
    ms = sum(table.get(k, {}).get("ms", 0.0) for k in names)
    if not ms:
        return None
    r = {"ms": round(ms, 4)}
    if flop:
        r.update(gflop=round(flop / 1e9, 2), tflops=round(flop / ms / 1e9, 2), frac_of_fp32_nominal=round(flop / ms / 1e9 / fp32_tflops, 4))
    if byts:
        r.update(MB=round(byts / 1e6, 2), frac_of_hbm=round(byts / (ms * 1e-3) / 1e9 / hbm, 4))
    return r


def measure_fubinex(dev, width, batch_prefill=4, prompt=2048, batch_decode=32, decode_steps=64, steps=5, warmup=3):
    from vyomai_b200 import FubinexConfig, FubinexForCausalLM, GelutarConfig, GelutarForCausalLM
    hbm, _, _, src = peaks()
    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    fp32_tflops = sms * 128 * 2 * 1.965e9 / 1e12
    cfgd = fubinex_config(width)
    cfg = FubinexConfig(cfgd)
    model = FubinexForCausalLM(cfg, FubinexForCausalLM.random_weights(cfg, seed=0, low_rank=64), dtype=torch.bfloat16, device=dev)
    out = {"width": width, "layers": [L["type"] for L in cfgd["layers"]], "vocab": cfg.vocab, "peaks": src, "fp32_tflops_nominal": round(fp32_tflops, 1)}
    z = _packed_numbers(dev, model, cfg.vocab, batch_prefill, prompt, batch_decode, decode_steps, steps, warmup, kernels=FUBINEX_KERNELS)
    kinds = [L["type"] for L in cfgd["layers"]]
    n_lat, n_par, n_ret, n_all = kinds.count("latent_attention"), kinds.count("parallel"), kinds.count("retention"), len(kinds)
    lat, par, ret = cfgd["layers"][0]["mixer"], cfgd["layers"][2]["mixer"], cfgd["layers"][3]["mixer"]
    lf, rt = par["left"], par["right"]
    tokens, C, ff = batch_prefill * prompt, lf["mask"]["size"], 4 * width
    rf = dict(fp32_tflops=fp32_tflops, hbm=hbm)
    pk, dk = z["prefill_kernels"], z["decode_kernels_eager"]
    # prompts. Attention: two contractions per visible (query, key, head) pair; the tiled kernel serves the causal latent layers (expanded
    # keys: dim + rot_dim and vdim channels) and the block-local layers (mean visible keys (chunk + 1) / 2) alike
    vis_c = sum(p % C + 1 for p in range(prompt)) / prompt
    fl_attn = n_lat * tokens * lat["heads"] * (prompt + 1) / 2.0 * (lat["dim"] + lat["rot_dim"] + lat["vdim"]) * 2 + \
        n_par * tokens * lf["heads"] * vis_c * (lf["dim"] + lf["vdim"]) * 2
    # recurrences: per (token, head) and state element, gated linear attention does a decay multiply and two multiply-adds (5 flop), the
    # chunked fixed-decay kernel is counted as in --workload hybrid
    z["prefill_roofline"] = {
        "window_attn_tiled": _roof(pk, ("window_attn_tiled",), flop=fl_attn, **rf),
        "gated_linear_attn (delta_rule kernel, no correction)": _roof(pk, ("delta_rule",), flop=n_par * tokens * rt["heads"] * rt["dim"] * rt["vdim"] * 5, **rf),
        "linear_attn_chunk": _roof(pk, ("linear_attn_chunk",), flop=n_ret * tokens * ret["heads"] * (2 * ret["dim"] * ret["vdim"] + 32 * (ret["dim"] + ret["vdim"])) * 2, **rf),
        # row kernels against the copy bandwidth: fp32 in, bf16 out (poly_norm); q / k read and written in fp32, v copied (rotation)
        "poly_norm": _roof(pk, ("poly_norm",), byts=n_all * tokens * ff * 6, **rf),
        "rope_heads": _roof(pk, ("rope_heads",), byts=tokens * (n_par * (lf["heads"] + 2 * lf["kv_heads"]) * lf["dim"] + n_ret * 2 * ret["heads"] * ret["dim"]) * 8, **rf),
        "rms_norm": _roof(pk, ("rms_norm",), byts=tokens * ((2 * n_all) * width * 6 + n_lat * lat["q_rank"] * 6 + (n_par * rt["heads"] * rt["vdim"] + n_ret * ret["heads"] * ret["vdim"]) * 10), **rf),
    }
    # single tokens at context `prompt`: attention reads the visible rows once per (sequence, layer); recurrences read and write their state
    row = lat["kv_rank"] + lat["rot_dim"]
    vis_d = prompt % C + 1   # keys of the decoded token's own block (the first steps after a prompt of a whole number of blocks see very few)
    by_lat = batch_decode * n_lat * (prompt + 1) * row * 4
    by_blk = batch_decode * n_par * vis_d * lf["kv_heads"] * (lf["dim"] + lf["vdim"]) * 4
    by_attn = by_lat + by_blk
    z["decode_roofline"] = {
        # 8 or more heads per latent row: heads-as-rows tiles with the keys split over CTAs, bound by the FMA rate (two contractions over
        # kv_rank + rot_dim and kv_rank channels per (head, key)), not by the rows' bytes
        "latent attention (window_attn_heads + merge)": _roof(dk, ("window_attn_heads", "window_attn_heads_merge"), byts=by_lat,
                                                              flop=n_lat * batch_decode * lat["heads"] * (prompt + 1) * (row + lat["kv_rank"]) * 2, **rf),
        "block-local attention (window_attn_decode)": _roof(dk, ("window_attn_decode",), byts=by_blk, **rf),
        "gated_linear_attn": _roof(dk, ("delta_rule",), byts=n_par * batch_decode * rt["heads"] * rt["dim"] * rt["vdim"] * 8, **rf),
        "linear_attn": _roof(dk, ("linear_attn",), byts=n_ret * batch_decode * ret["heads"] * ret["dim"] * ret["vdim"] * 8, **rf),
    }
    step_bytes = 2.0 * sum(t.numel() for t in fubinex_weights(model)) + by_attn + \
        batch_decode * (n_par * rt["heads"] * rt["dim"] * rt["vdim"] + n_ret * ret["heads"] * ret["dim"] * ret["vdim"]) * 8
    if z["decode"]["us_per_step_device"]:
        z["decode"].update(step_algorithmic_MB=round(step_bytes / 1e6, 1),
                           hbm_frac_device=round(step_bytes / (z["decode"]["us_per_step_device"] * 1e-6) / 1e9 / hbm, 3))
    out["fubinex"] = z
    del model
    torch.cuda.empty_cache()
    # the closest existing model: fixed-decay linear attention layers and a parallel (windowed softmax + gated delta rule) layer
    gd = hybrid_config(width)
    gcfg = GelutarConfig(gd)
    gmodel = GelutarForCausalLM(gcfg, GelutarForCausalLM.random_weights(gcfg, seed=0, low_rank=64), dtype=torch.bfloat16, device=dev)
    gz = _packed_numbers(dev, gmodel, gcfg.vocab, batch_prefill, prompt, batch_decode, decode_steps, steps, warmup, kernels=FUBINEX_KERNELS)
    glin, gpar = gd["layers"][0]["mixer"], gd["layers"][3]["mixer"]
    gl, gr = gpar["left"], gpar["right"]
    g_lin = sum(1 for L in gd["layers"] if L["type"] == "lightning")
    g_par = len(gd["layers"]) - g_lin
    Wg, K = gl["mask"]["size"], gl["mask"]["keep_first"]
    vis = sum(min(p + 1, Wg) + (min(K, p + 1 - Wg) if p + 1 > Wg else 0) for p in range(prompt)) / prompt
    gpk, gdk = gz["prefill_kernels"], gz["decode_kernels_eager"]
    gz["prefill_roofline"] = {
        "window_attn_tiled": _roof(gpk, ("window_attn_tiled",), flop=g_par * tokens * gl["heads"] * vis * (gl["dim"] + gl["vdim"]) * 2, **rf),
        # the delta rule adds the correction's contraction: a decay multiply and three multiply-adds per state element (7 flop)
        "delta_rule": _roof(gpk, ("delta_rule",), flop=g_par * tokens * gr["heads"] * gr["dim"] * gr["vdim"] * 7, **rf),
        "linear_attn_chunk": _roof(gpk, ("linear_attn_chunk",), flop=g_lin * tokens * glin["heads"] * (2 * glin["dim"] * glin["vdim"] + 32 * (glin["dim"] + glin["vdim"])) * 2, **rf),
        "unary (relu^2 between the feed-forward products, fp32 in / bf16 out)": _roof(gpk, ("unary",), byts=len(gd["layers"]) * tokens * ff * 6, **rf),
    }
    gz["decode_roofline"] = {
        "window_attn (all single-token forms)": _roof(gdk, ("window_attn_heads", "window_attn_heads_merge", "window_attn_decode"),
                                                      byts=g_par * batch_decode * (Wg + K) * gl["kv_heads"] * (gl["dim"] + gl["vdim"]) * 4, **rf),
        "delta_rule": _roof(gdk, ("delta_rule",), byts=g_par * batch_decode * gr["heads"] * gr["dim"] * gr["vdim"] * 8, **rf),
        "linear_attn": _roof(gdk, ("linear_attn",), byts=g_lin * batch_decode * glin["heads"] * glin["dim"] * glin["vdim"] * 8, **rf),
    }
    out["gelutar"] = gz
    del gmodel
    torch.cuda.empty_cache()
    return out


def fubinex_weights(model):
    """Every weight a Fubinex decode step reads."""
    seen = []
    for L in model.layers:
        seen.append(L.inp.weight)
        for m in L.mixers:
            seen += [getattr(m, n).weight for n in ("o", "uq", "a2") if hasattr(m, n)] + [getattr(m, n) for n in ("uk_t", "uv") if hasattr(m, n)]
        if L.mlp is not None:
            seen += [L.mlp.up.weight, L.mlp.down.weight]
    seen.append(model.head.weight)
    return seen


def run_fubinex(args):
    from vyomai_b200 import _lib
    if int(os.environ.get("WORLD_SIZE", "1")) > 1 or args.gpus != 1:
        print(json.dumps({"workload": "fubinex", "error": "the Fubinex decoder measurement runs on one GPU"}))
        return
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    L = _lib.lib()
    sampler = ClockSampler(0)
    sampler.start()
    n0 = L.vy_launch_count()
    res = [_guarded(measure_fubinex, dev, int(w), steps=max(args.steps // 2, 3), warmup=max(args.warmup, 3)) for w in args.hybrid_sizes.split(",")]
    launches = L.vy_launch_count() - n0
    sampler.stop_flag = True
    sampler.join(timeout=2)
    print(json.dumps({"workload": "fubinex", "metric": "fubinex_prefill_and_decode_tokens_per_s", "n_gpus": 1, "dtype": "bf16 (fp32 residual / scores / state)",
                      "data": "synthetic", "sizes": res, "gpu_launches_total": int(launches), "gemm_poisoned": int(L.vy_gemm_poisoned()),
                      "clocks": sampler.result(), "l2": "160 MB buffer rewritten between timed prefill iterations"}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--workload", default="package", choices=["package", "slots", "hybrid", "latent", "talking", "fubinex"],
                    help="package: VisionLanguageModel of the reference package (1 image token + 127 text, the headline); "
                         "slots: the notebook-II form (197 image tokens in a 248-token sequence); "
                         "hybrid: prefill / decode throughput of the Gelutar hybrid decoder beside DecoderModel at equal size (1 GPU, "
                         "its own JSON line; not the headline metric); "
                         "latent: the same for the Zugunex latent-attention / mixture-of-experts decoder beside Gelutar at equal size; "
                         "talking: the same for the Vazepel parallel-layer decoder (score-exchanging attention heads) beside Zugunex; "
                         "fubinex: the same for the Fubinex decoder (latent / block-local / gated-linear / retention mixers) beside Gelutar")
    ap.add_argument("--hybrid-sizes", default="1024,2048", help="--workload hybrid / latent / talking / fubinex: model widths to measure")
    ap.add_argument("--no-configs-1-2", action="store_true", help="skip the encoder (C1) / ViT (C2) measurements appended at N = 1")
    ap.add_argument("--no-config5", action="store_true", help="skip the PaliGemma-scale prefill + decode measurement appended at N = 1")
    ap.add_argument("--no-slots", action="store_true", help="skip the notebook-II measurement appended at N = 1")
    ap.add_argument("--no-decode", action="store_true", help="skip the config-3 decode measurement appended at N = 1")
    ap.add_argument("--no-grad-overwrite", action="store_true", help="zero + accumulate every gradient instead of overwrite mode")
    ap.add_argument("--no-graph", action="store_true", help="launch every kernel eagerly instead of replaying a CUDA graph")
    ap.add_argument("--no-overlap", action="store_true", help="one gradient all-reduce after backward instead of bucketed overlap")
    ap.add_argument("--dp-mode", default=None, choices=["p2p", "nccl"],
                    help="N > 1: p2p = sharded optimizer step over NVLink peer memory (default), nccl = bucketed all-reduce + full AdamW")
    ap.add_argument("--bucket-mb", type=float, default=64.0, help="gradient bucket size of the overlapped all-reduce")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "hybrid":
        run_hybrid(args)
    elif args.workload == "latent":
        run_latent(args)
    elif args.workload == "talking":
        run_talking(args)
    elif args.workload == "fubinex":
        run_fubinex(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
