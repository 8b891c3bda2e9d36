#!/usr/bin/env python3
"""Benchmark of the engine on one GPU: decode tokens/s (batch 8 by default; batch 1 and 64 as points),
prefill tokens/s at 2,048 tokens, each with its fraction of the measured roofline.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--impl reference]

A "step" is one decode step of the whole batch.  Weights are random (made on the device), token ids are
seeded uniform-random: synthetic data throughout.  One JSON line is printed.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# Llama-3-8B's layer sizes
MODEL = dict(architectures=["LlamaForCausalLM"], model_type="llama", hidden_size=4096, num_hidden_layers=32,
             num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=14336, vocab_size=128256,
             rope_theta=500000.0, rms_norm_eps=1e-5, tie_word_embeddings=False, max_position_embeddings=8192,
             hidden_act="silu", torch_dtype="bfloat16", bos_token_id=128000, eos_token_id=128001)
MODELS = {
    "llama3-8b": MODEL,
    # Llama-3.2-1B's and Llama-2-13B's layer sizes
    "llama3.2-1b": dict(MODEL, hidden_size=2048, num_hidden_layers=16, num_attention_heads=32, num_key_value_heads=8,
                        head_dim=64, intermediate_size=8192, tie_word_embeddings=True, max_position_embeddings=131072,
                        rope_scaling=dict(rope_type="llama3", factor=32.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                          original_max_position_embeddings=8192)),
    "llama2-13b": dict(MODEL, hidden_size=5120, num_hidden_layers=40, num_attention_heads=40, num_key_value_heads=40,
                       head_dim=128, intermediate_size=13824, vocab_size=32000, rope_theta=10000.0,
                       max_position_embeddings=4096, bos_token_id=1, eos_token_id=2),
}
CONTEXT = 2048          # tokens each request holds while decoding is timed
MAX_MODEL_LEN = 4096
BLOCK_SIZE = 16
PREFILL_TOKENS = 2048
E2E_WARMUP = 16         # untimed steps of the end-to-end run at least: the first steps after the prompts run slower
E2E_WARMUP_SECONDS = 0.3
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(p):
        with open(p) as f:
            d = json.load(f)
        d["source"] = "measured"
        return d
    return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region is timed."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.proc, self.lines = None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "20"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=lambda: self.lines.extend(self.proc.stdout), daemon=True).start()
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], None, set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 6:
                continue
            try:
                sm.append(float(f[0]))
                mx = float(f[1])
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


def model_numbers(cfg, n_layers):
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    per_layer = H * (nh + 2 * nkv) * hd + nh * hd * H + 3 * H * I
    return dict(layer_params=per_layer, linear_params=per_layer * n_layers, head_params=V * H,
                kv_bytes_per_token=2 * nkv * hd * 2 * n_layers)


def decode_bytes(nums, batch, context):
    """What a decode step has to read: every weight it uses once, and the cache of the live requests."""
    return 2 * (nums["linear_params"] + nums["head_params"]) + batch * context * nums["kv_bytes_per_token"]


def prefill_flops(cfg, nums, T, n_layers):
    attn = 4 * cfg["num_attention_heads"] * cfg["head_dim"] * T * T / 2 * n_layers     # causal QK^T and PV
    return 2 * T * nums["linear_params"] + attn + 2 * nums["head_params"]               # the head runs on one row


def fill_requests(runner, mgr, batch, context, prefix):
    """Puts `batch` requests of `context - 1` cached tokens into the manager without running a prefill (the
    cache holds random values, which is all that decode timing needs)."""
    ids = []
    for i in range(batch):
        rid = f"{prefix}{i}"
        mgr.add(rid)
        mgr.reserve(rid, context - 1)
        mgr.commit(rid, context - 1)
        ids.append(rid)
    return ids


def time_decode(runner, mgr, ids, steps, warmup, vocab, seed=0):
    import torch
    from lmsf_b200 import kernels
    from lmsf_b200.engine.model_runner import StepEntry
    g = torch.Generator().manual_seed(seed)
    toks = torch.randint(0, vocab, (steps + warmup, len(ids)), generator=g).tolist()
    sampler_out = torch.empty(len(ids), dtype=torch.int32, device=runner.device)

    def one(k):
        logits = runner.decode_step([StepEntry(r, [toks[k][j]], [0]) for j, r in enumerate(ids)], mgr)
        kernels.sample(sampler_out, logits)

    for k in range(warmup):
        one(k)
    torch.cuda.synchronize()
    l0 = kernels.launch_count()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for k in range(warmup, warmup + steps):
        one(k)
    end.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(end) / steps
    return ms, kernels.launch_count() - l0


def time_prefill(runner, mgr, T, reps, warmup, vocab):
    import torch
    from lmsf_b200.engine.model_runner import StepEntry
    g = torch.Generator().manual_seed(1)
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=runner.device)     # larger than L2
    times = []
    for k in range(warmup + reps):
        toks = torch.randint(0, vocab, (T,), generator=g).tolist()
        mgr.add("prefill")
        flush.zero_()
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        runner.step([StepEntry("prefill", toks, [T - 1])], mgr, check=False)
        end.record()
        torch.cuda.synchronize()
        mgr.free("prefill")
        if k >= warmup:
            times.append(start.elapsed_time(end))
    return statistics.median(times)


def measure_shape(cfg, n_layers, ctx_len, batches, steps, warmup, pk, with_prefill=True):
    """Builds the model of `cfg` with random weights and times decode steps at each batch size of `batches` (requests
    of ctx_len tokens each) and a prefill of PREFILL_TOKENS tokens.  Returns {batch: (ms per step, launches, clocks)}
    and the prefill record (or None)."""
    import torch
    from lmsf_b200.engine.factory import build_model
    from lmsf_b200.engine.model_runner import ModelRunner
    cfg = dict(cfg, num_hidden_layers=n_layers)
    folder = tempfile.mkdtemp(prefix="lmsf_bench_")
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    nums = model_numbers(cfg, n_layers)
    dev = torch.device("cuda:0")
    model, _, dtype = build_model(folder, "bfloat16", dev, load_format="dummy")
    pages = (max(batches) * (ctx_len + 64) + PREFILL_TOKENS) // BLOCK_SIZE + 64
    runner = ModelRunner(model, dtype, dev, BLOCK_SIZE, num_blocks=pages, max_num_seqs=max(80, max(batches)),
                         max_model_len=max(MAX_MODEL_LEN, ctx_len + 64))
    for t in runner.storage.tensors:
        t.normal_(0.0, 1.0)
    mgr = runner.make_cache_manager()
    V = cfg["vocab_size"]
    out = {}
    for b in batches:
        clocks = ClockSampler()
        clocks.start()
        ids = fill_requests(runner, mgr, b, ctx_len, f"b{b}_")
        ms, launches = time_decode(runner, mgr, ids, steps if b == batches[0] else max(8, steps // 2), warmup, V)
        rec = clocks.stop()
        for r in ids:
            mgr.free(r)
        out[b] = (ms, launches, rec)
    prefill = None
    if with_prefill:
        pf_ms = time_prefill(runner, mgr, PREFILL_TOKENS, 3, 2, V)
        pf_flops = prefill_flops(cfg, nums, PREFILL_TOKENS, n_layers)
        prefill = {"value": round(PREFILL_TOKENS / (pf_ms * 1e-3), 1), "tokens": PREFILL_TOKENS, "ms": round(pf_ms, 3),
                   "frac": round(pf_flops / (pf_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)}
    del runner, mgr, model
    torch.cuda.empty_cache()
    return out, prefill, nums, folder


def other_model_points(pk, steps, warmup):
    """The other workloads that the baseline names, as points of the same line: 64 requests under continuous batching
    on the headline shape; Llama-3.2-1B (decode at batch 64 and the same 64 requests) and Llama-2-13B (decode at batch 8 with 4,000-token contexts and a
    2,048-token prefill).  Each point has its own clock record."""
    points, clocks = {}, {}
    cfg = dict(MODELS["llama3-8b"])
    sampler = ClockSampler()
    sampler.start()
    srv = serve(cfg, cfg["num_hidden_layers"], 64, 256, 2048, quiet=True)
    clocks["llama3-8b_serve"] = sampler.stop()
    points["llama3-8b_serve_generated_tok_s"] = srv["value"]
    points["llama3-8b_serve_total_tok_s"] = srv["total_tokens_per_s"]
    cfg = dict(MODELS["llama3.2-1b"])
    res, _, nums, _ = measure_shape(cfg, cfg["num_hidden_layers"], CONTEXT, [64], steps, warmup, pk, with_prefill=False)
    ms, _, rec = res[64]
    points["llama3.2-1b_decode_b64"] = round(64 / (ms * 1e-3), 1)
    points["llama3.2-1b_decode_b64_hbm_frac"] = round(decode_bytes(nums, 64, CONTEXT) / (ms * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
    clocks["llama3.2-1b_decode_b64"] = rec
    sampler = ClockSampler()
    sampler.start()
    srv = serve(cfg, cfg["num_hidden_layers"], 64, 256, 2048, quiet=True)
    clocks["llama3.2-1b_serve"] = sampler.stop()
    points["llama3.2-1b_serve_generated_tok_s"] = srv["value"]
    points["llama3.2-1b_serve_total_tok_s"] = srv["total_tokens_per_s"]
    cfg = dict(MODELS["llama2-13b"])
    res, prefill, nums, _ = measure_shape(cfg, cfg["num_hidden_layers"], 4000, [8], steps, warmup, pk)
    ms, _, rec = res[8]
    points["llama2-13b_decode_b8_ctx4000"] = round(8 / (ms * 1e-3), 1)
    points["llama2-13b_decode_b8_ctx4000_hbm_frac"] = round(decode_bytes(nums, 8, 4000) / (ms * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
    points["llama2-13b_prefill_2048_tok_s"] = prefill["value"]
    points["llama2-13b_prefill_2048_frac"] = prefill["frac"]
    clocks["llama2-13b"] = rec
    return points, clocks


def time_e2e(folder, n_layers, batch, context, steps, warmup, vocab):
    """Decode through the public entry point: every step takes the host's token lists through the scheduler,
    copies the step's inputs from pinned host memory to the device and reads the sampled tokens back."""
    import torch
    from lmsf_b200 import EngineArgs, LLMEngine, SamplingParams
    engine = LLMEngine(EngineArgs(model=folder, dtype="bfloat16", block_size=BLOCK_SIZE, max_model_len=max(MAX_MODEL_LEN, context + 64),
                                  max_num_batched_tokens=8192, max_num_seqs=max(batch, 8),
                                  gpu_memory_utilization=0.85), load_format="dummy")
    g = torch.Generator().manual_seed(2)
    # Untimed steps: at least max(warmup, E2E_WARMUP), and on until E2E_WARMUP_SECONDS have passed (the clocks need
    # that long to settle after the prompts), as far as the context length leaves room.
    room = max(MAX_MODEL_LEN, context + 64) - context - steps - 8
    warm_min, warm_max = max(warmup, E2E_WARMUP), max(max(warmup, E2E_WARMUP), min(room, 512))
    sp = SamplingParams(temperature=0.0, max_tokens=steps + warm_max + 8, ignore_eos=True)
    for i in range(batch):
        engine.add_request(i, None, sp, prompt_token_ids=torch.randint(0, vocab, (context - 1,), generator=g).tolist())
    while any(s.num_computed < len(s.prompt_token_ids) for s in engine.seqs.values()) or len(engine.seqs) < batch:
        engine.step()
    t_warm, n_warm = time.perf_counter(), 0
    while n_warm < warm_min or (n_warm < warm_max and time.perf_counter() - t_warm < E2E_WARMUP_SECONDS):
        engine.step()
        n_warm += 1
    torch.cuda.synchronize()
    h2d0 = engine.runner.h2d_bytes
    t0 = time.perf_counter()
    produced = 0
    for _ in range(steps):
        produced += len(engine.step())
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    h2d = (engine.runner.h2d_bytes - h2d0) / steps
    del engine
    torch.cuda.empty_cache()
    return produced / dt, h2d, batch * 4 + 4


def serve(cfg, n_layers, n_requests, decode_tokens, budget, quiet=False):
    """Continuous batching through the engine: requests with seeded uniform-random prompt lengths in [128, 2048],
    `decode_tokens` generated tokens each.  Prints its own JSON line (not the line of the contract)."""
    import random

    import torch
    from lmsf_b200 import EngineArgs, LLMEngine, SamplingParams
    cfg = dict(cfg, num_hidden_layers=n_layers)
    folder = tempfile.mkdtemp(prefix="lmsf_bench_")
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    engine = LLMEngine(EngineArgs(model=folder, dtype="bfloat16", block_size=BLOCK_SIZE, max_model_len=MAX_MODEL_LEN,
                                  max_num_batched_tokens=budget, max_num_seqs=n_requests, gpu_memory_utilization=0.85),
                       load_format="dummy")
    rng = random.Random(0)
    lens = [rng.randint(128, 2048) for _ in range(n_requests)]
    g = torch.Generator().manual_seed(3)
    sp = SamplingParams(temperature=0.0, max_tokens=decode_tokens, ignore_eos=True)
    # Two passes warm up (compilation; a decode graph is captured the second time its size is seen, and the sizes of
    # the last steps, when requests run out, are seen once or twice a pass); the third is timed.
    for rep in range(3):
        for i, n in enumerate(lens):
            engine.add_request((rep, i), None, sp, prompt_token_ids=torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist())
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        steps = generated = preempted = 0
        while engine.has_unfinished_requests():
            generated += len(engine.step())
            preempted += engine.last_stats.num_preempted
            steps += 1
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
    rec = {"metric": "generated tokens/s under continuous batching", "value": round(generated / dt, 1),
           "unit": "tokens/s", "requests": n_requests, "prompt_tokens": sum(lens), "generated_tokens": generated,
           "total_tokens_per_s": round((generated + sum(lens)) / dt, 1), "seconds": round(dt, 3), "steps": steps,
           "preemptions": preempted, "max_num_batched_tokens": budget, "layers": n_layers,
           "layers_of_model": cfg["num_hidden_layers"], "dtype": "bf16", "data": "synthetic", "impl": "ours"}
    del engine
    torch.cuda.empty_cache()
    if quiet:
        return rec
    print(json.dumps(rec))
    return 0


def reference_arm(a) -> int:
    """The comparison arm: one step of the same model, batch and context made of yinqiwen/lmsf's own CUDA kernels
    (built unmodified for sm_100a into baseline/_ref) in the reference's order, with the library products the
    reference calls.  The Rust engine around them cannot be built here (no cargo, no network); nothing of
    lmsf_b200 runs on this path."""
    try:
        from baseline import build_ref
        build_ref.ensure_built()
    except Exception as e:                                  # no sources, no compiler: say so and leave
        print(json.dumps({"impl": "reference", "unavailable": " ".join(str(e).split())[:300]}))
        return 0
    import torch
    if not torch.cuda.is_available():
        print(json.dumps({"impl": "reference", "unavailable": "no CUDA device here; the reference's kernels are built"}))
        return 0
    from baseline.reference_step import DecodeBatch, ReferenceLlama
    a.warmup = max(a.warmup, 3)
    pk = peaks()
    cfg = dict(MODELS[a.model])
    full_layers = cfg["num_hidden_layers"]
    n_layers = a.layers or full_layers
    ctx_len, V = a.context, cfg["vocab_size"]
    nums = model_numbers(cfg, n_layers)
    dev = torch.device("cuda:0")
    max_batch = 64 if not a.skip_points else a.batch
    per_seq = -(-(ctx_len + 600) // BLOCK_SIZE)
    pages = max_batch * per_seq + PREFILL_TOKENS // BLOCK_SIZE + 8
    model = ReferenceLlama(cfg, n_layers, pages, BLOCK_SIZE, dev)
    g = torch.Generator().manual_seed(0)

    def decode(batch, steps, warmup, e2e=False):
        db = DecodeBatch(model, batch, ctx_len)
        toks = torch.randint(0, V, (steps + warmup, batch), generator=g).tolist()
        for k in range(warmup):
            db.step(toks[k], read_back=e2e)
        torch.cuda.synchronize()
        l0 = model.launches
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        start.record()
        for k in range(warmup, warmup + steps):
            db.step(toks[k], read_back=e2e)
        end.record()
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
        return start.elapsed_time(end) / steps, wall / steps, model.launches - l0, db

    clocks = ClockSampler()
    clocks.start()
    ms, _, launches, _ = decode(a.batch, a.steps, a.warmup)
    clock_rec = clocks.stop()
    value = a.batch / (ms * 1e-3)
    achieved = decode_bytes(nums, a.batch, ctx_len) / (ms * 1e-3) / 1e9
    points = {}
    if not a.skip_points:
        for b in (1, 64):
            pms, _, _, _ = decode(b, max(8, a.steps // 2), a.warmup)
            points[f"decode_b{b}"] = round(b / (pms * 1e-3), 1)
            points[f"decode_b{b}_hbm_frac"] = round(decode_bytes(nums, b, ctx_len) / (pms * 1e-3) / 1e9 / pk["hbm_gbs"], 4)

    # prefill of one prompt
    T = PREFILL_TOKENS
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)
    first = max_batch * per_seq
    pos = torch.arange(T, dtype=torch.int64, device=dev)
    slots = (first * BLOCK_SIZE + pos).contiguous()
    times = []
    for k in range(2 + 3):
        ids = torch.randint(0, V, (T,), generator=g).to(dev)
        flush.zero_()
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        model.prefill(ids, pos, slots)
        end.record()
        torch.cuda.synchronize()
        if k >= 2:
            times.append(start.elapsed_time(end))
    pf_ms = statistics.median(times)
    pf_flops = prefill_flops(cfg, nums, T, n_layers)
    prefill = {"value": round(T / (pf_ms * 1e-3), 1), "tokens": T, "ms": round(pf_ms, 3),
               "frac": round(pf_flops / (pf_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)}
    del flush
    model._bufs.clear()
    torch.cuda.empty_cache()

    e2e = None
    if not a.skip_e2e:
        _, wall, _, db = decode(a.batch, a.steps, max(a.warmup, E2E_WARMUP), e2e=True)
        e2e = {"value": round(a.batch / wall, 1), "unit": "tokens/s", "h2d_bytes_per_step": int(db.h2d_bytes),
               "d2h_bytes_per_step": int(db.d2h_bytes)}

    line = {
        "metric": f"decode tokens/s ({a.model} shape, batch {a.batch}, {ctx_len}-token contexts)", "value": round(value, 1),
        "unit": "tokens/s", "n_gpus": 1, "steps": a.steps, "warmup": a.warmup, "ms_per_step": round(ms, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"model": f"{a.model} shape, random weights", "layers": n_layers, "layers_of_model": full_layers,
                   "hidden_size": cfg["hidden_size"], "num_attention_heads": cfg["num_attention_heads"],
                   "num_key_value_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                   "intermediate_size": cfg["intermediate_size"], "vocab_size": V, "global_batch": a.batch,
                   "seq_len": ctx_len, "max_model_len": max(MAX_MODEL_LEN, ctx_len + 64), "block_size": BLOCK_SIZE,
                   "prefill_tokens": PREFILL_TOKENS, "e2e_warmup": f">= {max(a.warmup, E2E_WARMUP)} steps", "parallelism": "1 GPU",
                   "l2": "inputs larger than L2 (weights + cache of a step >> 126 MB); prefill flushes L2",
                   "peaks": pk["source"],
                   "arm": "the reference's CUDA kernels (unmodified, sm_100a) in its order, torch.mm (cuBLAS) products, "
                          "no CUDA graph; its Rust engine cannot be built here"},
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points, "clocks": clock_rec, "gpu_launches": int(launches), "impl": "reference",
    }
    if e2e is not None:
        line["e2e"] = e2e
    print(json.dumps(line))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=24)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--layers", type=int, default=None, help="run fewer layers than the model has (named in config)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--skip-e2e", action="store_true")
    ap.add_argument("--skip-points", action="store_true")
    ap.add_argument("--skip-models", action="store_true", help="leave out the points of the 1B and 13B shapes")
    ap.add_argument("--model", default="llama3-8b", choices=sorted(MODELS), help="whose layer sizes to run")
    ap.add_argument("--context", type=int, default=CONTEXT, help="tokens each request holds while decoding is timed")
    ap.add_argument("--budget", type=int, default=2048, help="--serve: max_num_batched_tokens of the engine")
    ap.add_argument("--serve", action="store_true",
                    help="instead of the contract's line: 64 requests of 128..2048 prompt tokens and 256 generated "
                         "tokens each through the engine's continuous batching")
    a = ap.parse_args()
    if a.impl == "reference":
        if a.gpus != 1:
            print(f"bench.py: the comparison arm runs on one GPU; --gpus {a.gpus} is not supported")
            return 2
        return reference_arm(a)
    if a.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {a.gpus} is not supported")
        return 2
    a.warmup = max(a.warmup, 3)

    pk = peaks()
    cfg = dict(MODELS[a.model])
    if a.serve:
        return serve(cfg, a.layers or cfg["num_hidden_layers"], 64, 256, a.budget)
    ctx_len = a.context
    # a context beyond the shape's own limit (--context 32000 on the 8B shape): the limit of the random model is raised
    cfg["max_position_embeddings"] = max(cfg["max_position_embeddings"], ctx_len + 64)
    full_layers = cfg["num_hidden_layers"]
    n_layers = a.layers or full_layers
    V = cfg["vocab_size"]
    batches = [a.batch] + ([b for b in (1, 64) if b != a.batch] if not a.skip_points else [])
    res, prefill, nums, folder = measure_shape(cfg, n_layers, ctx_len, batches, a.steps, a.warmup, pk)
    ms, launches, clock_rec = res[a.batch]
    value = a.batch / (ms * 1e-3)
    achieved = decode_bytes(nums, a.batch, ctx_len) / (ms * 1e-3) / 1e9
    points, points_clocks = {}, {}
    for b in batches[1:]:
        pms, _, rec = res[b]
        points[f"decode_b{b}"] = round(b / (pms * 1e-3), 1)
        points[f"decode_b{b}_hbm_frac"] = round(decode_bytes(nums, b, ctx_len) / (pms * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
        points_clocks[f"decode_b{b}"] = rec

    e2e = None
    if not a.skip_e2e:
        ev, h2d, d2h = time_e2e(folder, n_layers, a.batch, ctx_len, a.steps, a.warmup, V)
        e2e = {"value": round(ev, 1), "unit": "tokens/s", "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h)}

    if not a.skip_points and not a.skip_models and a.model == "llama3-8b" and a.layers is None:
        more, more_clocks = other_model_points(pk, max(8, a.steps // 2), a.warmup)
        points.update(more)
        points_clocks.update(more_clocks)

    line = {
        "metric": f"decode tokens/s ({a.model} shape, batch {a.batch}, {ctx_len}-token contexts)", "value": round(value, 1),
        "unit": "tokens/s", "n_gpus": 1, "steps": a.steps, "warmup": a.warmup, "ms_per_step": round(ms, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"model": f"{a.model} shape, random weights", "layers": n_layers, "layers_of_model": full_layers,
                   "hidden_size": cfg["hidden_size"], "num_attention_heads": cfg["num_attention_heads"],
                   "num_key_value_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                   "intermediate_size": cfg["intermediate_size"], "vocab_size": V, "global_batch": a.batch,
                   "seq_len": ctx_len, "max_model_len": max(MAX_MODEL_LEN, ctx_len + 64), "block_size": BLOCK_SIZE,
                   "prefill_tokens": PREFILL_TOKENS, "e2e_warmup": f">= {max(a.warmup, E2E_WARMUP)} steps, up to {E2E_WARMUP_SECONDS} s", "parallelism": "1 GPU",
                   "l2": "inputs larger than L2 (weights + cache of a step >> 126 MB); prefill flushes L2",
                   "peaks": pk["source"]},
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points, "points_clocks": points_clocks, "clocks": clock_rec, "gpu_launches": int(launches), "impl": "ours",
    }
    if e2e is not None:
        line["e2e"] = e2e
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
