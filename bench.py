#!/usr/bin/env python3
"""Decode and prefill throughput of the engine at Qwen2.5-7B layer sizes, random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

One JSON line on standard output.  A "step" is one decode step of the whole batch: the
host-to-device copy of the step's inputs, the model's forward pass from the cache (a
captured CUDA graph once the shape has been seen twice) and the argmax kernel.

  value     decoded tokens per second at batch 8 with 4,096 tokens of context each, timed on
            the device with CUDA events around exactly K steps; the tokens fed are drawn
            beforehand, so no step waits for the host.  The K-step region is run REPEATS times
            (every repeat cut back to the same context, so each ends at 4,096 tokens) after
            decode steps have run for at least half a second since the cache was filled; the
            median repeat is reported, and every repeat with its median SM clock in ``repeats``
  e2e       the same through ``Engine.add_request`` / ``Engine.step``: host token ids in,
            sampled token ids back on the host every step
  prefill   one step of 2,048 prompt tokens (flops / time / peak); --prefill-tokens N times a step of N instead
  roofline  bytes a decode step has to read (every weight it uses once, and the cache of
            the live requests) / its time, against the measured copy bandwidth
  points    decoded tokens per second at batch 1 and 64

This engine runs on one GPU; with --gpus above 1 it says so and exits with 2.
"""
from __future__ import annotations

import argparse
import json
import os
import random
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# the layer sizes of Qwen2.5-7B (the configuration the headline numbers are quoted on)
QWEN25_7B = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": 28, "hidden_size": 3584, "num_attention_heads": 28, "num_key_value_heads": 4,
    "head_dim": 128, "intermediate_size": 18944, "vocab_size": 152064, "rope_theta": 1000000.0,
    "rms_norm_eps": 1e-6, "tie_word_embeddings": False, "use_sliding_window": False,
    "max_position_embeddings": 32768, "hidden_act": "silu",
}
# the other shapes the same two metrics are asked for (--shape); the default stays the 7B one
OTHER_SHAPES = {
    "14b": {"num_hidden_layers": 48, "hidden_size": 5120, "num_attention_heads": 40, "num_key_value_heads": 8,
            "intermediate_size": 13824, "vocab_size": 152064, "rms_norm_eps": 1e-5, "tie_word_embeddings": False},
    "0.5b": {"num_hidden_layers": 24, "hidden_size": 896, "num_attention_heads": 14, "num_key_value_heads": 2,
             "head_dim": 64, "intermediate_size": 4864, "vocab_size": 151936, "rms_norm_eps": 1e-6, "tie_word_embeddings": True},
}
SHAPE_NAMES = {"7b": "Qwen2.5-7B shape", "14b": "Qwen2.5-14B shape", "0.5b": "Qwen2.5-0.5B shape"}
CONTEXT = 4096
PREFILL_TOKENS = 2048
REPEATS = 5                 # timed K-step regions; the median one is reported
WARM_SECONDS = 0.5          # decode steps run at least this long between the cache fill and the first timed region
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "source": "measured"}
    return dict(FALLBACK_PEAKS, bf16_tflops_sustained=1400.0, source="fallback")


from infero_b200.tools.clocks import ClockSampler  # noqa: E402


def matmul_params_per_layer(c):
    d, ff = c["hidden_size"], c["intermediate_size"]
    da = c["num_attention_heads"] * c["head_dim"]
    dkv = c["num_key_value_heads"] * c["head_dim"]
    return d * (da + 2 * dkv) + da * d + 3 * d * ff


def decode_bytes(c, layers, batch, kv_tokens_total, esize=2):
    """Bytes one decode step has to read: every matrix and vector it uses once, the embedding
    rows of its tokens, and the cached keys and values of the live requests."""
    d, V = c["hidden_size"], c["vocab_size"]
    da = c["num_attention_heads"] * c["head_dim"]
    dkv = c["num_key_value_heads"] * c["head_dim"]
    per_layer = matmul_params_per_layer(c) + (da + 2 * dkv) + 2 * d          # + biases + two norms
    weights = (layers * per_layer + V * d + d) * esize
    kv = kv_tokens_total * layers * 2 * dkv * esize
    return weights + kv + batch * d * esize


def prefill_flops(c, layers, T):
    gemm = 2.0 * T * layers * matmul_params_per_layer(c) + 2.0 * c["vocab_size"] * c["hidden_size"]
    attn = layers * 2.0 * T * T * c["num_attention_heads"] * c["head_dim"]    # causal: half of 4 T^2 H D
    return gemm + attn


def random_prompt(rng, vocab, n):
    return [rng.randrange(vocab) for _ in range(n)]


def fill_cache(runner, rids, length, vocab, rng, chunk):
    """Bring each request to ``length`` cached tokens by prompt portions without logits."""
    from infero_b200.engine import StepEntry
    for rid in rids:
        runner.open(rid)
        done = 0
        while done < length:
            n = min(chunk, length - done)
            runner.step([StepEntry(rid, random_prompt(rng, vocab, n), [])])
            done += n


def time_decode(model, cfg_json, layers, batch, steps, warmup, clocks, page_size, repeats=REPEATS):
    """Device-timed decode steps at ``batch`` requests that end at CONTEXT tokens each: ``repeats``
    regions of exactly ``steps`` steps, every one cut back to the same starting context first."""
    import torch
    from infero_b200 import kernels as K
    from infero_b200.config import EngineConfig
    from infero_b200.engine import ModelRunner, StepEntry
    vocab = cfg_json["vocab_size"]
    rng = random.Random(1000 + batch)
    start_len = CONTEXT - steps
    ecfg = EngineConfig(dtype="bfloat16", page_size=page_size, num_pages=batch * (-(-CONTEXT // page_size)),
                        max_seqs=batch, ctx=CONTEXT, max_batch_tokens=PREFILL_TOKENS, max_logit_rows=max(batch, 8),
                        cuda_graphs=True)
    runner = ModelRunner(model, ecfg)
    rids = [f"b{batch}_{i}" for i in range(batch)]
    fill_cache(runner, rids, start_len, vocab, rng, PREFILL_TOKENS)
    torch.cuda.synchronize()
    filled_at = time.perf_counter()
    feed = [[rng.randrange(vocab) for _ in range(batch)] for _ in range(steps)]
    picked = torch.empty(batch, dtype=torch.int32, device="cuda")

    def region(n):
        for rid in rids:
            if runner.length(rid) > start_len:
                runner.truncate(rid, start_len)
        for i in range(n):
            logits = runner.step([StepEntry(rid, [feed[i][j]], [0]) for j, rid in enumerate(rids)])
            K.argmax(logits, picked)

    # warm-up: at least `warmup` steps, and decode steps until WARM_SECONDS have passed since the fill (the
    # fill runs at the power limit; the first steps after it would be timed at its clocks)
    region(min(steps, max(warmup, 3)))
    torch.cuda.synchronize()
    while time.perf_counter() - filled_at < WARM_SECONDS:
        region(steps)
        torch.cuda.synchronize()
    runs = []
    for _ in range(repeats):
        for rid in rids:
            runner.truncate(rid, start_len)
        launches0, replays0 = K.launch_count(), runner.graph_replays
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        clocks.on = True
        t0 = time.perf_counter()
        e0.record()
        for i in range(steps):
            logits = runner.step([StepEntry(rid, [feed[i][j]], [0]) for j, rid in enumerate(rids)])
            K.argmax(logits, picked)
        e1.record()
        torch.cuda.synchronize()
        t1 = time.perf_counter()
        clocks.on = False
        graph_nodes = max((g.n_kernels for g in runner._graphs.values()), default=0)
        runs.append({"ms_per_step": e0.elapsed_time(e1) / steps, "t": (t0, t1),
                     "launches": int((K.launch_count() - launches0) + (runner.graph_replays - replays0) * graph_nodes),
                     "graph_replays": runner.graph_replays - replays0})
    # the keys a step reads, averaged over the region: each request grows from start_len to CONTEXT - 1
    kv_tokens = batch * (start_len + (steps - 1) / 2.0)
    order = sorted(range(repeats), key=lambda i: runs[i]["ms_per_step"])
    mid = runs[order[repeats // 2]]
    out = {"ms_per_step": mid["ms_per_step"], "tok_s": batch / (mid["ms_per_step"] / 1e3), "launches": mid["launches"],
           "bytes": decode_bytes(cfg_json, layers, batch, kv_tokens), "h2d": runner.last_h2d_bytes,
           "graph_replays": mid["graph_replays"], "kv_tokens": kv_tokens,
           "repeats": [{"ms_per_step": round(r["ms_per_step"], 4),
                        "sm_mhz": clocks.median_between(*r["t"]) if hasattr(clocks, "median_between") else None}
                       for r in runs]}
    for r in rids:
        runner.close(r)
    del runner
    torch.cuda.empty_cache()
    return out


def time_prefill(model, cfg_json, layers, reps, warmup, clocks, page_size, tokens=PREFILL_TOKENS):
    """One step of ``tokens`` prompt tokens of one request (the whole prompt: its attention runs over
    ``tokens`` keys), median of ``reps``."""
    import torch
    from infero_b200.config import EngineConfig
    from infero_b200.engine import ModelRunner, StepEntry
    vocab = cfg_json["vocab_size"]
    rng = random.Random(77)
    ecfg = EngineConfig(dtype="bfloat16", page_size=page_size, num_pages=2 * (-(-tokens // page_size)),
                        max_seqs=2, ctx=tokens, max_batch_tokens=tokens, cuda_graphs=False)
    runner = ModelRunner(model, ecfg)
    times = []
    for i in range(warmup + reps):
        prompt = random_prompt(rng, vocab, tokens)
        runner.open("p")
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if i >= warmup:
            clocks.on = True
        e0.record()
        runner.step([StepEntry("p", prompt, [tokens - 1])])
        e1.record()
        torch.cuda.synchronize()
        clocks.on = False
        if i >= warmup:
            times.append(e0.elapsed_time(e1))
        runner.close("p")
    del runner
    torch.cuda.empty_cache()
    times.sort()
    ms = times[len(times) // 2]
    return {"ms": ms, "flops": prefill_flops(cfg_json, layers, tokens)}


def time_e2e(model, cfg_json, batch, steps, warmup, clocks, page_size, repeats=REPEATS):
    """Through the Engine: requests in as host token ids, sampled ids out on the host each step.
    ``repeats`` regions of ``steps`` steps one after the other (generation cannot be cut back, so the
    contexts grow through the regions and reach CONTEXT at the end of the last); the median is reported."""
    import torch
    from infero_b200.engine import Engine
    from infero_b200.sampling import SamplingParams
    vocab = cfg_json["vocab_size"]
    rng = random.Random(2000 + batch)
    repeats = max(1, min(repeats, 300 // steps)) if steps < 300 else 1
    warm_steps = max(warmup, 30)
    eng = Engine(model=model, dtype="bfloat16", ctx=CONTEXT, max_seqs=batch, kv_slots=batch * CONTEXT,
                 max_batch_tokens=PREFILL_TOKENS, page_size=page_size, cuda_graphs=True)
    # requests that finish their prompt early decode while the others are still fed: 4 * batch steps at most
    start_len = CONTEXT - repeats * steps - warm_steps - 4 * batch - 2
    pure_argmax = SamplingParams(temperature=0.0, repetition_penalty=1.0)
    for _ in range(batch):
        eng.add_request(random_prompt(rng, vocab, start_len), pure_argmax,
                        max_new_tokens=CONTEXT, ignore_eos=True)
    started = set()
    while len(started) < batch:              # prompts, in portions, until every request has its first token
        started.update(ev.rid for ev in eng.step() if ev.token is not None)
    torch.cuda.synchronize()
    filled_at = time.perf_counter()
    n = 0
    while n < warmup or (n < warm_steps and time.perf_counter() - filled_at < WARM_SECONDS):
        eng.step()
        n += 1
    runs = []
    for _ in range(repeats):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        tokens = 0
        for _ in range(steps):
            tokens += sum(1 for ev in eng.step() if ev.token is not None)
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        runs.append((dt, tokens))
    runs.sort(key=lambda r: r[0] / max(1, r[1]))
    dt, tokens = runs[len(runs) // 2]
    h2d = eng.runner.last_h2d_bytes + 2 * batch * 4     # the step's arrays, and the sampler's (slot, flag) per row
    d2h = (batch + 1) * 4                    # one picked token per row, and the device's fault flag
    eng.abort_all("bench done")
    del eng
    torch.cuda.empty_cache()
    return {"tok_s": tokens / dt, "ms_per_step": dt * 1e3 / steps, "h2d": h2d, "d2h": d2h, "tokens": tokens,
            "repeats": len(runs)}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=None, help="run fewer layers than the configuration has")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--shape", default="7b", choices=sorted(SHAPE_NAMES), help="layer sizes: Qwen2.5-7B (the headline), 14B or 0.5B")
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--skip-points", action="store_true", help="leave out batch 1 and 64")
    ap.add_argument("--skip-e2e", action="store_true")
    ap.add_argument("--skip-prefill", action="store_true")
    ap.add_argument("--prefill-tokens", type=int, default=PREFILL_TOKENS,
                    help="size of the timed prompt step (the contract's 2,048; 8,192 and more show attention over long contexts)")
    args = ap.parse_args(argv)

    if args.impl == "reference":
        print(json.dumps({"impl": "reference",
                          "unavailable": "jackwangfeng/infero is a Rust workspace (no setup.py / pyproject.toml; "
                                         "pip: 'not installable') and this image has no cargo or rustc"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not built")
        return 2
    steps, warmup = max(1, args.steps), max(3, args.warmup)

    import torch
    from infero_b200 import kernels as K
    from infero_b200.loading import random_model
    K.lib()
    cfg_json = dict(QWEN25_7B)
    cfg_json.update(OTHER_SHAPES.get(args.shape, {}))
    shape_name = SHAPE_NAMES[args.shape]
    full_layers = cfg_json["num_hidden_layers"]
    layers = args.layers or full_layers
    cfg_json["num_hidden_layers"] = layers
    pk = peaks()
    clocks = ClockSampler(0)
    t_start = time.time()
    model, _ = random_model(cfg_json, seed=0, dtype="bfloat16", device="cuda:0", generate_on_device=True)
    torch.cuda.synchronize()

    main_pt = time_decode(model, cfg_json, layers, args.batch, steps, warmup, clocks, args.page_size)
    main_clocks = clocks.summary()
    quiet = ClockSampler.__new__(ClockSampler)
    quiet.on = False
    quiet.median_between = lambda t0, t1: None
    points = {}
    if not args.skip_points:
        for b in (1, 64):
            r = time_decode(model, cfg_json, layers, b, min(steps, 50), warmup, quiet, args.page_size, repeats=3)
            points[f"decode_b{b}"] = round(r["tok_s"], 1)
            points[f"decode_b{b}_hbm_frac"] = round(r["bytes"] / (r["ms_per_step"] / 1e3) / 1e9 / pk["hbm_gbs"], 3)
    prefill = None
    if not args.skip_prefill:
        r = time_prefill(model, cfg_json, layers, 5, 3, quiet, args.page_size, args.prefill_tokens)
        prefill = {"value": round(args.prefill_tokens / (r["ms"] / 1e3), 1), "tokens": args.prefill_tokens,
                   "ms": round(r["ms"], 3),
                   "frac": round(r["flops"] / (r["ms"] / 1e3) / 1e12 / pk["bf16_tflops"], 4),
                   # frac is against the burst GEMM peak; the same against the sustained (power-capped) one
                   "frac_of_sustained": round(r["flops"] / (r["ms"] / 1e3) / 1e12 / pk["bf16_tflops_sustained"], 4)}
    e2e = None
    if not args.skip_e2e:
        r = time_e2e(model, cfg_json, args.batch, steps, warmup, quiet, args.page_size)
        e2e = {"value": round(r["tok_s"], 1), "unit": "tok/s", "h2d_bytes_per_step": r["h2d"],
               "d2h_bytes_per_step": r["d2h"], "ms_per_step": round(r["ms_per_step"], 4)}

    achieved = main_pt["bytes"] / (main_pt["ms_per_step"] / 1e3) / 1e9
    line = {
        "metric": f"decode tok/s at batch {args.batch} (4K ctx), {shape_name}",
        "value": round(main_pt["tok_s"], 1), "unit": "tok/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": round(main_pt["ms_per_step"], 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic: random weights N(0,0.02) from a seed, uniform random token ids",
        "impl": "ours",
        "config": {"model": shape_name, "global_batch": args.batch, "seq_len": CONTEXT,
                   "parallelism": "single GPU", "layers": layers, "layers_of_configuration": full_layers,
                   "hidden": cfg_json["hidden_size"], "heads": cfg_json["num_attention_heads"],
                   "kv_heads": cfg_json["num_key_value_heads"], "head_dim": cfg_json["head_dim"],
                   "intermediate": cfg_json["intermediate_size"], "vocab": cfg_json["vocab_size"],
                   "page_size": args.page_size, "l2": "inputs larger than L2 (weights and cache)",
                   "peaks": pk["source"], "prefill_tokens": args.prefill_tokens, "repeats": REPEATS,
                   "timing": f"median of {REPEATS} regions of {steps} steps, each ending at {CONTEXT} tokens"},
        "e2e": e2e, "gpu_launches": main_pt["launches"], "clocks": main_clocks,
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
        "repeats": main_pt["repeats"],
        "wall_s": round(time.time() - t_start, 1),
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
