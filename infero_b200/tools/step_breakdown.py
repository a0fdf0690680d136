"""What each class of kernel costs inside a captured decode step.

    python -m infero_b200.tools.step_breakdown [--batch 8] [--context 3900] [--layers 28] [--steps 30]
    python -m infero_b200.tools.step_breakdown --prefill 2048          (a prompt step instead, launched one by one)

Kernels of a captured step overlap (programmatic dependent launch), so a profiler's serialised
per-launch times do not add up to the step.  This tool measures the step as it runs, with CUDA
events, once whole and once with each class of kernel left out, and reports the differences.
The results of the shortened steps are garbage (and are thrown away); only their time is used.
Sizes are Qwen2.5-7B's unless overridden; weights are random.
"""
from __future__ import annotations

import argparse
import random
import sys


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="step_breakdown")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=3900)
    ap.add_argument("--layers", type=int, default=28)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--hidden", type=int, default=3584)
    ap.add_argument("--heads", type=int, default=28)
    ap.add_argument("--kv-heads", type=int, default=4)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--intermediate", type=int, default=18944)
    ap.add_argument("--vocab", type=int, default=152064)
    ap.add_argument("--prefill", type=int, default=0, help="time a prompt step of this many tokens instead of decode steps")
    ap.add_argument("--only", default=None, help="leave out just this class (norm, rope, attn, gemm_qkv, ..., head)")
    args = ap.parse_args(argv)

    import torch
    from infero_b200 import kernels as K
    from infero_b200.config import EngineConfig
    from infero_b200.engine import ModelRunner, StepEntry
    from infero_b200.kernels import attention as A
    from infero_b200.kernels import tc_gemm
    from infero_b200.loading import random_model

    cfg = {"architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "num_hidden_layers": args.layers,
           "hidden_size": args.hidden, "num_attention_heads": args.heads, "num_key_value_heads": args.kv_heads,
           "head_dim": args.head_dim, "intermediate_size": args.intermediate, "vocab_size": args.vocab,
           "rope_theta": 1e6, "rms_norm_eps": 1e-6, "tie_word_embeddings": False, "hidden_act": "silu",
           "max_position_embeddings": 32768}
    # The classes are left out by replacing the Python functions that launch them, so the layers must
    # be launched from Python here; the native launcher issues the same kernels in the same order, and
    # inside a captured step who launched them makes no difference.
    from infero_b200.parts import native_block
    native_block.set_enabled(False)
    model, _ = random_model(cfg, seed=0, dtype="bfloat16", device="cuda:0", generate_on_device=True)
    real = {"norm": K.add_rmsnorm, "rope": K.rope_cache_partials, "rope_many": K.rope_cache, "attn": A.paged_attention,
            "partials": tc_gemm.partials, "swiglu": tc_gemm.gemm_swiglu, "gemm": tc_gemm.gemm}
    da, dkv = args.heads * args.head_dim, args.kv_heads * args.head_dim
    shapes = {"gemm_qkv": {(da + 2 * dkv, args.hidden)}, "gemm_o": {(args.hidden, da)},
              "gemm_down": {(args.hidden, args.intermediate)}}
    shapes["all_gemm"] = shapes["gemm_qkv"] | shapes["gemm_o"] | shapes["gemm_down"]
    shapes["head"] = {(args.vocab, args.hidden)}

    def restore():
        K.add_rmsnorm, K.rope_cache_partials, A.paged_attention = real["norm"], real["rope"], real["attn"]
        K.rope_cache = real["rope_many"]
        tc_gemm.partials, tc_gemm.gemm_swiglu, tc_gemm.gemm = real["partials"], real["swiglu"], real["gemm"]

    def without(tag):
        if tag == "norm":
            K.add_rmsnorm = lambda *a, **k: None
        elif tag == "rope":
            K.rope_cache_partials = lambda *a, **k: None
            K.rope_cache = lambda *a, **k: None
        elif tag == "attn":
            A.paged_attention = lambda *a, **k: None
        if tag in shapes:
            skip = shapes[tag]

            def fake(a, w):
                if (w.shape[0], w.shape[1]) in skip:
                    s, _, _ = tc_gemm.plan(a.shape[0], w.shape[0], w.shape[1], a.device)
                    return torch.empty((s, a.shape[0], w.shape[0]), dtype=torch.float32, device=a.device)
                return real["partials"](a, w)
            tc_gemm.partials = fake

            def fake_gemm(a, w, bias, out, tile_n=0):         # (many-token products come this way)
                if (w.shape[0], w.shape[1]) not in skip:
                    real["gemm"](a, w, bias, out, tile_n)
            tc_gemm.gemm = fake_gemm
        if tag in ("gemm_gate_up", "all_gemm"):
            tc_gemm.gemm_swiglu = lambda a, w, out: True

    B = args.batch
    blocks = -(-(args.context + args.steps + 16) // 16)

    def measure_prefill(tag):
        """A prompt of --prefill tokens as one step of a fresh request, kernels launched one by one."""
        restore()
        T = args.prefill
        pages = -(-T // 16) + 1
        runner = ModelRunner(model, EngineConfig(dtype="bfloat16", page_size=16, num_pages=pages, max_seqs=1,
                                                 ctx=pages * 16, max_batch_tokens=T, max_logit_rows=8, cuda_graphs=False))
        rng = random.Random(1)
        prompt = [rng.randrange(args.vocab) for _ in range(T)]
        without(tag)

        def one():
            runner.open(0)
            runner.step([StepEntry(0, prompt, [T - 1])])
            runner.close(0)
        for _ in range(3):
            one()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        n = max(3, args.steps // 3)
        e0.record()
        for _ in range(n):
            one()
        e1.record()
        torch.cuda.synchronize()
        restore()
        del runner
        torch.cuda.empty_cache()
        return e0.elapsed_time(e1) / n

    def measure(tag):
        if args.prefill:
            return measure_prefill(tag)
        restore()
        runner = ModelRunner(model, EngineConfig(dtype="bfloat16", page_size=16, num_pages=B * blocks, max_seqs=B,
                                                 ctx=blocks * 16, max_batch_tokens=2048, max_logit_rows=max(B, 8),
                                                 cuda_graphs=True))
        rng = random.Random(1)
        for r in range(B):
            runner.open(r)
            done = 0
            while done < args.context:
                n = min(2048, args.context - done)
                runner.step([StepEntry(r, [rng.randrange(args.vocab) for _ in range(n)], [])])
                done += n
        without(tag)
        picked = torch.empty(B, dtype=torch.int32, device="cuda:0")

        def one():
            K.argmax(runner.step([StepEntry(r, [5], [0]) for r in range(B)]), picked)
        for _ in range(4):
            one()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            one()
        e1.record()
        torch.cuda.synchronize()
        restore()
        for r in range(B):
            runner.close(r)
        del runner
        torch.cuda.empty_cache()
        return e0.elapsed_time(e1) / args.steps

    base = measure("none")
    if args.prefill:
        print(f"prompt of {args.prefill} tokens, {args.layers} layers: whole step {base:.3f} ms")
    else:
        print(f"batch {B}, context {args.context}, {args.layers} layers: whole step {base:.3f} ms")
    tags = ("norm", "rope", "attn", "gemm_qkv", "gemm_o", "gemm_gate_up", "gemm_down", "all_gemm", "head")
    for tag in (tags if args.only is None else (args.only,)):
        ms = measure(tag)
        if tag == "head":
            print(f"  without {tag:13s} {ms:.3f} ms: the product with the output matrix costs {1000 * (base - ms):6.1f} us "
                  f"({100 * (base - ms) / base:4.1f} % of the step)")
            continue
        print(f"  without {tag:13s} {ms:.3f} ms: costs {1000 * (base - ms) / args.layers:6.1f} us per layer "
              f"({100 * (base - ms) / base:4.1f} % of the step)")
    if args.only is None:
        again = measure("none")
        print(f"  whole step again      {again:.3f} ms: {1000 * abs(again - base) / max(1, args.layers):.1f} us per layer apart from the "
              f"first; no line above means more than that")
    return 0


if __name__ == "__main__":
    sys.exit(main())
