"""A serving-like run through the Engine: many requests with prompts of mixed lengths arrive at
once, at most ``--max-seqs`` are live, each generates ``--new`` tokens.

    python -m infero_b200.tools.serving_bench [--shape 0.5b|7b] [--requests 128] [--max-seqs 64]
        [--new 128] [--passes 3] [--profile]

Random weights of the named Qwen2.5 shape, uniform random prompts of 16..2,048 tokens, greedy
picks with end-of-sequence ignored.  Every pass feeds the same requests again; the first pays
for the CUDA graphs it captures, the later ones show the steady state.  Wall-clock time from the
first ``Engine.step`` to the last token on the host (the reference times its scheduler loop the
same way, crates/server/src/scheduler.rs:1268-1429).  ``--profile`` adds a cProfile table of the
last pass: where the host's time goes.
"""
from __future__ import annotations

import argparse
import random
import sys
import time

SHAPES = {
    "0.5b": {"num_hidden_layers": 24, "hidden_size": 896, "num_attention_heads": 14, "num_key_value_heads": 2,
             "intermediate_size": 4864, "vocab_size": 151936, "tie_word_embeddings": True},
    "7b": {"num_hidden_layers": 28, "hidden_size": 3584, "num_attention_heads": 28, "num_key_value_heads": 4,
           "intermediate_size": 18944, "vocab_size": 152064, "tie_word_embeddings": False},
}
COMMON = {"architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "rope_theta": 1e6, "rms_norm_eps": 1e-6,
          "use_sliding_window": False, "max_position_embeddings": 32768, "hidden_act": "silu"}
PROMPT_LENGTHS = (16, 50, 130, 400, 900, 2048)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="serving_bench")
    ap.add_argument("--shape", default="0.5b", choices=sorted(SHAPES))
    ap.add_argument("--requests", type=int, default=128)
    ap.add_argument("--max-seqs", type=int, default=64)
    ap.add_argument("--new", type=int, default=128, help="tokens generated per request")
    ap.add_argument("--passes", type=int, default=3)
    ap.add_argument("--profile", action="store_true")
    args = ap.parse_args(argv)

    import torch
    from infero_b200 import kernels as K
    from infero_b200.engine import Engine
    from infero_b200.loading import random_model
    from infero_b200.sampling import SamplingParams
    K.lib()
    cfg = dict(COMMON, **SHAPES[args.shape])
    model, _ = random_model(cfg, seed=0, dtype="bfloat16", device="cuda:0", generate_on_device=True)
    ctx = max(PROMPT_LENGTHS) + args.new + 16
    eng = Engine(model=model, dtype="bfloat16", ctx=ctx, max_seqs=args.max_seqs, kv_slots=args.max_seqs * ctx,
                 max_batch_tokens=2048, page_size=16, cuda_graphs=True)
    pick = SamplingParams(temperature=0.0, repetition_penalty=1.0)

    def one_pass(tag: str, profile: bool) -> None:
        rng = random.Random(0)
        prompt_tokens = 0
        for i in range(args.requests):
            n = rng.choice(PROMPT_LENGTHS)
            prompt_tokens += n
            eng.add_request([rng.randrange(cfg["vocab_size"]) for _ in range(n)], pick, max_new_tokens=args.new,
                            rid=f"{tag}{i}", ignore_eos=True)
        prof = None
        if profile:
            import cProfile
            prof = cProfile.Profile()
        torch.cuda.synchronize()
        captures0 = eng.runner.graph_captures
        t0 = time.time()
        generated = steps = 0
        if prof:
            prof.enable()
        while not eng.is_idle():
            generated += sum(1 for ev in eng.step() if ev.token is not None)
            steps += 1
        if prof:
            prof.disable()
        torch.cuda.synchronize()
        dt = time.time() - t0
        print(f"{args.shape} pass {tag}: {args.requests} requests, {prompt_tokens} prompt tokens + {generated} generated "
              f"in {dt:.3f} s over {steps} steps: {(prompt_tokens + generated) / dt:.0f} tok/s in all, "
              f"{generated / dt:.0f} generated tok/s; {eng.runner.graph_captures - captures0} graphs captured"
              + (" (profiled)" if prof else ""))
        if prof:
            import pstats
            pstats.Stats(prof).sort_stats("cumulative").print_stats(25)

    for p in range(max(1, args.passes)):
        one_pass(chr(ord("a") + p), args.profile and p == args.passes - 1)
    return 0


if __name__ == "__main__":
    sys.exit(main())
