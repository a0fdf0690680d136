"""generate: run one prompt through a model and report prefill and decode speed.

    generate <model_dir> [token ids...] [--greedy] [-n N]
    generate --model <model_dir> --prompt-ids 5,17,3 -n 32 --temperature 0.7 --top-k 20 --top-p 0.8
    generate --config <config.json> --random-weights --seed 3 --prompt-len 64 --dtype float32
             --max-seq-len 512 --page-size 16 --num-pages 40

After the reference's example (crates/model/examples/generate.rs:26-161): the positional
words after the model are the prompt, ``--greedy`` fixes the sampler, ``-n`` caps the
generation (128), ``GEN_CTX`` sets the context (4096), and the report lines have its form.
There is no tokenizer in this engine, so the prompt is token ids (``--raw`` is accepted and
changes nothing); ``--prompt-len L`` makes a seeded random prompt instead.
``--max-seq-len`` is the context (it wins over ``GEN_CTX``), ``--page-size`` and ``--num-pages``
the geometry of the cache pool (by default one context's worth of pages).
``--kv-quant`` only takes the unquantised cache and ``--gpu-layers`` is not taken at all:
quantised caches and host offload are not built.
"""
from __future__ import annotations

import argparse
import os
import random
import sys
import time


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="generate")
    ap.add_argument("model", nargs="?", default=None,
                    help="model folder (config.json + model.safetensors), or a config.json with --random-weights")
    ap.add_argument("prompt", nargs="*", help="prompt token ids")
    ap.add_argument("--model", dest="model_opt", default=None, help="the model folder, as an option")
    ap.add_argument("--config", default=None, help="a config.json (with --random-weights)")
    ap.add_argument("--prompt-ids", default=None, help="prompt token ids, comma-separated")
    ap.add_argument("--raw", action="store_true", help="accepted for compatibility; prompts are always raw ids")
    ap.add_argument("--greedy", action="store_true")
    ap.add_argument("-n", type=int, default=128, dest="max_new")
    ap.add_argument("--kv-quant", default="f16")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32", "bf16", "fp32"])
    ap.add_argument("--max-seq-len", type=int, default=None, help="context length (default: GEN_CTX, else 4096)")
    ap.add_argument("--page-size", type=int, default=16, choices=[16, 32, 64])
    ap.add_argument("--num-pages", type=int, default=None, help="pages in the cache pool (default: one context's worth)")
    ap.add_argument("--repetition-penalty", type=float, default=None)
    ap.add_argument("--prompt-len", type=int, default=None)
    ap.add_argument("--random-weights", action="store_true", help="MODEL is a config.json; weights are drawn from --seed")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--temperature", type=float, default=None)
    ap.add_argument("--top-k", type=int, default=None)
    ap.add_argument("--top-p", type=float, default=None)
    ap.add_argument("--ignore-eos", action="store_true")
    ap.add_argument("--no-warmup", action="store_true",
                    help="time the very first run (kernel loading and graph capture included)")
    args = ap.parse_args(argv)
    if args.model_opt is not None or args.config is not None:
        if args.model is not None:               # with --model / --config every positional word is the prompt
            args.prompt = [args.model] + list(args.prompt)
        args.model = args.model_opt if args.model_opt is not None else args.config
        if args.config is not None and not args.random_weights:
            print("generate: --config needs --random-weights (a configuration alone has no weights)", file=sys.stderr)
            return 2
    if args.model is None:
        ap.print_usage(sys.stderr)
        print("generate: no model given", file=sys.stderr)
        return 2
    args.dtype = {"bf16": "bfloat16", "fp32": "float32"}.get(args.dtype, args.dtype)
    if args.kv_quant not in ("f16", "bf16", "none"):
        print(f"generate: --kv-quant {args.kv_quant}: quantised caches are not built (f16 only)", file=sys.stderr)
        return 2

    import json
    import torch
    from infero_b200.engine import Engine
    from infero_b200.sampling import SamplingParams

    ctx = args.max_seq_len if args.max_seq_len is not None else int(os.environ.get("GEN_CTX", "4096"))
    slots = args.num_pages * args.page_size if args.num_pages is not None else ctx
    kw = dict(dtype=args.dtype, ctx=ctx, max_seqs=1, kv_slots=slots, page_size=args.page_size,
              max_batch_tokens=min(ctx, 2048))
    if args.random_weights:
        with open(args.model) as f:
            eng = Engine(config=json.load(f), seed=args.seed, **kw)
    else:
        eng = Engine(args.model, **kw)
    vocab = eng.model.spec.vocab_size
    if args.prompt_ids is not None:
        tokens = [int(t) for t in args.prompt_ids.split(",") if t.strip()]
    elif args.prompt:
        tokens = [int(t) for word in args.prompt for t in word.split(",") if t]
    else:
        rng = random.Random(args.seed)
        tokens = [rng.randrange(vocab) for _ in range(args.prompt_len or 16)]
    params = SamplingParams.greedy() if args.greedy else SamplingParams(seed=args.seed)
    if args.temperature is not None:
        params.temperature = args.temperature
    if args.top_k is not None:
        params.top_k = args.top_k
    if args.top_p is not None:
        params.top_p = args.top_p
    if args.repetition_penalty is not None:
        params.repetition_penalty = args.repetition_penalty

    print(f"--- prompt ({len(tokens)} tokens) ---")
    print(" ".join(map(str, tokens)) + "\n")
    print(f"weights  : {eng.model.weight_bytes() / (1 << 20):.0f} MiB in VRAM")
    print(f"kv cache : {eng.cfg.dtype}, {eng.runner.storage.bytes() / (1 << 20):.1f} MiB for "
          f"{eng.runner.num_pages * eng.cfg.page_size} positions")

    if not args.no_warmup:
        # a throw-away request of the same length: loads the kernels and captures the decode step,
        # so that the timed run below measures the engine and not its first call
        eng.generate([tokens], params, max_new_tokens=min(4, args.max_new), ignore_eos=True)
    eng.add_request(tokens, params, max_new_tokens=args.max_new, ignore_eos=args.ignore_eos)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    generated = []
    prefill_ms = None
    n_decoded = 0
    t1 = t0
    while not eng.is_idle():
        events = eng.step()
        for ev in events:
            if ev.token is not None:
                if prefill_ms is None:
                    torch.cuda.synchronize()
                    t1 = time.perf_counter()
                    prefill_ms = (t1 - t0) * 1000.0
                else:
                    n_decoded += 1
                generated.append(ev.token)
                print(ev.token, end=" ", flush=True)
            if ev.finished and ev.reason == "error":
                print(f"\n[error] {ev.message}", file=sys.stderr)
                return 1
    torch.cuda.synchronize()
    decode_s = time.perf_counter() - t1
    if prefill_ms is None:
        prefill_ms = (time.perf_counter() - t0) * 1000.0
    print("\n")
    print(f"prefill  {prefill_ms:7.1f} ms  ({len(tokens) / (prefill_ms / 1000.0):.1f} tok/s over {len(tokens)} tokens)")
    print(f"decode   {decode_s * 1000.0:7.1f} ms  ({n_decoded / max(decode_s, 1e-9):.1f} tok/s over {n_decoded} tokens)")
    return 0


if __name__ == "__main__":
    sys.exit(main())
