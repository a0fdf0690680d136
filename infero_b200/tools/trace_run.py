"""Trace replay: feed given token ids through a model step by step and write logits.

    trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

Reads one JSON object per line from standard input,

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

runs all entries of a step as one batch through the engine's own model, step function,
cache manager and kernels (the ones generation uses; nothing is sampled), writes
``OUT/<step>.f32`` (little-endian float32, [wanted, vocab], in the order of the entries and
of ``want``) when something is wanted, closes the requests named in ``end`` and prints
``done <step>``.  The cache pool is sized for ``--max-tokens`` tokens (each request's count
rounded up to a whole number of pages), so pages are used again during a long trace.
"""
from __future__ import annotations

import argparse
import json
import os
import sys


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (rounded up to pages)")
    ap.add_argument("--page-size", type=int, default=16, choices=[16, 32, 64])
    ap.add_argument("--device", default="cuda:0")
    args = ap.parse_args(argv)

    print("[trace_run] loading torch and the CUDA library (compiles on a first call)...",
          file=sys.stderr, flush=True)
    import torch
    if not torch.cuda.is_available():
        print("trace_run: no CUDA device is visible; this engine has no CPU path", file=sys.stderr)
        return 3
    from infero_b200 import kernels
    from infero_b200.config import EngineConfig
    from infero_b200.engine import ModelRunner, StepEntry
    from infero_b200.kernels import tc_gemm
    from infero_b200.loading import load_model

    kernels.lib()
    os.makedirs(args.out, exist_ok=True)
    n_tok = max(int(args.max_tokens), args.page_size)
    pages = -(-n_tok // args.page_size)
    model, _cfg = load_model(args.model, args.dtype, args.device)
    ecfg = EngineConfig(dtype=args.dtype, page_size=args.page_size, num_pages=pages, max_seqs=16,
                        ctx=pages * args.page_size, max_batch_tokens=max(pages * args.page_size, 64),
                        max_logit_rows=max(pages * args.page_size, 64), cuda_graphs=False,
                        device=args.device)
    runner = ModelRunner(model, ecfg)
    print(f"[trace_run] ready: {model.spec.architecture}, {len(model.spec.schedule)} layers, "
          f"{pages} pages of {args.page_size} tokens", file=sys.stderr, flush=True)

    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        entries = []
        for e in rec.get("entries", []):
            rid = e["id"]
            if rid not in runner.manager.requests:
                runner.open(rid)
            entries.append(StepEntry(rid=rid, tokens=e["tokens"], want=e.get("want", [])))
        if entries:
            logits = runner.step(entries)
            if logits is not None:
                arr = logits.detach().to("cpu", torch.float32).contiguous().numpy()
                arr.astype("<f4", copy=False).tofile(os.path.join(args.out, f"{step}.f32"))
            else:
                torch.cuda.current_stream().synchronize()
            fault = tc_gemm.error_flag()
            if fault:
                print(f"trace_run: step {step}: a kernel's bounded wait ran out (code {fault}); "
                      "its logits are not to be trusted", file=sys.stderr, flush=True)
                return 4
        for rid in rec.get("end", []):
            if rid in runner.manager.requests:
                runner.close(rid)
        sys.stdout.write(f"done {step}\n")
        sys.stdout.flush()
    return 0


if __name__ == "__main__":
    sys.exit(main())
