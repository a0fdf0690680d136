"""When the kernels of one decode step ran, block by block, as the device's own clock saw it.

    python -m infero_b200.tools.timeline [--batch 8] [--context 4000] [--layers 8] [--shape 7b]
                                         [--steps 3] [--raw FILE]

Under programmatic dependent launch the kernels of a step overlap, so neither a kernel's time alone
nor a profiler's serialised list says what a kernel costs in place.  This tool loads the library's
timeline variant (built with INFERO_TIMELINE=1 into a folder of its own: every block of the
instrumented kernels logs its kind, grid, multiprocessor and its first and last nanosecond of the
global timer), runs captured decode steps of a random model and prints, for the last step, an
averaged timeline of a layer (from its q/k/v product to the next layer's): for each launch when its first block started, when all had started,
when the first and the last ended, relative to the start of the layer's first kernel.  Nothing of
the step is replaced or left out; the log costs each block one atomic and one 32-byte store.
The reference's counterpart times kernels one by one with events (crates/cuda/src/profile.rs:28-130).
"""
from __future__ import annotations

import argparse
import os
import sys

KINDS = {1: "embed", 2: "norm", 3: "product", 4: "rotary+append", 5: "decode attention", 6: "argmax",
         7: "argmax final", 8: "keep tokens", 9: "swiglu", 10: "prompt attention"}
UNITS = ("elementwise", "rope_cache", "sampling", "gemm_tc", "attention_decode")


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="timeline")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=4000)
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--shape", default="7b", choices=["7b", "14b", "0.5b"])
    ap.add_argument("--steps", type=int, default=4, help="decode steps to run; the last one is reported")
    ap.add_argument("--raw", default=None, help="also write every record of the last step to this file (CSV)")
    args = ap.parse_args(argv)

    os.environ["INFERO_TIMELINE"] = "1"            # before the library is built and loaded
    import ctypes
    import random

    import numpy as np
    import torch

    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    sys.path.insert(0, root)
    import bench
    from infero_b200 import kernels as K
    from infero_b200.config import EngineConfig
    from infero_b200.engine import ModelRunner, StepEntry
    from infero_b200.loading import random_model

    lib = K.lib()
    cfg = dict(bench.QWEN25_7B)
    cfg.update(bench.OTHER_SHAPES.get(args.shape, {}))
    cfg["num_hidden_layers"] = args.layers
    model, _ = random_model(cfg, seed=0, dtype="bfloat16", device="cuda:0", generate_on_device=True)
    B, P = args.batch, 16
    ctx = -(-(args.context + args.steps + 8) // P) * P
    ecfg = EngineConfig(dtype="bfloat16", page_size=P, num_pages=B * (ctx // P), max_seqs=B, ctx=ctx,
                        max_batch_tokens=2048, max_logit_rows=max(B, 8), cuda_graphs=True)
    runner = ModelRunner(model, ecfg)
    rng = random.Random(5)
    rids = [f"r{i}" for i in range(B)]
    bench.fill_cache(runner, rids, args.context, cfg["vocab_size"], rng, 2048)
    picked = torch.empty(B, dtype=torch.int32, device="cuda")

    # the log: a 16-byte header (cursor, capacity) and 32-byte records
    capacity = 1 << 20
    log = torch.zeros(16 + 32 * capacity, dtype=torch.uint8, device="cuda")
    log[4:8] = torch.tensor(list(int(capacity).to_bytes(4, "little")), dtype=torch.uint8, device="cuda")
    for unit in UNITS:
        rc = getattr(lib, f"infero_tl_attach_{unit}")(ctypes.c_void_p(log.data_ptr()))
        assert rc == 0, f"cannot attach the log to {unit}"

    def step():
        logits = runner.step([StepEntry(rid, [rng.randrange(cfg["vocab_size"])], [0]) for rid in rids])
        K.argmax(logits, picked)

    for _ in range(max(3, args.steps)):            # eager, captured, then replayed
        step()
    torch.cuda.synchronize()
    log[0:4] = 0
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    step()
    e1.record()
    torch.cuda.synchronize()
    assert runner.graph_replays > 0, "the step was not a captured one"
    host = log.cpu().numpy()
    n = int(np.frombuffer(host[0:4].tobytes(), dtype=np.uint32)[0])
    n = min(n, capacity)
    rec = np.frombuffer(host[16:16 + 32 * n].tobytes(),
                        dtype=np.dtype([("t0", "<u8"), ("t1", "<u8"), ("kind", "<i4"), ("grid", "<i4"),
                                        ("block", "<i4"), ("sm", "<i4")]))
    if n == 0:
        print("timeline: no records (is the library the timeline variant?)", file=sys.stderr)
        return 1
    t_origin = int(rec["t0"].min())
    if args.raw:
        with open(args.raw, "w") as fh:
            fh.write("kind,grid,block,sm,t0_ns,t1_ns\n")
            for r in np.sort(rec, order="t0"):
                fh.write(f"{KINDS.get(int(r['kind']), r['kind'])},{r['grid']},{r['block']},{r['sm']},"
                         f"{int(r['t0']) - t_origin},{int(r['t1']) - t_origin}\n")

    # launches: records of one (kind, grid) in order of their start, cut where a block index repeats
    launches = []
    for key in sorted({(int(k), int(g)) for k, g in zip(rec["kind"], rec["grid"])}):
        sel = np.sort(rec[(rec["kind"] == key[0]) & (rec["grid"] == key[1])], order="t0")
        seen, cur = set(), []
        for r in sel:
            b = int(r["block"])
            if b in seen:
                launches.append((key, cur))
                seen, cur = set(), []
            seen.add(b)
            cur.append(r)
        if cur:
            launches.append((key, cur))
    rows = []
    for (kind, grid), rs in launches:
        t0 = np.array([int(r["t0"]) for r in rs], dtype=np.int64) - t_origin
        t1 = np.array([int(r["t1"]) for r in rs], dtype=np.int64) - t_origin
        rows.append({"kind": kind, "grid": grid, "n": len(rs), "first_start": t0.min(), "last_start": t0.max(),
                     "first_end": t1.min(), "last_end": t1.max(), "sms": len({int(r["sm"]) for r in rs})})
    rows.sort(key=lambda r: r["first_start"])
    total_us = (max(r["last_end"] for r in rows)) / 1e3
    print(f"step of {B} requests at {args.context} cached tokens, {args.layers} layers ({args.shape}): "
          f"{e0.elapsed_time(e1) * 1e3:.0f} us by events, {total_us:.0f} us from the first block's start to the last block's end; "
          f"{n} blocks in {len(rows)} launches")

    marks = [r for r in rows if r["kind"] >= 50]
    rows = [r for r in rows if r["kind"] < 50]
    # a layer's window = from the product in front of decode attention (q/k/v) up to the next one
    layer_starts = [i - 1 for i, r in enumerate(rows) if r["kind"] == 5 and i >= 1 and rows[i - 1]["kind"] == 3]
    if any(rows[i - 1]["kind"] == 4 for i, r in enumerate(rows) if r["kind"] == 5 and i >= 2):
        layer_starts = [i - 2 for i, r in enumerate(rows) if r["kind"] == 5 and i >= 2]    # (separate rotary kernel)
    per_layer = [rows[a:b] for a, b in zip(layer_starts, layer_starts[1:])]
    if len(per_layer) >= 3:
        shape = [(r["kind"], r["grid"]) for r in per_layer[1]]
        same = [L for L in per_layer[1:] if [(r["kind"], r["grid"]) for r in L] == shape]
        print(f"\naverage over {len(same)} layers (the first left out), microseconds from the start of the layer's first block:")
        print(f"{'launch':<22}{'blocks':>7}{'SMs':>5}{'first start':>13}{'all started':>13}{'first end':>11}{'last end':>10}{'busy':>8}")
        for j, (kind, grid) in enumerate(shape):
            def avg(f):
                return sum(f(L[j]) - L[0]["first_start"] for L in same) / len(same) / 1e3
            fs, ls, fe, le = (avg(lambda r, k=k: r[k]) for k in ("first_start", "last_start", "first_end", "last_end"))
            print(f"{KINDS.get(kind, kind):<22}{grid:>7}{same[0][j]['sms']:>5}{fs:>13.1f}{ls:>13.1f}{fe:>11.1f}{le:>10.1f}{le - fs:>8.1f}")
        span = sum(b[0]["first_start"] - a[0]["first_start"] for a, b in zip(same, same[1:])) / max(1, len(same) - 1) / 1e3
        print(f"a layer every {span:.1f} us")
    if marks:
        # marks inside kernels: how long after its own start each block passed the mark
        print("\nmarks inside kernels (microseconds after the block's own start: least, median, most), per launch:")
        by_kind = {}
        for (kind, grid), rs in launches:
            if kind >= 50:
                by_kind.setdefault(kind, []).append(sorted((int(r["t1"]) - int(r["t0"])) / 1e3 for r in rs))
        for kind in sorted(by_kind):
            ls = by_kind[kind][1:] or by_kind[kind]
            lo = sum(v[0] for v in ls) / len(ls)
            mid = sum(v[len(v) // 2] for v in ls) / len(ls)
            hi = sum(v[-1] for v in ls) / len(ls)
            print(f"mark {kind}: {lo:8.1f}{mid:8.1f}{hi:8.1f}   ({len(ls)} launches)")
    print("\nall launches of the step (microseconds from the first block of the step):")
    for r in rows:
        print(f"{KINDS.get(r['kind'], r['kind']):<22}{r['grid']:>7}{r['first_start'] / 1e3:>11.1f}{r['last_start'] / 1e3:>11.1f}"
              f"{r['first_end'] / 1e3:>11.1f}{r['last_end'] / 1e3:>11.1f}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
