"""Helpers that cut requests into steps in several ways and replay them."""
from __future__ import annotations

import json
import os
import random
import subprocess
import sys
from typing import Dict, List, Sequence, Tuple

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def round64(n: int) -> int:
    return -(-n // 64) * 64


# ---- ways of cutting --------------------------------------------------------------------------
def steps_whole(reqs: Dict[str, List[int]]) -> List[dict]:
    """Each request alone and whole, all logits wanted."""
    steps = []
    for i, (rid, toks) in enumerate(reqs.items()):
        steps.append({"step": i, "entries": [{"id": rid, "tokens": toks, "want": list(range(len(toks)))}],
                      "end": [rid]})
    return steps


def steps_tail_decode(reqs: Dict[str, List[int]], tail: int = 32) -> List[dict]:
    """Most of each request in one step, its last ``tail`` tokens one by one."""
    steps = []
    n = 0
    for rid, toks in reqs.items():
        head = max(1, len(toks) - tail)
        steps.append({"step": n, "entries": [{"id": rid, "tokens": toks[:head], "want": [head - 1]}], "end": []})
        n += 1
        for p in range(head, len(toks)):
            steps.append({"step": n, "entries": [{"id": rid, "tokens": [toks[p]], "want": [0]}],
                          "end": [rid] if p == len(toks) - 1 else []})
            n += 1
        if head == len(toks):
            steps[-1]["end"] = [rid]
    return steps


def steps_chunked(reqs: Dict[str, List[int]], seed: int = 0, sizes=(2, 3, 5, 8, 13, 17, 31, 2, 64, 7)) -> List[dict]:
    """Portions of changing size, down to two tokens; every position wanted."""
    steps = []
    n = 0
    rng = random.Random(seed)
    for rid, toks in reqs.items():
        p = 0
        k = rng.randrange(len(sizes))
        while p < len(toks):
            size = min(sizes[k % len(sizes)], len(toks) - p)
            k += 1
            chunk = toks[p:p + size]
            p += size
            steps.append({"step": n, "entries": [{"id": rid, "tokens": chunk, "want": list(range(size))}],
                          "end": [rid] if p == len(toks) else []})
            n += 1
    return steps


def steps_mixed(reqs: Dict[str, List[int]], seed: int = 0, max_live: int = 4, tail: int = 12) -> List[dict]:
    """Up to ``max_live`` requests live at once: prompt portions of some beside single tokens
    of others; requests sometimes sit out a step; new ones start as others end."""
    rng = random.Random(seed)
    waiting = list(reqs.items())
    live: List[Tuple[str, List[int], int]] = []      # rid, tokens, done
    steps = []
    n = 0
    while waiting or live:
        while waiting and len(live) < max_live and (not live or rng.random() < 0.7):
            rid, toks = waiting.pop(0)
            live.append((rid, toks, 0))
        entries, ended, nxt = [], [], []
        for rid, toks, done in live:
            if len(live) > 1 and rng.random() < 0.2 and entries:
                nxt.append((rid, toks, done))          # sits this step out
                continue
            remaining = len(toks) - done
            if remaining <= tail:
                size = 1
            else:
                size = min(remaining - tail, rng.choice([2, 3, 4, 7, 16, 33, 50]))
            chunk = toks[done:done + size]
            want = list(range(size)) if rng.random() < 0.8 else [size - 1]
            entries.append({"id": rid, "tokens": chunk, "want": want})
            done += size
            if done == len(toks):
                ended.append(rid)
            else:
                nxt.append((rid, toks, done))
        rng.shuffle(entries)
        live = nxt
        if entries:
            steps.append({"step": n, "entries": entries, "end": ended})
            n += 1
    return steps


def max_live_tokens(steps: Sequence[dict], reqs: Dict[str, List[int]]) -> int:
    """Most tokens live requests hold at any time, each rounded up to a multiple of 64."""
    live = set()
    best = 0
    for st in steps:
        for e in st["entries"]:
            live.add(e["id"])
        best = max(best, sum(round64(len(reqs[r])) for r in live))
        for r in st.get("end", []):
            live.discard(r)
    return best


# ---- replay -------------------------------------------------------------------------------------
def replay_inprocess(runner, steps: Sequence[dict]) -> Dict[Tuple[str, int], np.ndarray]:
    """Drive a ModelRunner with the steps; returns (request, position) -> logits row."""
    from infero_b200.engine import StepEntry
    out: Dict[Tuple[str, int], np.ndarray] = {}
    pos: Dict[str, int] = {}
    for st in steps:
        entries = []
        for e in st["entries"]:
            if e["id"] not in runner.manager.requests:
                runner.open(e["id"])
                pos[e["id"]] = 0
            entries.append(StepEntry(e["id"], e["tokens"], e.get("want", [])))
        logits = runner.step(entries)
        if logits is not None:
            arr = logits.float().cpu().numpy()
            r = 0
            for e in st["entries"]:
                for w in e.get("want", []):
                    out[(e["id"], pos[e["id"]] + w)] = arr[r]
                    r += 1
            assert r == arr.shape[0]
        for e in st["entries"]:
            pos[e["id"]] += len(e["tokens"])
        for rid in st.get("end", []):
            runner.close(rid)
        runner.manager.check()
    return out


def replay_subprocess(model_dir: str, dtype: str, steps: Sequence[dict], max_tokens: int, out_dir: str,
                      vocab: int, env=None, cwd=None, page_size=None) -> Dict[Tuple[str, int], np.ndarray]:
    """Drive bin/trace_run over a pipe, waiting for ``done <step>`` after each line."""
    exe = os.path.join(cwd or ROOT, "bin", "trace_run")
    cmd = [sys.executable, exe, "--model", model_dir, "--dtype", dtype, "--out", out_dir,
           "--max-tokens", str(max_tokens)]
    if page_size:
        cmd += ["--page-size", str(page_size)]
    proc = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, env=env, cwd=cwd)
    out: Dict[Tuple[str, int], np.ndarray] = {}
    pos: Dict[str, int] = {}
    try:
        for st in steps:
            proc.stdin.write(json.dumps(st) + "\n")
            proc.stdin.flush()
            line = proc.stdout.readline().strip()
            assert line == f"done {st['step']}", f"trace_run answered {line!r}"
            n_want = sum(len(e.get("want", [])) for e in st["entries"])
            if n_want:
                arr = np.fromfile(os.path.join(out_dir, f"{st['step']}.f32"), dtype="<f4").reshape(n_want, vocab)
                r = 0
                for e in st["entries"]:
                    for w in e.get("want", []):
                        out[(e["id"], pos.get(e["id"], 0) + w)] = arr[r]
                        r += 1
            for e in st["entries"]:
                pos[e["id"]] = pos.get(e["id"], 0) + len(e["tokens"])
        proc.stdin.close()
        rc = proc.wait(timeout=120)
        assert rc == 0, f"trace_run exited with {rc}"
    finally:
        if proc.poll() is None:
            proc.kill()
    return out


def compare(got: Dict[Tuple[str, int], np.ndarray], plain: Dict[str, np.ndarray]) -> Tuple[float, Tuple]:
    """Largest |got - plain| over all rows, relative to the largest |plain| logit of its
    request, and where it is."""
    worst, where = 0.0, None
    for (rid, p), row in got.items():
        ref = plain[rid]
        scale = float(np.abs(ref).max()) + 1e-30
        err = float(np.abs(row.astype(np.float64) - ref[p]).max()) / scale
        if not np.isfinite(err):
            return float("inf"), (rid, p)
        if err > worst:
            worst, where = err, (rid, p)
    return worst, where
