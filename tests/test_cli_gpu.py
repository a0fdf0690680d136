"""The ``generate`` command line, run as a user runs it: a subprocess of ``bin/generate``."""
import json
import os
import re
import subprocess
import sys

import pytest

import plain_qwen2
from engine_fixtures import make_requests, model_dir, plain_model
from tiny_configs import CONFIGS

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EXE = os.path.join(ROOT, "bin", "generate")


def _run(args, env=None):
    proc = subprocess.run([sys.executable, EXE] + [str(a) for a in args], capture_output=True, text=True,
                          timeout=600, env=dict(os.environ, **(env or {})))
    return proc.returncode, proc.stdout, proc.stderr


def _tokens_and_report(stdout):
    """The generated token ids (the line after the ``kv cache`` line) and the two report lines, whose form
    is the reference's (crates/model/examples/generate.rs:149-161)."""
    lines = stdout.splitlines()
    at = next(i for i, l in enumerate(lines) if l.startswith("kv cache"))
    toks = next(l for l in lines[at + 1:] if l.strip())
    pre = next(l for l in lines if l.startswith("prefill"))
    dec = next(l for l in lines if l.startswith("decode"))
    return [int(t) for t in toks.split()], pre, dec


def test_generate_prints_the_plain_greedy_continuation():
    mdir = model_dir("B", seed=77, qk_gain=1.5)
    cfg, w = plain_model(mdir)
    prompt = make_requests("B", [23], seed=3)["r0"]
    # --greedy is the reference's SamplingParams::greedy(): temperature 0 with the default repetition
    # penalty of 1.05 still on (crates/model/src/sampling.rs:12-48), which here demotes a repeated token
    want = plain_qwen2.greedy_generate(cfg, w, prompt, 8, repetition_penalty=1.05)
    assert want != plain_qwen2.greedy_generate(cfg, w, prompt, 8), "the penalty was meant to change a token"
    rc, out, err = _run([mdir] + prompt + ["--greedy", "-n", 8, "--dtype", "float32", "--ignore-eos"], env={"GEN_CTX": "256"})
    assert rc == 0, err
    assert f"--- prompt ({len(prompt)} tokens) ---" in out
    assert re.search(r"weights  : \d+ MiB in VRAM", out)
    assert re.search(r"kv cache : float32, [\d.]+ MiB for 256 positions", out)
    toks, pre, dec = _tokens_and_report(out)
    assert toks == want
    assert re.fullmatch(rf"prefill\s+[\d.]+ ms  \([\d.]+ tok/s over {len(prompt)} tokens\)", pre), pre
    assert re.fullmatch(r"decode\s+[\d.]+ ms  \([\d.]+ tok/s over 7 tokens\)", dec), dec


def test_generate_options_for_the_pool_and_a_model_from_a_configuration(tmp_path):
    """--config with --random-weights draws the tensors a written folder of the same seed holds;
    --max-seq-len, --page-size and --num-pages set the cache's geometry; --prompt-ids gives the prompt."""
    from infero_b200.loading import write_random_model_dir
    cfg_json = dict(CONFIGS["D"])
    cfg_path = tmp_path / "config.json"
    cfg_path.write_text(json.dumps(cfg_json))
    folder = str(tmp_path / "same_seed")
    write_random_model_dir(folder, cfg_json, seed=5, dtype="float32")
    cfg, w = plain_qwen2.read_model(folder)
    prompt = make_requests("D", [70], seed=9)["r0"]
    want = plain_qwen2.greedy_generate(cfg, w, prompt, 6)
    rc, out, err = _run(["--config", cfg_path, "--random-weights", "--seed", 5, "--prompt-ids", ",".join(map(str, prompt)),
                         "--greedy", "--repetition-penalty", 1.0, "-n", 6, "--dtype", "fp32", "--ignore-eos", "--max-seq-len", 192, "--page-size", 32,
                         "--num-pages", 5])
    assert rc == 0, err
    assert re.search(r"kv cache : float32, [\d.]+ MiB for 160 positions", out), out
    toks, _, _ = _tokens_and_report(out)
    assert toks == want
    # the default sampler with a seed: the same tokens twice, inside the vocabulary, in bfloat16
    runs = []
    for _ in range(2):
        rc, out, err = _run(["--model", folder, "--prompt-len", 12, "--seed", 4, "-n", 10, "--ignore-eos",
                             "--temperature", 0.9, "--top-k", 30, "--top-p", 0.9, "--max-seq-len", 128])
        assert rc == 0, err
        runs.append(_tokens_and_report(out)[0])
    assert runs[0] == runs[1] and len(runs[0]) == 10 and all(0 <= t < cfg_json["vocab_size"] for t in runs[0])


def test_generate_refuses_what_is_not_built(tmp_path):
    mdir = model_dir("A")
    rc, out, err = _run([mdir, 1, 2, 3, "--kv-quant", "tq4"])
    assert rc == 2 and "not built" in err
    rc, out, err = _run(["--greedy"])
    assert rc == 2 and "no model" in err
