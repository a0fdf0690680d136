"""The measurement tools run: the timeline of a decode step (the library's timeline variant, every block's
first and last nanosecond) and one kernel alone."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(args):
    env = dict(os.environ, PYTHONPATH=ROOT)
    env.pop("INFERO_TIMELINE", None)
    r = subprocess.run([sys.executable, "-m"] + args, capture_output=True, text=True, cwd=ROOT, env=env, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    return r.stdout


def test_timeline_of_a_decode_step():
    """The averaged layer of a step of single tokens: its launches in the order they started, decode
    attention among them, and launches seen to start before the one in front has ended (programmatic
    dependent launch)."""
    out = _run(["infero_b200.tools.timeline", "--batch", "2", "--context", "300", "--layers", "6", "--shape", "0.5b"])
    assert "decode attention" in out and "a layer every" in out, out[-1500:]
    rows = [ln.split() for ln in out.splitlines() if ln.startswith(("product", "decode attention", "norm"))]
    assert len(rows) >= 5
    # the table of the averaged layer: columns are name..., blocks, SMs, first start, all started, first end, last end, busy
    layer = []
    for ln in out.splitlines():
        if ln.startswith("a layer every"):
            break
        if ln.startswith(("product", "decode attention", "norm", "swiglu", "rotary")):
            layer.append(ln)
    assert any(ln.startswith("decode attention") for ln in layer)
    firsts = [float(ln.split()[-5]) for ln in layer]
    ends = [float(ln.split()[-2]) for ln in layer]
    assert all(b >= a for a, b in zip(firsts, firsts[1:])), "launches are listed in the order they started"
    assert any(firsts[i + 1] < ends[i] for i in range(len(layer) - 1)), "no launch started under the one in front"


def test_one_kernel_alone():
    out = _run(["infero_b200.tools.kernel_bench", "attn_decode_fused", "--batch", "2", "--context", "512", "--reps", "3"])
    assert "attn_decode_fused:" in out and "us per launch" in out and "error flag" not in out
