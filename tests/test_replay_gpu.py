"""The engine against the plain implementation under every way of cutting the work."""
import numpy as np
import pytest

import replay_util as R
from engine_fixtures import TOL, make_requests, make_runner, model_dir, plain_logits
from tiny_configs import CONFIGS

pytestmark = pytest.mark.gpu

LENGTHS = {"A": [40, 1, 17, 33, 64, 90], "B": [120, 3, 70, 49, 97, 130], "C": [150, 31, 66],
           "D": [150, 3, 70, 49, 97, 300], "E": [290, 31, 66, 130]}
CASES = [(n, d) for n in ("A", "B", "C", "D", "E") for d in ("float32", "bfloat16")]
# configurations whose bfloat16 steps must go through the kernels serving uses (head sizes 64 and 128)
SERVING_PATH = ("D", "E")


class ServingPath:
    """Around a bfloat16 run of a SERVING_PATH configuration: proves which path ran.  Layers went
    through the native launcher of the built-in block (which launches the tensor-core products, the
    TMA-fed decode attention and the tcgen05 prompt attention, and nothing else), and no bounded
    wait of those kernels ran out."""

    def __init__(self, name, dtype):
        self.on = name in SERVING_PATH and dtype == "bfloat16"

    def __enter__(self):
        if self.on:
            from infero_b200.kernels import tc_gemm
            from infero_b200.parts import native_block
            tc_gemm.clear_error_flag()
            self.calls = native_block.CALLS[0]
        return self

    def __exit__(self, *exc):
        if self.on and exc[0] is None:
            from infero_b200.kernels import tc_gemm
            from infero_b200.parts import native_block
            assert native_block.CALLS[0] > self.calls, "no layer went through the native launcher"
            assert tc_gemm.error_flag() == 0, "a bounded wait of a tensor-core kernel ran out"
        return False


def _check(name, dtype, steps, reqs, mdir, max_tokens=None, page_size=16):
    plain = plain_logits(mdir, reqs)
    n = max_tokens or R.max_live_tokens(steps, reqs)
    runner = make_runner(mdir, dtype, n, page_size=page_size)
    with ServingPath(name, dtype):
        got = R.replay_inprocess(runner, steps)
    assert got, "the trace asked for no logits"
    err, where = R.compare(got, plain)
    assert err <= TOL[dtype], f"{name} {dtype}: relative error {err:.3e} at {where}"
    assert not runner.manager.requests
    for a in runner.manager.allocators:
        assert a.num_free == a.num_pages
    return runner, err


@pytest.mark.parametrize("name", SERVING_PATH)
def test_a_prompt_cut_at_256_and_at_257_rows(name):
    """Products of up to 256 rows reach the residual stream as 32-bit partial sums, those of more rows as
    finished products: 32-bit too, so a token's logits do not depend on which side of that line its
    portion fell.  Both cuts against the plain implementation, and against each other much closer than
    bf16 rounding of the residual updates would leave them."""
    mdir = model_dir(name)
    reqs = make_requests(name, [300], seed=21)
    toks = reqs["r0"]
    plain = plain_logits(mdir, reqs)
    got = {}
    for cut in (256, 257):
        steps = [{"step": 0, "entries": [{"id": "r0", "tokens": toks[:cut], "want": list(range(cut - 8, cut))}], "end": []},
                 {"step": 1, "entries": [{"id": "r0", "tokens": toks[cut:], "want": list(range(len(toks) - cut))}], "end": ["r0"]}]
        runner = make_runner(mdir, "bfloat16", 320)
        with ServingPath(name, "bfloat16"):
            got[cut] = R.replay_inprocess(runner, steps)
        err, where = R.compare(got[cut], plain)
        assert err <= TOL["bfloat16"], f"{name} cut at {cut}: relative error {err:.3e} at {where}"
    both = sorted(set(got[256]) & set(got[257]))
    assert len(both) >= 40
    scale = float(np.abs(plain["r0"]).max())
    gap = max(float(np.abs(got[256][k] - got[257][k]).max()) for k in both) / scale
    assert gap <= TOL["bfloat16"] / 3, f"{name}: the two cuts differ by {gap:.3e}"


@pytest.mark.parametrize("name,dtype", CASES)
def test_each_request_alone_and_whole(name, dtype):
    mdir = model_dir(name)
    reqs = make_requests(name, LENGTHS[name], seed=1)
    _check(name, dtype, R.steps_whole(reqs), reqs, mdir)


@pytest.mark.parametrize("name,dtype", CASES)
def test_last_32_tokens_one_by_one(name, dtype):
    mdir = model_dir(name)
    reqs = make_requests(name, LENGTHS[name], seed=2)
    _check(name, dtype, R.steps_tail_decode(reqs, 32), reqs, mdir)


@pytest.mark.parametrize("name,dtype", CASES)
def test_portions_of_changing_size(name, dtype):
    mdir = model_dir(name)
    reqs = make_requests(name, LENGTHS[name], seed=3)
    _check(name, dtype, R.steps_chunked(reqs, seed=5), reqs, mdir)


@pytest.mark.parametrize("name,dtype", CASES)
@pytest.mark.parametrize("seed", [0, 1])
def test_mixed_batches_with_page_reuse(name, dtype, seed):
    mdir = model_dir(name)
    lengths = LENGTHS[name] + [l + 5 for l in LENGTHS[name]]
    reqs = make_requests(name, lengths, seed=10 + seed)
    steps = R.steps_mixed(reqs, seed=seed, max_live=4)
    runner, _ = _check(name, dtype, steps, reqs, mdir)
    assert runner.manager.pages_reused > 0, "the pool was large enough that no page was used twice"
    if CONFIGS[name].get("use_sliding_window"):
        assert runner.manager.pages_reclaimed > 0, "no page of the window group came back early"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_one_model_serves_several_pools(dtype):
    """Runners made one after the other over the same model object, each with a pool of its own
    (other addresses, other sizes): every one computes in its own cache.  The pool of the runner
    before is poisoned, so a layer that kept a pointer into it would read NaN or leave the new
    pool untouched."""
    import torch
    from infero_b200.config import EngineConfig
    from infero_b200.engine import ModelRunner
    from infero_b200.loading import load_model
    mdir = model_dir("B", seed=31, qk_gain=1.5)
    model, _ = load_model(mdir, dtype, "cuda:0")
    reqs = make_requests("B", [70, 45, 100], seed=8)
    plain = plain_logits(mdir, reqs)
    steps = R.steps_tail_decode(reqs, 6)
    earlier = None
    for pages in (8, 40, 11):
        cfg = EngineConfig(dtype=dtype, page_size=16, num_pages=pages, max_seqs=2, ctx=128, max_batch_tokens=128,
                           max_logit_rows=128, cuda_graphs=False)
        runner = ModelRunner(model, cfg)
        got = R.replay_inprocess(runner, steps)
        err, where = R.compare(got, plain)
        assert err <= TOL[dtype], f"pool of {pages} pages, {dtype}: relative error {err:.3e} at {where}"
        assert all(bool((a != 0).any()) for a in runner.storage.arrays), "this runner's own pool was never written"
        if earlier is not None:
            assert all(bool(torch.isnan(a).all()) for a in earlier.storage.arrays), "the pool before was written to"
        for a in runner.storage.arrays:
            a.fill_(float("nan"))
        earlier = runner


@pytest.mark.parametrize("name,dtype", CASES)
def test_sharp_attention(name, dtype):
    """Scaled q/k projections make single keys dominate, so a wrong or missing key shows."""
    # float32: scores spread by about +-5 (max near 25; a score s carries a rounding error near
    # |s| * 1e-6, which the softmax turns into the same relative error of a weight).  bfloat16: queries and keys are rounded to 8 bits, so a
    # score s carries an error near |s| * 2^-8 that the softmax turns into the same relative
    # error of a weight; the gain is set so that scores spread by about +-2 (max near 9),
    # which keeps single keys dominant (weights differ by e^4) and the rounding inside TOL.
    gain = ({"A": 6.0, "B": 4.5, "C": 3.0, "D": 3.9, "E": 2.4}[name] if dtype == "float32" else
            {"A": 3.6, "B": 2.8, "C": 1.9, "D": 2.5, "E": 1.75}[name])
    mdir = model_dir(name, qk_gain=gain)
    reqs = make_requests(name, LENGTHS[name][:4], seed=7)
    _check(name, dtype, R.steps_mixed(reqs, seed=3, max_live=3), reqs, mdir)
    _check(name, dtype, R.steps_tail_decode(reqs, 32), reqs, mdir)


@pytest.mark.parametrize("name", ["B", "D"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("page_size", [32, 64])
def test_other_page_sizes(name, dtype, page_size):
    mdir = model_dir(name)
    reqs = make_requests(name, [130, 70, 65, 100, 127], seed=4)
    steps = R.steps_mixed(reqs, seed=9, max_live=3)
    _check(name, dtype, steps, reqs, mdir, page_size=page_size)


@pytest.mark.parametrize("name,dtype", CASES)
def test_long_decoding(name, dtype):
    """One prompt token, then every further token alone: hundreds of single-token steps."""
    mdir = model_dir(name)
    n = {"A": 250, "B": 400, "C": 300, "D": 400, "E": 600}[name]
    reqs = make_requests(name, [n], seed=11)
    steps = R.steps_tail_decode(reqs, tail=n - 1)
    _check(name, dtype, steps, reqs, mdir)


@pytest.mark.parametrize("name,dtype", CASES)
def test_first_tokens_of_a_sequence(name, dtype):
    mdir = model_dir(name)
    reqs = make_requests(name, [1, 2, 3, 4], seed=12)
    steps = R.steps_whole(reqs)
    _check(name, dtype, steps, reqs, mdir)
    steps = R.steps_tail_decode(reqs, tail=8)
    _check(name, dtype, steps, reqs, mdir)


def test_float32_cuts_agree_bitwise():
    """On the 32-bit path a token's arithmetic does not depend on the cut at all."""
    mdir = model_dir("B")
    reqs = make_requests("B", [90, 61], seed=13)
    a = R.replay_inprocess(make_runner(mdir, "float32", 256), R.steps_whole(reqs))
    b = R.replay_inprocess(make_runner(mdir, "float32", 256), R.steps_chunked(reqs, seed=2))
    c = R.replay_inprocess(make_runner(mdir, "float32", 256), R.steps_mixed(reqs, seed=4, max_live=2))
    for key, row in a.items():
        assert np.array_equal(row, b[key]), f"chunked differs at {key}"
        if key in c:
            assert np.array_equal(row, c[key]), f"mixed differs at {key}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(tmp_path, dtype):
    """The same through bin/trace_run over a pipe."""
    mdir = model_dir("B")
    reqs = make_requests("B", [80, 45, 100, 33], seed=14)
    steps = R.steps_mixed(reqs, seed=6, max_live=3)
    n = R.max_live_tokens(steps, reqs)
    got = R.replay_subprocess(mdir, dtype, steps, n, str(tmp_path / "out"), CONFIGS["B"]["vocab_size"])
    err, where = R.compare(got, plain_logits(mdir, reqs))
    assert err <= TOL[dtype], f"trace_run {dtype}: relative error {err:.3e} at {where}"


@pytest.mark.parametrize("name,dtype", [("B", "bfloat16"), ("C", "bfloat16"), ("B", "float32"), ("D", "bfloat16"),
                                        ("E", "bfloat16")])
def test_captured_decode_steps_equal_eager_ones(name, dtype):
    """Decode steps replayed from a captured CUDA graph give the logits of eager steps, while
    requests grow across pages and the batch changes size."""
    import torch
    from infero_b200.engine import StepEntry
    mdir = model_dir(name)
    reqs = make_requests(name, [70, 40, 55], seed=21)
    plain = plain_logits(mdir, reqs)
    runner = make_runner(mdir, dtype, 512, cuda_graphs=True)
    head = 20
    for rid, toks in reqs.items():
        runner.open(rid)
        runner.step([StepEntry(rid, toks[:head], [])])
    worst = 0.0
    with ServingPath(name, dtype):
        for p in range(head, 70):
            live = [rid for rid, toks in reqs.items() if p < len(toks)]
            logits = runner.step([StepEntry(rid, [reqs[rid][p]], [0]) for rid in live])
            got = logits.float().cpu().numpy()
            for i, rid in enumerate(live):
                ref = plain[rid][p]
                worst = max(worst, float(np.abs(got[i] - ref).max() / np.abs(plain[rid]).max()))
    assert runner.graph_captures >= 2 and runner.graph_replays > 40
    assert worst <= TOL[dtype], f"{name} {dtype}: relative error {worst:.3e}"
    torch.cuda.synchronize()


@pytest.mark.parametrize("name", SERVING_PATH)
@pytest.mark.parametrize("n_live", [20, 40, 300])
def test_steps_of_many_single_tokens(name, n_live):
    """Twenty and forty requests decoding together in bfloat16 (the token-side tile of the few-token products
    is then 32 and 64 wide, and a CTA of a cluster-summed product sums several tokens), eager and captured,
    against the plain implementation; and three hundred, which is more rows than the few-token kernels take
    and more entries than a captured step holds: single tokens through the many-token products."""
    import torch
    from infero_b200.engine import StepEntry
    mdir = model_dir(name)
    lens = [14 + (7 * i) % 23 for i in range(n_live)]
    reqs = make_requests(name, lens, seed=55)
    plain = plain_logits(mdir, reqs)
    runner = make_runner(mdir, "bfloat16", 64 * n_live, max_seqs=n_live, cuda_graphs=True)
    head = 6
    for rid, toks in reqs.items():
        runner.open(rid)
        runner.step([StepEntry(rid, toks[:head], [])])
    worst = 0.0
    with ServingPath(name, "bfloat16"):
        for p in range(head, 14):                       # every request is live throughout: the batch keeps its size
            logits = runner.step([StepEntry(rid, [toks[p]], [0]) for rid, toks in reqs.items()])
            got = logits.float().cpu().numpy()
            for i, rid in enumerate(reqs):
                worst = max(worst, float(np.abs(got[i] - plain[rid][p]).max() / np.abs(plain[rid]).max()))
    assert runner.graph_replays >= 5 or n_live > runner.MAX_GRAPH_ENTRIES
    assert worst <= TOL["bfloat16"], f"{name}, {n_live} requests: relative error {worst:.3e}"
    torch.cuda.synchronize()


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_captured_steps_padded_to_a_size(dtype):
    """A batch of five single tokens runs as the captured step of six, of which one entry belongs
    to no request; as requests end the batch shrinks through sizes that capture nothing new.  The
    logits of the real entries are those of eager steps (float32: bit for bit, since a row's
    arithmetic does not depend on the batch)."""
    import torch
    from infero_b200.engine import StepEntry
    name = "B"
    mdir = model_dir(name)
    lens = [64, 57, 50, 43, 36]
    reqs = make_requests(name, lens, seed=33)
    head = 12

    def run(graphs):
        runner = make_runner(mdir, dtype, 512, cuda_graphs=graphs)
        for rid, toks in reqs.items():
            runner.open(rid)
            runner.step([StepEntry(rid, toks[:head], [])])
        out = {rid: [] for rid in reqs}
        for p in range(head, max(lens)):
            live = [rid for rid, toks in reqs.items() if p < len(toks)]
            logits = runner.step([StepEntry(rid, [reqs[rid][p]], [0]) for rid in live]).float().cpu()
            for i, rid in enumerate(live):
                out[rid].append(logits[i].clone())
            for rid in list(reqs):
                if p + 1 == len(reqs[rid]):
                    runner.close(rid)
        runner.manager.check()
        assert not runner.manager.requests
        return out, runner

    eager, _ = run(False)
    captured, runner = run(True)
    assert runner._graph_size(5) == 6 and runner._graph_size(3) == 3 and runner._graph_size(7) == 8
    # sizes met: 5 -> 6, 4, 3, 2, 1: five graphs at most for this key bound, far fewer than steps
    assert 2 <= runner.graph_captures <= 6 and runner.graph_replays > 30
    worst = 0.0
    for rid in reqs:
        for a, b in zip(eager[rid], captured[rid]):
            if dtype == "float32":
                assert torch.equal(a, b), f"{rid}: a padded captured step changed a real row"
            worst = max(worst, float((a - b).abs().max() / a.abs().max()))
    assert worst <= TOL[dtype]
    torch.cuda.synchronize()


@pytest.mark.parametrize("name", ["A", "B"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_entry_point(name, dtype):
    """Engine.generate (scheduler, prompt portions, captured decode steps, device argmax)
    against the plain implementation's argmax continuation."""
    import plain_qwen2
    from engine_fixtures import plain_model
    from infero_b200.engine import Engine
    from infero_b200.sampling import SamplingParams
    # wider weights than 0.02 so that the largest logit leads by more than bf16 rounding
    mdir = model_dir(name, seed=77, qk_gain=1.5)
    cfg, w = plain_model(mdir)
    reqs = make_requests(name, [9, 30, 3, 21], seed=31)
    n_new = 10
    want = [plain_qwen2.greedy_generate(cfg, w, toks, n_new) for toks in reqs.values()]
    eng = Engine(mdir, dtype=dtype, ctx=128, max_seqs=3, kv_slots=256, max_batch_tokens=32)
    got = eng.generate(list(reqs.values()), SamplingParams(temperature=0.0, repetition_penalty=1.0),
                       max_new_tokens=n_new, ignore_eos=True)
    if dtype == "float32":
        assert got == want
    else:
        # bfloat16 may pick another token only where the plain logits nearly tie; from there on
        # the two continuations are different sequences and are not compared
        for toks, g, x in zip(reqs.values(), got, want):
            assert len(g) == n_new
            for i in range(n_new):
                if g[i] != x[i]:
                    row = plain_qwen2.forward(cfg, w, list(toks) + x[:i])[-1]
                    gap = float(row.max() - row[g[i]]) / float(row.abs().max())
                    assert gap <= TOL[dtype], f"token {i}: picked {g[i]}, plain {x[i]}, gap {gap:.3e}"
                    break
    assert eng.runner.graph_replays > 0
    assert not eng.runner.manager.requests


def test_generation_under_page_pressure_equals_plain():
    """More requests than the cache can hold at once: requests wait, the youngest is preempted and
    recomputed, window pages come back early, captured steps are padded and run ahead; in 32-bit
    every request still gets exactly the plain implementation's greedy continuation."""
    import plain_qwen2
    from engine_fixtures import plain_model
    from infero_b200.engine import Engine
    from infero_b200.sampling import SamplingParams
    mdir = model_dir("B", seed=77, qk_gain=1.5)
    cfg, w = plain_model(mdir)
    lens = [33, 5, 48, 17, 60, 9, 26, 41, 3, 55]
    reqs = make_requests("B", lens, seed=52)
    n_new = 14
    want = {rid: plain_qwen2.greedy_generate(cfg, w, toks, n_new) for rid, toks in reqs.items()}
    eng = Engine(mdir, dtype="float32", ctx=96, max_seqs=4, kv_slots=10 * 16, max_batch_tokens=24)
    pick = SamplingParams(temperature=0.0, repetition_penalty=1.0)
    for rid, toks in reqs.items():
        eng.add_request(toks, pick, max_new_tokens=n_new, ignore_eos=True, rid=rid)
    got = {rid: [] for rid in reqs}
    reasons = {}
    for _ in range(5000):
        if eng.is_idle():
            break
        for ev in eng.step():
            if ev.token is not None:
                got[ev.rid].append(ev.token)
            if ev.finished:
                reasons[ev.rid] = ev.reason
        eng.runner.manager.check()
    assert eng.is_idle()
    assert eng.scheduler.stats["preemptions"] > 0, "the pool was meant to be too small"
    assert set(reasons.values()) == {"length"}
    for rid in reqs:
        assert got[rid] == want[rid], f"request {rid}"
    assert not eng.runner.manager.requests
    for a in eng.runner.manager.allocators:
        assert a.num_free == a.num_pages


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_running_ahead_changes_no_token(dtype):
    """One step in flight (tokens fed from the device, end-of-sequence seen a step late) against
    waiting for every step's tokens: same tokens, same reasons, nothing left in the cache."""
    from infero_b200.engine import Engine
    from infero_b200.sampling import SamplingParams
    mdir = model_dir("B", seed=77, qk_gain=1.5)
    reqs = make_requests("B", [9, 30, 3, 21, 14, 40], seed=41)
    results = []
    for ahead in (False, True):
        eng = Engine(mdir, dtype=dtype, ctx=160, max_seqs=3, kv_slots=320, max_batch_tokens=32, run_ahead=ahead)
        # greedy rows and seeded temperature rows; a handful of token ids end a request
        eos = tuple(range(0, 1000, 9))
        for i, toks in enumerate(reqs.values()):
            p = SamplingParams(temperature=0.0 if i % 2 == 0 else 0.9, top_k=8, top_p=0.95, repetition_penalty=1.0, seed=5 + i)
            eng.add_request(toks, p, max_new_tokens=24, eos_token_ids=eos, rid=i)
        out, why = {}, {}
        while not eng.is_idle():
            for ev in eng.step():
                if ev.token is not None:
                    out.setdefault(ev.rid, []).append(ev.token)
                if ev.finished:
                    why[ev.rid] = ev.reason
        results.append((out, why))
        assert not eng.runner.manager.requests
        if ahead:
            assert eng.scheduler.stats["steps_ahead"] > 0
    assert results[0] == results[1]
    assert "stop" in results[0][1].values() or "length" in results[0][1].values()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_default_sampling_runs_ahead_and_changes_no_token(dtype):
    """The reference's default sampling (temperature, top-k, top-p and a repetition penalty over the
    last 256 tokens): the penalty is worked out from histories kept on the device, so steps run
    ahead; the tokens are those of an engine that waits for every step, and of one that is preempted."""
    from infero_b200.engine import Engine
    from infero_b200.sampling import SamplingParams
    mdir = model_dir("B", seed=77, qk_gain=1.5)
    reqs = make_requests("B", [9, 30, 3, 21, 14], seed=43)
    results = []
    # (a recomputed request sees its tokens again in other portions: the same logits bit for bit only in 32-bit)
    runs = [(False, 400), (True, 400)] + ([(True, 7 * 16)] if dtype == "float32" else [])
    for ahead, slots in runs:
        eng = Engine(mdir, dtype=dtype, ctx=128, max_seqs=3, kv_slots=slots, max_batch_tokens=32, run_ahead=ahead)
        for i, toks in enumerate(reqs.values()):
            p = SamplingParams(seed=7 + i) if i % 2 == 0 else SamplingParams(temperature=0.0, repetition_penalty=1.3,
                                                                               repetition_window=5)
            eng.add_request(toks, p, max_new_tokens=40, ignore_eos=True, rid=i)
        out = {}
        while not eng.is_idle():
            for ev in eng.step():
                if ev.token is not None:
                    out.setdefault(ev.rid, []).append(ev.token)
        results.append(out)
        if ahead:
            assert eng.scheduler.stats["steps_ahead"] > 0
        if slots < 400:
            assert eng.scheduler.stats["preemptions"] > 0, "the pool was meant to be too small"
        assert not eng.runner.manager.requests
    assert results[0] == results[1], "running ahead changed a token"
    if len(results) > 2:
        assert results[0] == results[2], "a preempted request did not continue with its history"


def test_a_missed_wait_fails_the_step_and_leaves_the_engine_usable():
    """The flag that kernels raise when one of their bounded waits runs out travels to the host with
    the picked tokens.  Here the host sets it (no kernel has to miss a wait): the next step's tokens are
    not handed on, every request ends with an error, nothing stays in the cache, and the same engine
    then serves a new request as if nothing had happened."""
    import plain_qwen2
    from engine_fixtures import plain_model
    from infero_b200.engine import Engine
    from infero_b200.kernels import tc_gemm
    from infero_b200.sampling import SamplingParams
    mdir = model_dir("D", seed=77, qk_gain=1.5)
    reqs = make_requests("D", [20, 9, 33], seed=5)
    pick = SamplingParams(temperature=0.0, repetition_penalty=1.0)
    eng = Engine(mdir, dtype="bfloat16", ctx=128, max_seqs=4, kv_slots=512, max_batch_tokens=64)
    tc_gemm.clear_error_flag()
    for rid, toks in reqs.items():
        eng.add_request(toks, pick, max_new_tokens=30, ignore_eos=True, rid=rid)
    seen = []
    for _ in range(4):
        seen += eng.step()
    assert seen and all(ev.reason != "error" for ev in seen)
    tc_gemm.set_error_flag(4)
    events = []
    for _ in range(3):                       # (a step that ran ahead may still deliver the step before)
        events += eng.step()
        if any(ev.reason == "error" for ev in events):
            break
    failed = {ev.rid for ev in events if ev.finished and ev.reason == "error"}
    assert failed == set(reqs), f"requests that ended with an error: {failed}"
    assert any("bounded wait" in (ev.message or "") for ev in events)
    assert eng.is_idle() and not eng.runner.manager.requests
    eng.runner.manager.check()
    for a in eng.runner.manager.allocators:
        assert a.num_free == a.num_pages
    assert tc_gemm.error_flag() == 0, "the flag was not cleared"
    # the engine is still good
    cfg, w = plain_model(mdir)
    prompt = make_requests("D", [17], seed=6)["r0"]
    got = eng.generate([prompt], pick, max_new_tokens=6, ignore_eos=True)[0]
    want = plain_qwen2.greedy_generate(cfg, w, prompt, 6)
    assert len(got) == 6
    for i in range(6):
        if got[i] != want[i]:
            row = plain_qwen2.forward(cfg, w, list(prompt) + want[:i])[-1]
            assert float(row.max() - row[got[i]]) / float(row.abs().max()) <= TOL["bfloat16"]
            break


@pytest.mark.parametrize("name,dtype", [("B", "float32"), ("D", "bfloat16"), ("D", "float32")])
def test_the_window_group_runs_in_a_far_smaller_pool(name, dtype):
    """Each group of layers has a pool of its own size: the layers that keep a window of 48 keys get
    what four live requests can hold at once, a third of what the all-keys layer gets, and the mixed
    trace (long prompts in portions, pages coming back as the window passes) still equals the plain
    implementation.  The memory that early returns save is memory that is never allocated."""
    from infero_b200.cache.storage import window_pool_pages
    from infero_b200.config import EngineConfig
    from infero_b200.engine import ModelRunner
    from infero_b200.loading import load_model
    mdir = model_dir(name)
    model, _ = load_model(mdir, dtype, "cuda:0")
    cfg = EngineConfig(dtype=dtype, page_size=16, num_pages=120, max_seqs=4, ctx=320, max_batch_tokens=256,
                       max_logit_rows=256, cuda_graphs=False)
    runner = ModelRunner(model, cfg)
    small = window_pool_pages(48, 16, 4, 256)
    assert small == 40 and runner.pages_per_group == [120, small]
    assert [a.num_pages for a in runner.manager.allocators] == [120, small]
    n_win = len(model.spec.schedule) - 1                     # layers from max_window_layers = 1 on
    per_page = runner.storage.bytes_per_token(0) * 16
    assert runner.storage.bytes_per_token(1) == n_win * runner.storage.bytes_per_token(0)
    assert runner.storage.bytes() == per_page * 121 + n_win * per_page * (small + 1)
    reqs = make_requests(name, [300, 150, 97, 210, 305, 60, 280], seed=17)
    steps = R.steps_mixed(reqs, seed=5, max_live=4)
    plain = plain_logits(mdir, reqs)
    with ServingPath(name, dtype):
        got = R.replay_inprocess(runner, steps)
    err, where = R.compare(got, plain)
    assert err <= TOL[dtype], f"{name} {dtype}: relative error {err:.3e} at {where}"
    assert runner.manager.pages_reclaimed > 20 and runner.manager.pages_reused > 0
    assert [runner.manager.free_pages(g) for g in (0, 1)] == [120, small] and not runner.manager.requests


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("E", "bfloat16"), ("E", "float32")])
def test_a_request_cut_back_continues_with_other_tokens(name, dtype):
    """Truncation (the reference's KvPool::truncate, crates/model/src/cache.rs:656-679): a request is
    cut back to a prefix and continues with other tokens; the logits are those of the new sequence, and
    the pages behind the cut were given back and used again."""
    from infero_b200.engine import StepEntry
    mdir = model_dir(name)
    base = make_requests(name, [100], seed=21)["r0"]
    other = make_requests(name, [100], seed=22)["r0"]
    runner = make_runner(mdir, dtype, 128)
    runner.open("x")
    runner.step([StepEntry("x", base, [99])])
    free_before = runner.manager.free_pages(0)
    runner.truncate("x", 37)
    assert runner.length("x") == 37 and runner.manager.free_pages(0) == free_before + 4
    new = base[:37] + other[37:90]
    rows = [runner.step([StepEntry("x", new[37:70], list(range(33)))]).float().cpu().numpy()]
    for p in range(70, 90):
        rows.append(runner.step([StepEntry("x", [new[p]], [0])]).float().cpu().numpy())
    got = {("x", 37 + i): row for i, row in enumerate(np.concatenate(rows))}
    err, where = R.compare(got, plain_logits(mdir, {"x": new}))
    assert err <= TOL[dtype], f"{name} {dtype}: relative error {err:.3e} at {where}"
    runner.manager.check()
    runner.close("x")
    assert runner.manager.free_pages(0) == runner.manager.allocators[0].num_pages
    # where a window has passed, the keys are gone and the cut is refused
    if name == "E":
        wdir = model_dir("D")
        r2 = make_runner(wdir, dtype, 128)
        r2.open("y")
        r2.step([StepEntry("y", make_requests("D", [100], seed=1)["r0"], [])])
        with pytest.raises(ValueError, match="window"):
            r2.truncate("y", 60)
        r2.truncate("y", 99)
