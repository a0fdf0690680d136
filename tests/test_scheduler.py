"""Scheduler decisions with a fake step function (no GPU)."""
import random

import pytest

from infero_b200.cache import CacheManager, GroupSpec
from infero_b200.engine.scheduler import Request, Scheduler
from infero_b200.sampling import SamplingParams


class FakeExecutor:
    """Reserves and commits pages like the real step function; the 'model' returns
    (sum of the request's tokens so far + position) % vocab, so outputs are checkable."""

    def __init__(self, manager, vocab=100):
        self.manager = manager
        self.vocab = vocab
        self.batches = []
        self.seen = {}

    def __call__(self, items):
        self.batches.append([(it.run.req.rid, len(it.tokens), it.is_decode, it.samples) for it in items])
        out = []
        for it in items:
            self.manager.reserve(it.run.rc, len(it.tokens))
        for it in items:
            self.manager.commit(it.run.rc, len(it.tokens))
            hist = self.seen.setdefault(it.run.req.rid, [])
            assert it.run.rc.length - len(it.tokens) == len(hist) or it.run.preemptions, "tokens fed out of order"
            if it.run.rc.length - len(it.tokens) == 0:
                hist.clear()
            hist.extend(it.tokens)
            if it.samples:
                out.append((sum(hist) + len(hist)) % self.vocab)
        self.manager.check()
        return out


def expected_output(prompt, n, vocab=100, eos=()):
    seq, out = list(prompt), []
    for _ in range(n):
        t = (sum(seq) + len(seq)) % vocab
        if t in eos:
            break
        out.append(t)
        seq.append(t)
    return out


def make(num_pages=64, page_size=16, max_seqs=4, budget=64, ctx=512, groups=None, chunk=None):
    m = CacheManager(groups or [GroupSpec(None)], num_pages=num_pages, page_size=page_size, max_requests=max_seqs)
    ex = FakeExecutor(m)
    return Scheduler(m, ex, max_seqs=max_seqs, max_batch_tokens=budget, ctx=ctx, max_prefill_chunk=chunk), ex, m


def run_all(s, limit=5000):
    out, reasons = {}, {}
    for _ in range(limit):
        if s.is_idle():
            break
        for ev in s.step():
            if ev.token is not None:
                out.setdefault(ev.rid, []).append(ev.token)
            if ev.finished:
                reasons[ev.rid] = (ev.reason, ev.message)
    assert s.is_idle(), "scheduler did not drain"
    return out, reasons


def req(rid, prompt, n=8, **kw):
    return Request(rid, list(prompt), SamplingParams.greedy(), max_new_tokens=n, **kw)


def test_prompt_is_cut_under_the_token_budget_and_decodes_go_first():
    s, ex, m = make(budget=32)
    s.enqueue(req("a", range(1, 71), n=3))
    out, reasons = run_all(s)
    assert [b[0][1] for b in ex.batches[:3]] == [32, 32, 6]
    assert [b[0][3] for b in ex.batches[:3]] == [False, False, True]
    assert out["a"] == expected_output(range(1, 71), 3) and reasons["a"][0] == "length"
    # a second request joins while the first decodes: decode item first, prompt portion after
    s, ex, m = make(budget=16)
    s.enqueue(req("a", [1, 2, 3], n=6))
    s.step()
    s.enqueue(req("b", range(40), n=2))
    s.step()
    assert ex.batches[1][0] == ("a", 1, True, True) and ex.batches[1][1] == ("b", 15, False, False)
    out, _ = run_all(s)
    assert m.free_pages(0) == 64


def test_several_prompts_share_a_step():
    s, ex, m = make(budget=64)
    s.enqueue(req("a", range(20), n=1))
    s.enqueue(req("b", range(30), n=1))
    s.enqueue(req("c", range(30), n=1))
    s.step()
    assert ex.batches[0] == [("a", 20, False, True), ("b", 30, False, True), ("c", 14, False, False)]


def test_eos_stops_without_appending_and_frees():
    prompt = [5, 6, 7]
    full = expected_output(prompt, 10)
    eos = full[4]
    s, ex, m = make()
    s.enqueue(req("a", prompt, n=10, eos_token_ids=(eos,)))
    out, reasons = run_all(s)
    assert out["a"] == full[:full.index(eos)] and reasons["a"][0] == "stop"
    assert m.free_pages(0) == 64 and not m.requests
    s.enqueue(req("b", prompt, n=10, eos_token_ids=(eos,), ignore_eos=True))
    out, reasons = run_all(s)
    assert out["b"] == full and reasons["b"][0] == "length"


def test_bad_requests_are_refused_up_front():
    s, ex, m = make(ctx=32, num_pages=2)
    s.enqueue(req("empty", []))
    s.enqueue(req("long", range(40)))
    s.enqueue(req("fits_ctx_not_pool", range(31)))          # 32 tokens = 2 pages: fits exactly
    out, reasons = run_all(s)
    assert reasons["empty"] == ("error", "empty prompt")
    assert reasons["long"][0] == "error" and "context" in reasons["long"][1]
    assert reasons["fits_ctx_not_pool"][0] == "length"
    s, ex, m = make(ctx=512, num_pages=2)
    s.enqueue(req("never", range(60)))
    out, reasons = run_all(s)
    assert reasons["never"][0] == "error" and "pool" in reasons["never"][1]


def test_admission_waits_for_pages_and_keeps_fifo_order():
    s, ex, m = make(num_pages=6, budget=128, max_seqs=4)
    s.enqueue(req("a", range(60), n=4))      # 4 pages
    s.enqueue(req("b", range(40), n=4))      # 3 pages: does not fit beside a
    s.enqueue(req("c", range(5), n=4))       # would fit, but waits behind b
    first = s.step()
    assert [r.req.rid for r in s.running] == ["a"] and len(s.waiting) == 2
    out, reasons = run_all(s)
    out["a"] = [ev.token for ev in first if ev.token is not None] + out["a"]
    assert out["a"] == expected_output(range(60), 4)
    assert out["b"] == expected_output(range(40), 4)
    assert out["c"] == expected_output(range(5), 4)
    first_seen = [next(i for i, b in enumerate(ex.batches) if any(x[0] == r for x in b)) for r in "abc"]
    assert first_seen == sorted(first_seen)


def test_max_seqs_bounds_the_running_set():
    s, ex, m = make(max_seqs=2)
    for i in range(5):
        s.enqueue(req(i, [i + 1, 2, 3], n=3))
    for _ in range(200):
        if s.is_idle():
            break
        s.step()
        assert len(s.running) <= 2
    assert s.stats["finished"] == 5


def test_when_pages_run_out_the_youngest_is_recomputed_and_outputs_do_not_change():
    # three requests that fit at admission but outgrow an 8-page pool while decoding
    s, ex, m = make(num_pages=8, budget=64, max_seqs=3)
    prompts = {"a": list(range(1, 31)), "b": list(range(2, 33)), "c": list(range(3, 30))}
    for k, p in prompts.items():
        s.enqueue(req(k, p, n=40))
    out, reasons = run_all(s)
    assert s.stats["preemptions"] > 0
    for k, p in prompts.items():
        assert out[k] == expected_output(p, 40), k
        assert reasons[k][0] == "length"
    assert m.free_pages(0) == 8 and not m.requests


def test_a_request_that_holds_the_whole_pool_ends_with_length():
    s, ex, m = make(num_pages=2, budget=64)
    s.enqueue(req("a", range(20), n=100))
    out, reasons = run_all(s)
    assert reasons["a"] == ("length", "cache exhausted")
    assert out["a"] == expected_output(range(20), 100)[:len(out["a"])] and 10 <= len(out["a"]) <= 13
    assert m.free_pages(0) == 2


def test_context_limit_ends_with_length():
    s, ex, m = make(ctx=24)
    s.enqueue(req("a", range(20), n=100))
    out, reasons = run_all(s)
    assert reasons["a"][0] == "length" and len(out["a"]) == 4


def test_prefill_chunk_cap():
    s, ex, m = make(budget=64, chunk=10)
    s.enqueue(req("a", range(25), n=1))
    run_all(s)
    assert [b[0][1] for b in ex.batches] == [10, 10, 5]


@pytest.mark.parametrize("seed", range(6))
def test_random_load_with_a_window_group_drains_and_matches(seed):
    rng = random.Random(seed)
    s, ex, m = make(num_pages=rng.randint(10, 20), page_size=16, max_seqs=4, budget=rng.choice([16, 48, 96]),
                    groups=[GroupSpec(None), GroupSpec(32)])
    prompts = {}
    for i in range(12):
        prompts[i] = [rng.randrange(100) for _ in range(rng.randint(1, 70))]
    pending = list(prompts.items())
    out, reasons = {}, {}
    for _ in range(5000):
        while pending and rng.random() < 0.3:
            k, p = pending.pop(0)
            s.enqueue(req(k, p, n=rng.randint(1, 30)))
        if s.is_idle() and not pending:
            break
        for ev in s.step():
            if ev.token is not None:
                out.setdefault(ev.rid, []).append(ev.token)
            if ev.finished:
                reasons[ev.rid] = ev.reason
        m.check()
    assert s.is_idle() and not pending
    for k, p in prompts.items():
        assert reasons[k] == "length"
        assert out[k] == expected_output(p, len(out[k]))
    assert all(a.num_free == a.num_pages for a in m.allocators)


# ---- running ahead: one step in flight ---------------------------------------------------------------
class FakeLauncher(FakeExecutor):
    """The same fake model behind the asynchronous interface: a step is 'launched' (pages taken,
    the picked tokens left 'on the device') and its tokens are only handed over by .result()."""

    class _Pending:
        def __init__(self, tokens, log):
            self._tokens, self._log = tokens, log

        def result(self):
            self._log.append("read")
            return self._tokens

    def __init__(self, manager, vocab=100):
        super().__init__(manager, vocab)
        self.device = {}               # rid -> last picked token, as the sampler leaves it on the device
        self.log = []

    def launch(self, items):
        from infero_b200.engine.step import FROM_DEVICE
        resolved = []                  # what the device would do: take the request's last pick
        for it in items:
            toks = [self.device[it.run.req.rid]] if it.tokens == [FROM_DEVICE] else list(it.tokens)
            resolved.append(toks)
        self.log.append("launch")
        self.batches.append([(it.run.req.rid, len(t), it.is_decode, it.samples) for it, t in zip(items, resolved)])
        out = []
        for it, toks in zip(items, resolved):
            self.manager.reserve(it.run.rc, len(toks))
        for it, toks in zip(items, resolved):
            self.manager.commit(it.run.rc, len(toks))
            hist = self.seen.setdefault(it.run.req.rid, [])
            if it.run.rc.length - len(toks) == 0:
                hist.clear()
            hist.extend(toks)
            if it.samples:
                tok = (sum(hist) + len(hist)) % self.vocab
                self.device[it.run.req.rid] = tok
                out.append(tok)
        return self._Pending(out, self.log)


def make_ahead(run_ahead=True, **kw):
    m = CacheManager([GroupSpec(None)], num_pages=kw.get("num_pages", 64), page_size=16, max_requests=kw.get("max_seqs", 4))
    ex = FakeLauncher(m)
    s = Scheduler(m, ex, max_seqs=kw.get("max_seqs", 4), max_batch_tokens=kw.get("budget", 64), ctx=kw.get("ctx", 512),
                  launch=ex.launch, run_ahead=run_ahead)
    return s, ex, m


def pure(rid, prompt, n=8, **kw):
    return Request(rid, list(prompt), SamplingParams(temperature=0.0, repetition_penalty=1.0), max_new_tokens=n, **kw)


def test_running_ahead_launches_the_next_step_before_reading_this_one():
    s, ex, m = make_ahead()
    s.enqueue(pure("a", range(1, 20), n=12))
    out, reasons = run_all(s)
    assert out["a"] == expected_output(range(1, 20), 12) and reasons["a"][0] == "length"
    assert s.stats["steps_ahead"] >= 8
    # in steady state a launch comes between two reads
    assert "launch launch read launch read" in " ".join(ex.log)
    assert all(a.num_free == a.num_pages for a in m.allocators)


def test_running_ahead_gives_the_same_tokens_as_waiting_for_every_step():
    rng = random.Random(3)
    reqs = [(f"r{i}", [rng.randrange(1, 100) for _ in range(rng.randrange(1, 60))], rng.randrange(1, 25))
            for i in range(14)]
    results = []
    for ahead in (False, True):
        s, ex, m = make_ahead(run_ahead=ahead, num_pages=40, budget=48)
        # tokens 7 and 42 end a request (the fake model hits them now and then)
        for rid, prompt, n in reqs:
            s.enqueue(pure(rid, prompt, n=n, eos_token_ids=(7, 42, 13, 77)))
        out, reasons = run_all(s)
        results.append((out, reasons))
        assert all(a.num_free == a.num_pages for a in m.allocators)
        if ahead:
            assert s.stats["steps_ahead"] > 0 and s.stats["tokens_dropped"] > 0
    assert results[0] == results[1]
    for rid, prompt, n in reqs:
        assert results[1][0].get(rid, []) == expected_output(prompt, n, eos=(7, 42, 13, 77))


def test_no_running_ahead_with_a_repetition_penalty_or_a_waiting_request():
    s, ex, m = make_ahead()
    s.enqueue(Request("a", list(range(1, 9)), SamplingParams.greedy(), max_new_tokens=6))     # penalty 1.05
    run_all(s)
    assert s.stats["steps_ahead"] == 0
    s, ex, m = make_ahead(max_seqs=1)
    s.enqueue(pure("a", range(1, 9), n=6))
    s.enqueue(pure("b", range(1, 5), n=3))       # waits for a's slot: a is never run ahead of
    out, _ = run_all(s)
    assert out["a"] == expected_output(range(1, 9), 6) and out["b"] == expected_output(range(1, 5), 3)
    assert "launch launch" not in " ".join(ex.log[:10])


def test_native_records_are_handed_back():
    """The decisions are made by the C++ core on integer records; when everything has drained
    neither side holds a record, and ids are used again."""
    s, ex, m = make(num_pages=12, budget=48, max_seqs=3)
    rng = random.Random(3)
    for round_ in range(3):
        for i in range(7):
            s.enqueue(req(f"r{round_}_{i}", [rng.randrange(1, 90) for _ in range(rng.randrange(1, 70))], n=rng.randrange(1, 9)))
        out, reasons = run_all(s)
        assert len(reasons) == 7 * (round_ + 1) or all(r[0] in ("length", "stop") for r in reasons.values())
        assert not s._runs and not s._ended and not m.requests
        assert s.running == [] and s.waiting == []
        m.check()
    assert s.stats["finished"] == 21
    sid = s._L.infero_sched_enqueue(s._h, 5, 1, 0)
    assert 0 <= sid < 8, "ids of finished requests are used again"


def test_a_small_window_pool_cuts_portions_and_never_blocks_admission():
    """The window group's pool is far smaller than the all-keys group's: prompts longer than it run in
    portions no longer than its free pages hold, admission looks at each group's own pool, and every
    request still gets its tokens; a request that cannot even fit the all-keys pool is refused."""
    W, P = 32, 16
    s, ex, m = make(num_pages=[48, 9], page_size=P, max_seqs=3, budget=96, ctx=1024,
                    groups=[GroupSpec(None), GroupSpec(W)])
    prompts = {"a": list(range(1, 201)), "b": list(range(3, 150)), "c": list(range(7, 60)), "d": list(range(2, 90))}
    for rid, p in prompts.items():
        s.enqueue(req(rid, p, n=12))
    s.enqueue(req("huge", range(48 * P + 5), n=2))
    out, reasons = run_all(s)
    for rid, p in prompts.items():
        assert out[rid] == expected_output(p, 12), rid
    assert reasons["huge"][0] == "error" and "pages" in reasons["huge"][1]
    portions = [n for b in ex.batches for (_, n, is_decode, _) in b if not is_decode]
    assert max(portions) <= 9 * P and any(n < 96 for n in portions)
    assert m.pages_reclaimed > 0
    assert [m.free_pages(g) for g in (0, 1)] == [48, 9] and not m.requests


def test_decode_attention_plan_covers_the_keys():
    """The one statement of how decode attention cuts its keys (native code; the parts and the native
    launcher of a block both call it): the splits cover the visible keys, a split has a multiple of 16
    keys and at least 256 unless there are fewer than that to see, there are at most 256 splits, and
    more multiprocessors never mean fewer splits."""
    from infero_b200.kernels.attention import plan_decode
    for n_tok, n_kv, group, vis in [(1, 4, 7, 4096), (8, 4, 7, 4096), (64, 4, 7, 4096), (1, 1, 1, 17), (3, 2, 2, 300),
                                    (1, 2, 7, 200000), (200, 8, 5, 32768), (1, 4, 7, 1)]:
        for sms in (0, 148, 64, 296):
            chunk, splits = plan_decode(n_tok, n_kv, group, vis, sms)
            assert chunk % 16 == 0 and 1 <= splits <= 256 and chunk * splits >= vis
            assert chunk >= 256 or splits == 256, (n_tok, vis, sms, chunk, splits)
            assert (splits - 1) * chunk < max(vis, 16), "a split with no keys"
        assert plan_decode(n_tok, n_kv, group, vis, 296)[1] >= plan_decode(n_tok, n_kv, group, vis, 64)[1]
    assert plan_decode(1, 4, 7, 4096, 148) == (256, 16)
    assert plan_decode(64, 4, 7, 4096, 148) == (4096, 1)
