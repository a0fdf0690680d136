"""Continuous batching above the step function.

Every step: admit waiting requests, give each running request that has a token to feed one
decode token, hand the rest of the token budget to unfinished prompts in running order,
run the batch, sample, advance, retire.  The rules follow the reference's scheduler
(crates/server/src/scheduler.rs): FIFO admission while a request's prompt plus one token
fits the free cache and a sequence row is free, the head of the queue going back to the
front otherwise (:1854-1957); decodes first (:2076-2098); prompt portions under the token
budget, several prompts may share a step (:2105-2127); finish on an end-of-sequence token
(not appended, :2151-2153), on the generation budget or when the context is full
(:2170-2178); retire frees the cache (:2257-2275).

When pages run out.  The reference never preempts: a sequence that finds the pool empty ends
with reason "length", and a step in which nothing can move fails every request (:1042-1055).
Here the decision is: (1) admission reserves nothing but only admits what fits now; (2) a
step never plans more pages than are free; (3) if a decode token finds no page, the
youngest running request is preempted by recompute: its pages are freed and it returns
to the front of the queue with prompt + generated tokens as its new prompt (its sampler
state and output so far are kept); (4) a request that cannot proceed even alone (it
holds the whole pool) finishes with reason "length".

Running ahead.  With a ``launch`` function (steps that return before their tokens have reached the
host) the scheduler keeps one step in flight: while step k runs it launches step k+1 for the
same requests, feeding each the token step k is about to pick, which the sampler leaves on the
device.  It does so only when nothing can change the batch behind its back: every running
request is decoding, none reaches its length limit at step k, none samples with a repetition
penalty (that needs the token on the host), nobody waits for admission, and pages for one more
token each are free.  A request that ends at step k on an end-of-sequence token has then run
one token too far; that token is dropped.  (The reference's scheduler reads every step's tokens
before it plans the next, crates/server/src/scheduler.rs:1268-1429.)
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Callable, Deque, Dict, Hashable, List, Optional, Sequence, Tuple

from ..cache import CacheManager, OutOfPages, RequestCache
from ..sampling import RowSampler, SamplingParams
from .step import FROM_DEVICE, StepEntry


@dataclass
class Request:
    rid: Hashable
    prompt: List[int]
    params: SamplingParams
    max_new_tokens: int = 128
    eos_token_ids: Tuple[int, ...] = ()
    ignore_eos: bool = False


@dataclass
class Running:
    req: Request
    rc: RequestCache
    sampler: RowSampler
    tokens: List[int]                      # everything that must be in the cache: prompt (+ generated on recompute)
    fed: int = 0                           # how many of ``tokens`` are in the cache
    generated: List[int] = field(default_factory=list)
    pending: Optional[int] = None          # sampled, not yet fed
    admitted_at: int = 0
    preemptions: int = 0
    finished: bool = False


@dataclass
class Event:
    rid: Hashable
    token: Optional[int]                   # newly generated token, if any
    finished: bool = False
    reason: Optional[str] = None           # "stop" | "length" | "error"
    message: Optional[str] = None


@dataclass
class PlanItem:
    run: Running
    tokens: List[int]
    samples: bool                          # the last token's logits are sampled
    is_decode: bool


class _Done:
    """Tokens that are already here (a synchronous ``execute``)."""

    def __init__(self, tokens):
        self._tokens = list(tokens)

    def result(self):
        return self._tokens


@dataclass
class _InFlight:
    items: List[PlanItem]
    pending: object                        # .result() -> one token per sampling item


class Scheduler:
    """``execute(items) -> tokens`` runs a planned batch and returns one sampled token per
    item with ``samples`` set, in order.  The engine supplies it; tests supply a fake."""

    def __init__(self, manager: CacheManager, execute: Callable[[List[PlanItem]], List[int]],
                 max_seqs: int, max_batch_tokens: int, ctx: int, max_prefill_chunk: Optional[int] = None,
                 launch: Optional[Callable[[List[PlanItem]], object]] = None, run_ahead: bool = True):
        self.manager = manager
        self.execute = execute
        self.launch = launch                   # like execute, but returns an object with .result()
        self.run_ahead = run_ahead and launch is not None
        self._inflight: Optional[_InFlight] = None
        self.max_seqs = max_seqs
        self.max_batch_tokens = max_batch_tokens
        self.ctx = ctx
        self.max_prefill_chunk = max_prefill_chunk
        self.waiting: Deque[Running | Request] = deque()
        self.running: List[Running] = []
        self.clock = 0
        self.stats = {"steps": 0, "preemptions": 0, "decode_tokens": 0, "prefill_tokens": 0,
                      "rejected": 0, "finished": 0, "steps_ahead": 0, "tokens_dropped": 0}
        self._events: List[Event] = []

    # ---- queue ------------------------------------------------------------------------------
    def enqueue(self, req: Request) -> None:
        if not req.prompt:
            self._events.append(Event(req.rid, None, True, "error", "empty prompt"))
            self.stats["rejected"] += 1
            return
        if len(req.prompt) + 1 > self.ctx:
            self._events.append(Event(req.rid, None, True, "error",
                                      f"prompt of {len(req.prompt)} tokens does not fit the context of {self.ctx}"))
            self.stats["rejected"] += 1
            return
        self.waiting.append(req)

    def is_idle(self) -> bool:
        return not self.waiting and not self.running and not self._events and self._inflight is None

    # ---- admission ----------------------------------------------------------------------------
    def _pages_for(self, n_tokens: int) -> int:
        return -(-n_tokens // self.manager.page_size)

    def _outstanding_pages(self) -> int:
        """Pages the running requests still have to take to hold their prompt plus one token."""
        return sum(max(0, self._pages_for(len(r.tokens) + 1) - max((r.rc.table_len(g) for g in range(len(self.manager.groups))), default=0))
                   for r in self.running)

    def _admit(self) -> None:
        committed = 0
        while self.waiting and len(self.running) < self.max_seqs:
            head = self.waiting[0]
            tokens = head.tokens if isinstance(head, Running) else head.prompt
            need = self._pages_for(len(tokens) + 1)
            if need > self.manager.num_pages:
                # can never fit, even alone
                self.waiting.popleft()
                resumed = isinstance(head, Running)
                rid = head.req.rid if resumed else head.rid
                self._events.append(Event(rid, None, True, "length" if resumed else "error",
                                          f"{len(tokens)} tokens need {need} pages, the pool has {self.manager.num_pages}"))
                self.stats["rejected"] += 1
                continue
            if need > self.manager.min_free_pages() - self._outstanding_pages():
                break                                   # stays at the front; tried again next step
            self.waiting.popleft()
            if isinstance(head, Running):
                run = head
                run.rc = self.manager.open(run.req.rid)
            else:
                run = Running(req=head, rc=self.manager.open(head.rid), sampler=RowSampler(head.params),
                              tokens=list(head.prompt))
            run.admitted_at = self.clock
            self.clock += 1
            self.running.append(run)

    # ---- planning -----------------------------------------------------------------------------
    def _plan(self) -> List[PlanItem]:
        budget = self.max_batch_tokens
        items: List[PlanItem] = []
        n_groups = len(self.manager.groups)
        used = [0] * n_groups                      # pages this plan takes, per group
        P = self.manager.page_size

        def free(g: int) -> int:
            return self.manager.free_pages(g) - used[g]

        # decodes first
        for run in self.running:
            if run.pending is None or run.fed < len(run.tokens) or budget <= 0:
                continue
            need = self.manager.pages_needed(run.rc, 1)
            if any(need[g] > free(g) for g in range(n_groups)):
                continue
            for g in range(n_groups):
                used[g] += need[g]
            items.append(PlanItem(run, [run.pending], samples=True, is_decode=True))
            budget -= 1
        # then prompt portions, in running order
        for run in self.running:
            if budget <= 0:
                break
            remaining = len(run.tokens) - run.fed
            if remaining <= 0:
                continue
            slack = (-(run.rc.length + run.rc.reserved)) % P       # free rows in its last page
            room = slack + max(0, min((free(g) for g in range(n_groups)), default=0)) * P
            n = min(remaining, budget, room)
            if self.max_prefill_chunk:
                n = min(n, self.max_prefill_chunk)
            if n <= 0:
                continue
            need = self.manager.pages_needed(run.rc, n)
            for g in range(n_groups):
                used[g] += need[g]
            items.append(PlanItem(run, run.tokens[run.fed:run.fed + n], samples=(n == remaining), is_decode=False))
            budget -= n
        return items

    def _preempt_youngest(self) -> bool:
        """Free the youngest running request and put it back at the front of the queue; what it
        generated so far becomes part of the prompt it recomputes."""
        if len(self.running) <= 1:
            return False
        victim = max(self.running, key=lambda r: r.admitted_at)
        self.running.remove(victim)
        self.manager.close(victim.req.rid)
        victim.tokens = list(victim.req.prompt) + list(victim.generated)
        victim.pending = None          # it is the last of ``generated`` and is fed with the recompute
        victim.fed = 0
        victim.preemptions += 1
        self.stats["preemptions"] += 1
        self.waiting.appendleft(victim)
        return True

    # ---- one step -----------------------------------------------------------------------------
    def _start(self, items: List[PlanItem]) -> _InFlight:
        pending = self.launch(items) if self.launch is not None else _Done(self.execute(items))
        self.stats["steps"] += 1
        return _InFlight(items, pending)

    def _can_run_ahead(self, cur: _InFlight) -> bool:
        """May the step after ``cur`` be launched before ``cur``'s tokens are known?"""
        if not self.run_ahead or self.waiting or len(cur.items) != len(self.running):
            return False
        for it in cur.items:
            run, req = it.run, it.run.req
            if not it.samples or run.finished:
                return False                                   # a prompt is still being fed
            if req.params.repetition_penalty != 1.0:
                return False                                   # the penalty needs the token on the host
            if len(run.generated) + 2 > req.max_new_tokens or len(req.prompt) + len(run.generated) + 2 > self.ctx:
                return False                                   # it ends at ``cur`` or at the step after
        n_groups = len(self.manager.groups)
        used = [0] * n_groups
        for it in cur.items:
            need = self.manager.pages_needed(it.run.rc, 1)
            for g in range(n_groups):
                used[g] += need[g]
        return all(used[g] <= self.manager.free_pages(g) for g in range(n_groups)) \
            and len(cur.items) <= self.max_batch_tokens

    def _complete(self, cur: _InFlight) -> List[Event]:
        """Wait for the step's tokens and advance its requests."""
        sampled = cur.pending.result()
        events: List[Event] = []
        k = 0
        for it in cur.items:
            run = it.run
            tok = None
            if it.samples:
                tok = int(sampled[k])
                k += 1
            if run.finished:                       # ended a step earlier: this one ran a token too far
                self.stats["tokens_dropped"] += 1
                continue
            if it.is_decode:
                run.pending = None
                run.tokens.append(it.tokens[0])
                run.fed += 1
                self.stats["decode_tokens"] += 1
            else:
                run.fed += len(it.tokens)
                self.stats["prefill_tokens"] += len(it.tokens)
            if it.samples:
                ev = self._advance(run, tok)
                if ev is not None:
                    events.append(ev)
        return events

    def step(self) -> List[Event]:
        events, self._events = self._events, []
        if self._inflight is None:
            self._admit()
            events += self._events
            self._events = []
            if not self.running:
                return events
            items = self._plan()
            while not items:
                if not self._preempt_youngest():
                    # a single request that cannot move: the cache is full for it
                    run = self.running[0]
                    events.append(self._finish(run, "length", "cache exhausted"))
                    return events
                items = self._plan()
            self._inflight = self._start(items)
        cur = self._inflight
        ahead = None
        if self._can_run_ahead(cur):
            # every request decodes on: feed each the token ``cur`` is picking, from the device
            ahead = self._start([PlanItem(it.run, [FROM_DEVICE], samples=True, is_decode=True) for it in cur.items])
            self.stats["steps_ahead"] += 1
        events += self._complete(cur)
        if ahead is not None:
            for it in ahead.items:                 # now the host knows what was fed
                if not it.run.finished:
                    it.tokens = [it.run.pending]
        self._inflight = ahead
        return events

    def drain(self) -> List[Event]:
        """Complete what is in flight (before aborting, or at the end)."""
        events: List[Event] = []
        while self._inflight is not None:
            cur, self._inflight = self._inflight, None
            events += self._complete(cur)
        return events

    def _advance(self, run: Running, tok: int) -> Optional[Event]:
        req = run.req
        if not req.ignore_eos and tok in req.eos_token_ids:
            return self._finish(run, "stop")                 # the end token is not appended
        run.generated.append(tok)
        if len(run.generated) >= req.max_new_tokens:
            ev = self._finish(run, "length")
            ev.token = tok
            return ev
        if len(req.prompt) + len(run.generated) >= self.ctx:
            ev = self._finish(run, "length", "context full")
            ev.token = tok
            return ev
        run.pending = tok
        return Event(req.rid, tok)

    def _finish(self, run: Running, reason: str, message: Optional[str] = None) -> Event:
        run.finished = True
        if run in self.running:
            self.running.remove(run)
        if run.req.rid in self.manager.requests:
            self.manager.close(run.req.rid)
        self.stats["finished"] += 1
        return Event(run.req.rid, None, True, reason, message)

    def abort_all(self, message: str) -> List[Event]:
        """A failed step fails every running and waiting request (crates/server/src/scheduler.rs:2314-2322)."""
        events = []
        try:
            self.drain()
        except Exception:                           # noqa: BLE001  (the step that failed)
            self._inflight = None
        for run in list(self.running):
            events.append(self._finish(run, "error", message))
        while self.waiting:
            w = self.waiting.popleft()
            rid = w.req.rid if isinstance(w, Running) else w.rid
            events.append(Event(rid, None, True, "error", message))
        return events
