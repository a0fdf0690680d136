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
penalty over a window longer than the device keeps (that would need the token on the host), nobody
waits for admission, and pages for one more
token each are free.  A request that ends at step k on an end-of-sequence token has then run
one token too far; that token is dropped.  (The reference's scheduler reads every step's tokens
before it plans the next, crates/server/src/scheduler.rs:1268-1429.)

The decisions themselves (admission, the plan of a step, the victim of a preemption, the end of a
request, whether to run ahead) are made in C++ (``csrc/host_sched.cpp``, in the engine's shared
library, no CUDA in it) on counters alone; this module keeps what belongs to Python (token lists,
samplers, events) and is that code's face.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass, field
from typing import Callable, Dict, Hashable, List, Optional, Tuple

from ..cache import CacheManager, RequestCache
from ..sampling import RowSampler, SamplingParams
from .step import FROM_DEVICE


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
    """A request from the moment it is queued (``rc`` is None while it waits)."""
    req: Request
    rc: Optional[RequestCache]
    sampler: RowSampler
    tokens: List[int]                      # everything that must be in the cache: prompt (+ generated on recompute)
    sid: int = -1                          # the native scheduler's name for it
    fed: int = 0                           # how many of ``tokens`` are in the cache
    generated: List[int] = field(default_factory=list)
    pending: Optional[int] = None          # sampled, not yet fed
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


def _lib():
    from ..kernels import lib
    L = lib()
    if not getattr(L, "_sched_api_ready", False):
        L.infero_sched_new.restype = ctypes.c_void_p
        L.infero_sched_stat.restype = ctypes.c_longlong
        L._sched_api_ready = True
    return L


_NATIVE_STATS = ("preemptions", "decode_tokens", "prefill_tokens", "rejected", "finished", "tokens_dropped")


class Scheduler:
    """``execute(items) -> tokens`` runs a planned batch and returns one sampled token per
    item with ``samples`` set, in order.  The engine supplies it; tests supply a fake."""

    def __init__(self, manager: CacheManager, execute: Callable[[List[PlanItem]], List[int]],
                 max_seqs: int, max_batch_tokens: int, ctx: int, max_prefill_chunk: Optional[int] = None,
                 launch: Optional[Callable[[List[PlanItem]], object]] = None, run_ahead: bool = True,
                 device_penalty_window: int = 0):
        self.manager = manager
        self.execute = execute
        self.launch = launch                   # like execute, but returns an object with .result()
        self.run_ahead = run_ahead and launch is not None
        # the longest repetition window whose penalty the launcher works out on the device (0: none);
        # a request with a longer one needs every token on the host before the next step
        self.device_penalty_window = device_penalty_window
        self._inflight: Optional[_InFlight] = None
        self.max_seqs = max_seqs
        self.max_batch_tokens = max_batch_tokens
        self.ctx = ctx
        self.max_prefill_chunk = max_prefill_chunk
        self._L = _lib()
        self._h = ctypes.c_void_p(self._L.infero_sched_new(manager._h, int(max_seqs), int(max_batch_tokens), int(ctx),
                                                           int(max_prefill_chunk or 0)))
        if not self._h:
            raise ValueError("bad scheduler limits")
        self._runs: Dict[int, Running] = {}          # by native id: waiting, running, or ended with a step still in flight
        self._ended: List[int] = []                  # ids to hand back once no step in flight names them
        self._buf = (ctypes.c_int * (5 * max(max_seqs, 1) * 2 + 16))()
        self._steps = 0
        self._steps_ahead = 0
        self._events: List[Event] = []

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._L.infero_sched_delete(h)

    # ---- views ------------------------------------------------------------------------------
    def _ids(self, fn) -> List[int]:
        cap = len(self._buf)
        n = fn(self._h, self._buf, cap)
        while n >= cap:                              # a long queue: ask again with room for all of it
            self._buf = (ctypes.c_int * (2 * cap))()
            cap = len(self._buf)
            n = fn(self._h, self._buf, cap)
        return [int(self._buf[i]) for i in range(n)]

    @property
    def running(self) -> List[Running]:
        return [self._runs[i] for i in self._ids(self._L.infero_sched_running)]

    @property
    def waiting(self) -> List[Running]:
        return [self._runs[i] for i in self._ids(self._L.infero_sched_waiting)]

    @property
    def stats(self) -> Dict[str, int]:
        out = {name: int(self._L.infero_sched_stat(self._h, i)) for i, name in enumerate(_NATIVE_STATS)}
        out["steps"] = self._steps
        out["steps_ahead"] = self._steps_ahead
        return out

    # ---- queue ------------------------------------------------------------------------------
    def enqueue(self, req: Request) -> None:
        p = req.params
        needs_host = (p.repetition_penalty != 1.0 and p.repetition_window > 0
                      and p.repetition_window > self.device_penalty_window)
        sid = self._L.infero_sched_enqueue(self._h, len(req.prompt), int(req.max_new_tokens), int(needs_host))
        if sid == -1:
            self._events.append(Event(req.rid, None, True, "error", "empty prompt"))
            return
        if sid == -2:
            self._events.append(Event(req.rid, None, True, "error",
                                      f"prompt of {len(req.prompt)} tokens does not fit the context of {self.ctx}"))
            return
        self._runs[sid] = Running(req=req, rc=None, sampler=RowSampler(req.params), tokens=list(req.prompt), sid=sid)

    def is_idle(self) -> bool:
        return (self._inflight is None and not self._events and self._L.infero_sched_num_waiting(self._h) == 0
                and self._L.infero_sched_num_running(self._h) == 0)

    def _release(self, sid: int) -> None:
        self._runs.pop(sid, None)
        self._L.infero_sched_release(self._h, sid)

    # ---- admission ----------------------------------------------------------------------------
    def _admit(self) -> None:
        while True:
            cap = len(self._buf) // 3
            n = self._L.infero_sched_admit(self._h, self._buf, cap)
            triples = [(int(self._buf[3 * i]), int(self._buf[3 * i + 1]), int(self._buf[3 * i + 2])) for i in range(n)]
            for sid, code, value in triples:
                run = self._runs[sid]
                if code == 0:
                    run.rc = self.manager.adopt(run.req.rid, value)
                    continue
                # can never fit, even alone
                run.finished = True
                self._events.append(Event(run.req.rid, None, True, "length" if code == 2 else "error",
                                          f"{len(run.tokens)} tokens need {value} pages, the pool has {self.manager.num_pages}"))
                self._release(sid)
            if n < cap:
                break

    # ---- planning -----------------------------------------------------------------------------
    def _plan(self) -> List[PlanItem]:
        n = self._L.infero_sched_plan(self._h, self._buf, len(self._buf) // 5)
        items: List[PlanItem] = []
        for i in range(n):
            sid, first, count, samples, is_decode = (int(self._buf[5 * i + k]) for k in range(5))
            run = self._runs[sid]
            if is_decode:
                items.append(PlanItem(run, [run.pending], samples=True, is_decode=True))
            else:
                items.append(PlanItem(run, run.tokens[first:first + count], samples=bool(samples), is_decode=False))
        return items

    def _preempt_youngest(self) -> bool:
        """Free the youngest running request and put it back at the front of the queue; what it
        generated so far becomes part of the prompt it recomputes."""
        sid = self._L.infero_sched_preempt_youngest(self._h)
        if sid < 0:
            return False
        victim = self._runs[sid]
        self.manager.forget(victim.req.rid)
        victim.rc = None
        victim.tokens = list(victim.req.prompt) + list(victim.generated)
        victim.pending = None          # it is the last of ``generated`` and is fed with the recompute
        victim.fed = 0
        victim.preemptions += 1
        return True

    # ---- one step -----------------------------------------------------------------------------
    def _start(self, items: List[PlanItem]) -> _InFlight:
        pending = self.launch(items) if self.launch is not None else _Done(self.execute(items))
        self._steps += 1
        return _InFlight(items, pending)

    def _can_run_ahead(self, cur: _InFlight) -> bool:
        """May the step after ``cur`` be launched before ``cur``'s tokens are known?"""
        if not self.run_ahead:
            return False
        n = len(cur.items)
        ids = (ctypes.c_int * max(1, n))(*[it.run.sid for it in cur.items])
        samples = (ctypes.c_int * max(1, n))(*[int(it.samples) for it in cur.items])
        return bool(self._L.infero_sched_can_run_ahead(self._h, n, ids, samples))

    def _complete(self, cur: _InFlight) -> List[Event]:
        """Wait for the step's tokens and advance its requests."""
        sampled = cur.pending.result()
        events: List[Event] = []
        k = 0
        for it in cur.items:
            run, req = it.run, it.run.req
            tok = None
            if it.samples:
                tok = int(sampled[k])
                k += 1
            is_eos = tok is not None and not req.ignore_eos and tok in req.eos_token_ids
            code = self._L.infero_sched_complete(self._h, run.sid, len(it.tokens), int(it.is_decode), int(it.samples),
                                                 int(is_eos))
            if code == 5:                          # ended a step earlier: this one ran a token too far
                continue
            if it.is_decode:
                run.pending = None
                run.tokens.append(it.tokens[0])
                run.fed += 1
            else:
                run.fed += len(it.tokens)
            if code == 0:
                continue
            if code == 1:
                run.generated.append(tok)
                run.pending = tok
                events.append(Event(req.rid, tok))
                continue
            # the request ended: on an end-of-sequence token (not appended), or with this token as its last
            self._ended_natively(run)
            if code == 2:
                events.append(Event(req.rid, None, True, "stop"))
            else:
                run.generated.append(tok)
                events.append(Event(req.rid, tok, True, "length", "context full" if code == 4 else None))
        return events

    def _ended_natively(self, run: Running) -> None:
        run.finished = True
        run.rc = None
        self.manager.forget(run.req.rid)
        self._ended.append(run.sid)

    def _hand_back_ended(self) -> None:
        """Ids of ended requests go back once no step in flight names them."""
        named = {it.run.sid for it in self._inflight.items} if self._inflight is not None else set()
        keep = []
        for sid in self._ended:
            if sid in named:
                keep.append(sid)
            else:
                self._release(sid)
        self._ended = keep

    def step(self) -> List[Event]:
        events, self._events = self._events, []
        if self._inflight is None:
            self._admit()
            events += self._events
            self._events = []
            if self._L.infero_sched_num_running(self._h) == 0:
                return events
            items = self._plan()
            while not items:
                if not self._preempt_youngest():
                    # a single request that cannot move: the cache is full for it
                    run = self.running[0]
                    events.append(self._finish(run, "length", "cache exhausted"))
                    self._hand_back_ended()
                    return events
                items = self._plan()
            self._inflight = self._start(items)
        cur = self._inflight
        ahead = None
        if self._can_run_ahead(cur):
            # every request decodes on: feed each the token ``cur`` is picking, from the device
            ahead = self._start([PlanItem(it.run, [FROM_DEVICE], samples=True, is_decode=True) for it in cur.items])
            self._steps_ahead += 1
        events += self._complete(cur)
        if ahead is not None:
            for it in ahead.items:                 # now the host knows what was fed
                if not it.run.finished:
                    it.tokens = [it.run.pending]
        self._inflight = ahead
        self._hand_back_ended()
        return events

    def drain(self) -> List[Event]:
        """Complete what is in flight (before aborting, or at the end)."""
        events: List[Event] = []
        while self._inflight is not None:
            cur, self._inflight = self._inflight, None
            events += self._complete(cur)
        self._hand_back_ended()
        return events

    def _finish(self, run: Running, reason: str, message: Optional[str] = None) -> Event:
        """End a request from outside the normal course (cache exhausted, a failed step)."""
        if not run.finished:
            self._L.infero_sched_finish(self._h, run.sid)
            self._ended_natively(run)
        return Event(run.req.rid, None, True, reason, message)

    def abort_all(self, message: str) -> List[Event]:
        """A failed step fails every running and waiting request (crates/server/src/scheduler.rs:2314-2322)."""
        events = []
        try:
            self.drain()
        except Exception:                           # noqa: BLE001  (the step that failed)
            self._inflight = None
        for run in self.running:
            events.append(self._finish(run, "error", message))
        while True:
            sid = self._L.infero_sched_pop_waiting(self._h)
            if sid < 0:
                break
            run = self._runs[sid]
            run.finished = True
            events.append(Event(run.req.rid, None, True, "error", message))
            self._release(sid)
        self._hand_back_ended()
        return events
