"""The step function: run one batch of (request, its next tokens) from the cache.

A step holds any mix of prompt portions and single decoded tokens, cut anywhere; it runs
only the tokens it is given, as one flat batch, against what earlier steps left in the
cache, and returns 32-bit logits at the wanted places.  The reference's counterpart is
``forward_batch_rows`` (crates/model/src/lib.rs:3423-4243): same flat layout
(token_ids, seq_of, positions; :3483-3557), same constraints (a sequence at most once,
:3464-3475; a token budget, :3445-3449), but logits only for the last rows of an item,
where this step takes arbitrary positions.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Hashable, List, Optional, Sequence

import ctypes

import numpy as np
import torch

from .. import kernels as K
from ..cache import CacheManager, CacheStorage, OutOfPages, RequestCache, plan_group_pages
from ..cache.storage import group_cache_slots
from ..config.engine_config import EngineConfig
from ..models.decoder import DecoderModel


# As a token of a single-token entry: "the token the sampler picked for this request in the
# step before, which is still on the device" (``ModelRunner.device_tokens[slot]``).
FROM_DEVICE = -1


class StepError(ValueError):
    """A batch the step function refuses (nothing was run, nothing was reserved)."""


@dataclass
class StepEntry:
    rid: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()


class StepContext:
    """What the parts see of a step."""

    def __init__(self, runner: "ModelRunner"):
        self._runner = runner
        self.act_dtype: torch.dtype = runner.act_dtype
        self.device = runner.device
        self.n_tokens = 0
        self.n_entries = 0
        # device int32
        self.token_ids: torch.Tensor = None
        self.positions: torch.Tensor = None
        self.tok_entry: torch.Tensor = None
        self.entry_q_start: torch.Tensor = None
        self.entry_q_len: torch.Tensor = None
        self.entry_pos0: torch.Tensor = None
        self.entry_slot: torch.Tensor = None
        self._tables: List[torch.Tensor] = []
        # host copies
        self.h_q_start: np.ndarray = None
        self.h_q_len: np.ndarray = None
        self.h_pos0: np.ndarray = None
        self.h_slot: np.ndarray = None
        self.decode_only = False
        self.max_q_len = 0
        self.max_kv_len = 0
        self.kv_bound: Optional[int] = None     # plan decode attention for this many keys (captured steps)
        self.device_tokens: torch.Tensor = runner.device_tokens
        self._empty_f32 = None
        # the native block launcher's view of the step (made at the first layer that uses it)
        self._native_step = None
        self.native_parity = 0
        self.native_arena: Optional[torch.Tensor] = None

    def kv_cache(self, slot: int):
        return self._runner.storage.layer_kv(slot)

    def state(self, slot: int) -> torch.Tensor:
        """[max_requests, *shape]; row ``entry_slot[e]`` belongs to entry e."""
        return self._runner.storage.state(slot)

    def block_table(self, group: int) -> torch.Tensor:
        return self._tables[group]

    def native_step(self, x: torch.Tensor, block_desc):
        """The step as ``infero_block_forward`` takes it (see parts/native_block.py); None when this
        step cannot go that way."""
        from ..kernels import attention as A
        from ..kernels import tc_gemm
        from ..parts import native_block as NB
        r = self._runner
        arena = r.native_arena(block_desc)
        if arena is None or self.h_q_len is None:
            return None
        st = self._native_step
        if st is None:
            n_dec, vis_now, tiles_128, _ = A._batch_shape(self)
            vis = vis_now if self.kv_bound is None else int(self.kv_bound)
            counters = A._arrival_counters(self.device)
            ptr = lambda t: t.data_ptr()                       # noqa: E731
            st = NB._Step(self.n_tokens, self.n_entries, n_dec, vis, tiles_128, tc_gemm.sm_count(self.device),
                          ptr(self.positions), ptr(self.tok_entry), ptr(self.entry_q_start), ptr(self.entry_q_len),
                          ptr(self.entry_pos0), ptr(x), ptr(arena), arena.numel(), ptr(counters), A.N_COUNTERS,
                          K._stream().value)
            self._native_step = st
            self._native_keep = (x, counters)
        elif st.arena != arena.data_ptr():
            st.arena, st.arena_bytes = arena.data_ptr(), arena.numel()
        self.native_arena = arena
        return st

    def zero_inv_freq(self, device) -> torch.Tensor:
        if self._empty_f32 is None:
            self._empty_f32 = torch.empty(0, dtype=torch.float32, device=device)
        return self._empty_f32


class ModelRunner:
    """Owns the cache (bookkeeping + device arrays) and runs steps of one model."""

    def __init__(self, model: DecoderModel, cfg: EngineConfig, device=None):
        self.model = model
        self.cfg = cfg
        self.device = torch.device(device or cfg.device)
        self.act_dtype = torch.bfloat16 if cfg.dtype == "bfloat16" else torch.float32
        self.page_size = cfg.page_size
        self.num_pages = cfg.resolved_num_pages()
        self.max_blocks = max(1, -(-cfg.ctx // cfg.page_size))
        # Every group of cache slots has a pool of its own: cfg.num_pages where every key is kept, what
        # max_seqs requests under the step's token budget can ever hold where only a window is.
        # One page (in every group) and one state slot beyond what the manager hands out: where the
        # entries that pad a captured step to its captured size read and write.
        groups, _ = group_cache_slots(model.kv_specs)
        self.pages_per_group = plan_group_pages(groups, self.num_pages, cfg.page_size, cfg.max_seqs,
                                                int(cfg.max_batch_tokens))
        self.pad_slot = cfg.max_seqs
        self.storage = CacheStorage(model.kv_specs, model.state_specs, [n + 1 for n in self.pages_per_group],
                                    cfg.page_size, cfg.max_seqs + 1, self.act_dtype, self.device)
        self.manager = CacheManager(self.storage.bookkeeping_groups(), self.pages_per_group, cfg.page_size,
                                    cfg.max_seqs, max_blocks=self.max_blocks)
        # the sampler's last pick per request slot, for steps launched before the host has read it
        self.device_tokens = torch.zeros(max(1, cfg.max_seqs), dtype=torch.int32, device=self.device)
        # the requests' generated tokens, per slot, for a repetition penalty worked out on the device:
        # the n-th token of a request sits at history[slot, n % HISTORY_WIDTH]
        self.history = torch.zeros((max(1, cfg.max_seqs), self.HISTORY_WIDTH), dtype=torch.int32, device=self.device)
        self.history_len = torch.zeros(max(1, cfg.max_seqs), dtype=torch.int32, device=self.device)
        self.steps_run = 0
        self.tokens_run = 0
        # captured decode steps: (entries, key bound) -> _DecodeGraph; a shape is run eagerly the
        # first time it is seen, captured the second time and replayed from then on (the
        # reference does the same per (pool, tokens, kv bucket), crates/model/src/lib.rs:3887-3981)
        self._graphs: Dict[tuple, "_DecodeGraph"] = {}
        self._arena: Optional[torch.Tensor] = None         # scratch of the native block launcher
        self._old_arenas: List[torch.Tensor] = []
        self._arena_need: Dict[tuple, int] = {}
        self._graph_seen: Dict[tuple, int] = {}
        self.graph_replays = 0
        self.graph_captures = 0
        self.last_h2d_bytes = 0

    # ---- requests --------------------------------------------------------------------------
    def open(self, rid: Hashable) -> RequestCache:
        return self.manager.open(rid)

    def close(self, rid: Hashable) -> None:
        self.manager.close(rid)

    def length(self, rid: Hashable) -> int:
        return self.manager.get(rid).length

    def truncate(self, rid: Hashable, length: int) -> None:
        """Cut a request back to its first ``length`` tokens; the next step appends from there."""
        self.manager.truncate(self.manager.get(rid), length)

    # ---- the step ----------------------------------------------------------------------------
    def _validate(self, entries: Sequence[StepEntry]) -> List[RequestCache]:
        if not entries:
            raise StepError("a step needs at least one entry")
        seen = set()
        rcs = []
        total = 0
        rows = 0
        vocab = self.model.spec.vocab_size
        for e in entries:
            if e.rid in seen:
                raise StepError(f"request {e.rid!r} appears twice in one step")
            seen.add(e.rid)
            if e.rid not in self.manager.requests:
                raise StepError(f"request {e.rid!r} is not open")
            n = len(e.tokens)
            if n == 0:
                raise StepError(f"request {e.rid!r} brings no tokens")
            rc = self.manager.get(e.rid)
            if rc.length + n > self.cfg.ctx:
                raise StepError(f"request {e.rid!r} would reach {rc.length + n} tokens, context is {self.cfg.ctx}")
            if len(e.want) and not (0 <= min(e.want) and max(e.want) < n):
                raise StepError(f"request {e.rid!r}: wanted places {list(e.want)} outside its {n} tokens")
            lo, hi = (e.tokens[0], e.tokens[0]) if n == 1 else (min(e.tokens), max(e.tokens))
            if not (0 <= lo and hi < vocab) and not (n == 1 and int(lo) == FROM_DEVICE):
                bad = next(t for t in e.tokens if not 0 <= int(t) < vocab)
                raise StepError(f"request {e.rid!r}: token id {bad} outside the vocabulary of {vocab}")
            total += n
            rows += len(e.want)
            rcs.append(rc)
        if total > self.cfg.max_batch_tokens:
            raise StepError(f"step of {total} tokens exceeds the budget of {self.cfg.max_batch_tokens}")
        if rows > self.cfg.max_logit_rows:
            raise StepError(f"step wants {rows} rows of logits, at most {self.cfg.max_logit_rows}")
        return rcs

    def step(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """Run the batch; returns float32 logits [rows wanted, vocab] on the device, in the
        order of the entries and of each entry's ``want`` (None if nothing is wanted).  A captured
        decode step returns its graph's own output tensor: use or copy it before the next step.
        Raises OutOfPages (nothing reserved, nothing run) when the cache cannot hold it."""
        rcs = self._validate(entries)
        done: List[RequestCache] = []
        try:
            for rc, e in zip(rcs, entries):
                self.manager.reserve(rc, len(e.tokens))
                done.append(rc)
        except OutOfPages:
            for rc in done:
                self.manager.abort_reservation(rc)
            raise
        try:
            for rc in rcs:
                if rc.fresh and self.storage.states:
                    self.storage.zero_state(rc.slot)
            logits = None
            key = self._graph_key(entries, rcs)
            if key is not None:
                logits = self._graph_step(key, entries, rcs)
            if key is None or logits is None:
                ctx, rows = self._build_context(entries, rcs)
                with K.stream_scope():
                    logits = self.model.forward(ctx, ctx.token_ids, rows)
                n_tokens = ctx.n_tokens
            else:
                n_tokens = len(entries)
        except Exception:
            for rc in rcs:
                self.manager.abort_reservation(rc)
            raise
        for rc, e in zip(rcs, entries):
            self.manager.commit(rc, len(e.tokens))
        self.steps_run += 1
        self.tokens_run += n_tokens
        return logits

    # ---- scratch of the native block launcher -----------------------------------------------------
    def native_arena(self, block_desc) -> Optional[torch.Tensor]:
        """Device scratch large enough for any step of this runner through the given block
        (``infero_block_arena_bytes``).  It only ever grows; captured graphs keep the arenas they
        were captured with alive."""
        from ..kernels import tc_gemm
        from ..parts import native_block as NB
        d = block_desc                       # (the need depends on the block's sizes, not on which block it is)
        key = (d.hidden, d.n_heads, d.n_kv, d.head_dim, d.intermediate, tc_gemm._plan_epoch[0])
        need = self._arena_need.get(key)
        if need is None:
            # (a captured step may be padded past max_batch_tokens, up to the largest captured size)
            need = int(NB._lib().infero_block_arena_bytes(ctypes.byref(block_desc), max(int(self.cfg.max_batch_tokens), self.MAX_GRAPH_ENTRIES),
                                                          tc_gemm.sm_count(self.device)))
            self._arena_need[key] = need
        if self._arena is None or self._arena.numel() < need:
            if self._arena is not None:
                self._old_arenas.append(self._arena)
            self._arena = torch.empty(need, dtype=torch.uint8, device=self.device)
        return self._arena

    # ---- device inputs of a step ---------------------------------------------------------------
    def _layout_args(self, entries: Sequence[StepEntry], rcs: Sequence[RequestCache], pad: int = 0):
        """What the C++ layout builder takes: per entry slot, token count and wanted count, the
        flat token ids and wanted places, and the number of ints the step's arrays need (with
        ``pad`` single-token entries of no request behind the real ones)."""
        E = len(entries)
        slots = np.fromiter((rc.slot for rc in rcs), dtype=np.int32, count=E)
        lens = np.fromiter((len(e.tokens) for e in entries), dtype=np.int32, count=E)
        T = int(lens.sum())
        if T == E:
            tokens = np.fromiter((e.tokens[0] for e in entries), dtype=np.int32, count=E)
        else:
            tokens = np.concatenate([np.asarray(e.tokens, dtype=np.int32) for e in entries])
        want_counts = np.fromiter((len(e.want) for e in entries), dtype=np.int32, count=E)
        R = int(want_counts.sum())
        if R == E and T == E:
            wants = np.zeros(E, dtype=np.int32)
        elif R:
            wants = np.concatenate([np.asarray(e.want, dtype=np.int32) for e in entries if len(e.want)])
        else:
            wants = np.zeros(1, dtype=np.int32)
        total = 3 * (T + pad) + 4 * (E + pad) + R + pad + len(self.manager.groups) * max(1, E + pad) * self.max_blocks
        return (slots, lens, tokens, want_counts, wants), total, T + pad

    def _fill(self, args, out: np.ndarray, pad: int = 0):
        """Lay the step's arrays out in ``out`` (pinned host memory); returns the section sizes and
        host copies of the per-entry arrays."""
        sizes = self.manager.step_layout(*args, self.max_blocks, out, pad, self.pad_slot)
        T, E = sizes[0], sizes[3]
        o = 3 * T
        host = tuple(out[o + k * E:o + (k + 1) * E].copy() for k in range(4))    # first row, rows, cached length, slot
        return sizes, host

    def _context_from(self, dev: torch.Tensor, sizes: Sequence[int], host, E: int, T: int):
        views = []
        off = 0
        for n in sizes:
            views.append(dev[off:off + n])
            off += n
        q_start, lens, pos0, slots = host
        ctx = StepContext(self)
        ctx.n_tokens, ctx.n_entries = T, E
        (ctx.token_ids, ctx.positions, ctx.tok_entry, ctx.entry_q_start, ctx.entry_q_len, ctx.entry_pos0,
         ctx.entry_slot, d_rows) = views[:8]
        ctx._tables = [views[8 + g].view(E, self.max_blocks) for g in range(len(self.manager.groups))]
        ctx.h_q_start, ctx.h_q_len, ctx.h_pos0, ctx.h_slot = q_start, lens, pos0, slots
        ctx.decode_only = bool((lens == 1).all())
        ctx.max_q_len = int(lens.max())
        ctx.max_kv_len = int((pos0 + lens).max())
        return ctx, (d_rows if sizes[7] else None)

    def _build_context(self, entries: Sequence[StepEntry], rcs: Sequence[RequestCache]):
        args, total, T = self._layout_args(entries, rcs)
        # one pinned staging buffer, one host-to-device copy
        staging = torch.empty(total, dtype=torch.int32, pin_memory=(self.device.type == "cuda"))
        sizes, host = self._fill(args, staging.numpy())
        dev = staging.to(self.device, non_blocking=True)
        self.last_h2d_bytes = staging.numel() * 4
        ctx, rows = self._context_from(dev, sizes, host, len(entries), T)
        ctx._staging = staging          # keep the pinned buffer alive until the copy has run
        return ctx, rows

    # ---- captured decode steps -------------------------------------------------------------------
    def _graph_key(self, entries: Sequence[StepEntry], rcs: Sequence[RequestCache]):
        """(entries, key bound) if this step can run as a captured graph: single tokens only,
        each wanting its own logits.  The bound is the smallest 256 * 2^k that holds every
        request's keys, so a graph serves a request while it grows to twice its length."""
        if not self.cfg.cuda_graphs or self.device.type != "cuda" or len(entries) > self.MAX_GRAPH_ENTRIES:
            return None
        for e in entries:
            if len(e.tokens) != 1 or len(e.want) != 1 or int(e.want[0]) != 0:
                return None
        need = max(rc.length for rc in rcs) + 1
        bound = 256
        while bound < need:
            bound *= 2
        return (self._graph_size(len(entries)), min(bound, self.max_blocks * self.page_size))

    HISTORY_WIDTH = 1024          # the longest repetition window the device-side penalty covers

    def reset_history(self, slot: int, generated: Sequence[int]) -> None:
        """A request starts (or starts again after a preemption) in ``slot``: its history on the
        device becomes what it has generated so far."""
        n = len(generated)
        self.history_len[slot] = n
        if n:
            W = self.HISTORY_WIDTH
            tail = list(generated[-W:])
            first = n - len(tail)
            idx = torch.tensor([(first + i) % W for i in range(len(tail))], dtype=torch.long, device=self.device)
            self.history[slot].index_copy_(0, idx, torch.tensor(tail, dtype=torch.int32, device=self.device))

    MAX_GRAPH_ENTRIES = 256
    GRAPH_SIZES = (1, 2, 3, 4, 6, 8, 12, 16, 24, 32, 48, 64, 96, 128, 192, 256)

    def _graph_size(self, n: int) -> int:
        """A step of n single tokens runs as the captured step of the next size in GRAPH_SIZES, the
        difference made up by entries of no request (so that a batch that shrinks request by
        request does not capture a graph at every size), unless its logits would not fit."""
        for size in self.GRAPH_SIZES:
            if size >= n:
                return size if size <= self.cfg.max_logit_rows else n
        return n

    def _graph_step(self, key, entries, rcs) -> Optional[torch.Tensor]:
        seen = self._graph_seen.get(key, 0)
        self._graph_seen[key] = seen + 1
        g = self._graphs.get(key)
        if g is None:
            if seen == 0:
                return None          # first sight runs eagerly: it warms what is set up lazily
            g = _DecodeGraph(self, key, entries, rcs)
            self._graphs[key] = g
            self.graph_captures += 1
        g.load(entries, rcs)
        g.graph.replay()
        self.graph_replays += 1
        return g.logits[:len(entries)]

    def drop_graphs(self) -> None:
        self._graphs.clear()
        self._graph_seen.clear()


class _DecodeGraph:
    """One captured decode step.  Its inputs live in a device buffer of fixed address that is
    refilled from pinned host memory before every replay; two staging buffers alternate so
    that the host never writes one whose copy may still be in flight."""

    def __init__(self, runner: ModelRunner, key, entries, rcs):
        self.runner = runner
        E, bound = key                    # E: the captured size, len(entries) or the next size above it
        self.size = E
        args, n, _ = runner._layout_args(entries, rcs, E - len(entries))
        self.dev = torch.zeros(n, dtype=torch.int32, device=runner.device)
        self.staging = [torch.empty(n, dtype=torch.int32, pin_memory=True) for _ in range(2)]
        self.copied = [None, None]
        self.turn = 0
        self.sizes, host = self.load(entries, rcs, args)
        ctx, rows = runner._context_from(self.dev, self.sizes, host, E, E)
        ctx.kv_bound = bound
        ctx.max_kv_len = bound
        self.ctx = ctx
        torch.cuda.current_stream(runner.device).synchronize()
        from .. import kernels as K
        import gc
        before = K.launch_count()
        self.graph = torch.cuda.CUDAGraph()
        # No garbage collection while the stream is capturing: an old CUDA graph that is freed in
        # the middle of a capture (runners sit in reference cycles, so they go when the collector
        # gets to them) invalidates the capture.  The collector is held off meanwhile (a full
        # collection first would cost more than the capture itself).
        was_enabled = gc.isenabled()
        gc.disable()
        try:
            with torch.cuda.graph(self.graph):
                with K.stream_scope():
                    self.logits = runner.model.forward(ctx, ctx.token_ids, rows)
        finally:
            if was_enabled:
                gc.enable()
        self.n_kernels = K.launch_count() - before

    def load(self, entries, rcs, args=None):
        pad = self.size - len(entries)
        if args is None:
            args, _, _ = self.runner._layout_args(entries, rcs, pad)
        i = self.turn
        self.turn ^= 1
        if self.copied[i] is not None:
            self.copied[i].synchronize()
        filled = self.runner._fill(args, self.staging[i].numpy(), pad)
        self.dev.copy_(self.staging[i], non_blocking=True)
        self.runner.last_h2d_bytes = self.dev.numel() * 4
        ev = torch.cuda.Event()
        ev.record()
        self.copied[i] = ev
        return filled
