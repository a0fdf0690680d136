"""The Python entry point: load a model, queue requests, step, generate.

In the manner of the reference's library use (crates/model/examples/generate.rs:77-145:
load, new session, forward, sample) and of its server engine (crates/server/src/engine.rs:
submit -> events).  Option names follow its CLI where it has them: ``ctx``, ``max_seqs``,
``kv_slots``, ``gpu_memory_fraction`` (crates/server/src/main.rs:13-135).
"""
from __future__ import annotations

import itertools
from typing import Any, Dict, Hashable, List, Optional, Sequence

import torch

from ..config.engine_config import EngineConfig
from ..sampling import ReadyTokens, SamplingParams, sample_rows_async
from .scheduler import Event, PlanItem, Request, Scheduler
from .step import ModelRunner, StepEntry


def _auto_pages(model, page_size: int, act_dtype, device, max_seqs: int, ctx: int,
                fraction: Optional[float], max_batch_tokens: int) -> int:
    """Pages (of the groups that keep every key) that fit beside the weights: the reference leaves 1/8
    of the card plus 512 MiB free (crates/server/src/scheduler.rs:2341-2432); never more than max_seqs
    full contexts.  A group that keeps a window has a pool of fixed size, which comes off the room first."""
    from ..cache.storage import window_pool_pages
    esize = 2 if act_dtype == torch.bfloat16 else 4
    want = max_seqs * (-(-ctx // page_size))
    per_token, fixed = 0, 0
    for s in model.kv_specs.values():
        b = s.num_kv_heads * (s.head_dim + s.value_dim) * esize
        if s.window and window_pool_pages(s.window, page_size, max_seqs, max_batch_tokens) < want:
            fixed += b * page_size * (window_pool_pages(s.window, page_size, max_seqs, max_batch_tokens) + 1)
        else:
            per_token += b
    if per_token == 0:
        return max(1, want)
    free, total = torch.cuda.mem_get_info(device)
    if fraction is not None:
        room = int(total * fraction) - (total - free)
    else:
        room = free - total // 8 - (512 << 20)
    fit = max(1, (room - fixed) // (per_token * page_size))
    return int(max(1, min(want, fit)))


class Engine:
    def __init__(self, model_dir: Optional[str] = None, *, config: Optional[Dict[str, Any]] = None,
                 seed: int = 0, dtype: str = "bfloat16", ctx: int = 4096, max_seqs: int = 32,
                 kv_slots: Optional[int] = None, gpu_memory_fraction: Optional[float] = None,
                 max_batch_tokens: int = 2048, page_size: int = 16, device: str = "cuda:0",
                 cuda_graphs: bool = True, max_prefill_chunk: Optional[int] = None,
                 generate_on_device: bool = False, model=None, run_ahead: bool = True):
        from .. import kernels
        from ..loading import load_model, random_model
        if not torch.cuda.is_available():
            raise RuntimeError("no CUDA device is visible; this engine has no CPU path")
        kernels.lib()
        if model is not None:
            self.model, self.model_config = model, None
        elif model_dir is not None:
            self.model, self.model_config = load_model(model_dir, dtype, device)
        elif config is not None:
            self.model, self.model_config = random_model(config, seed, dtype, device,
                                                         generate_on_device=generate_on_device)
        else:
            raise ValueError("give a model folder, or a configuration (random weights)")
        act = torch.bfloat16 if EngineConfig(dtype=dtype).dtype == "bfloat16" else torch.float32
        if kv_slots is not None:
            pages = -(-kv_slots // page_size)
        else:
            pages = _auto_pages(self.model, page_size, act, torch.device(device), max_seqs, ctx,
                                gpu_memory_fraction, max_batch_tokens)
        self.cfg = EngineConfig(dtype=dtype, page_size=page_size, num_pages=pages, max_seqs=max_seqs, ctx=ctx,
                                max_batch_tokens=max_batch_tokens, max_logit_rows=max(max_seqs, 256),
                                seed=seed, cuda_graphs=cuda_graphs, device=device)
        self.runner = ModelRunner(self.model, self.cfg)
        self.scheduler = Scheduler(self.runner.manager, self._execute, max_seqs, max_batch_tokens, ctx,
                                   max_prefill_chunk=max_prefill_chunk, launch=self._launch, run_ahead=run_ahead,
                                   device_penalty_window=self.runner.HISTORY_WIDTH)
        self._ids = itertools.count()
        self.eos_token_ids = tuple(self.model.spec.eos_token_ids)

    # ---- requests ----------------------------------------------------------------------------
    def add_request(self, prompt_ids: Sequence[int], params: Optional[SamplingParams] = None,
                    max_new_tokens: int = 128, eos_token_ids: Optional[Sequence[int]] = None,
                    ignore_eos: bool = False, rid: Optional[Hashable] = None) -> Hashable:
        rid = next(self._ids) if rid is None else rid
        vocab = self.model.spec.vocab_size
        for t in prompt_ids:
            if not (0 <= int(t) < vocab):
                raise ValueError(f"token id {t} outside the vocabulary of {vocab}")
        self.scheduler.enqueue(Request(rid=rid, prompt=[int(t) for t in prompt_ids],
                                       params=params or SamplingParams(), max_new_tokens=max_new_tokens,
                                       eos_token_ids=tuple(self.eos_token_ids if eos_token_ids is None else eos_token_ids),
                                       ignore_eos=ignore_eos))
        return rid

    def step(self) -> List[Event]:
        """One scheduler step; a failing step fails every request and leaves the engine usable
        (crates/server/src/engine.rs:835-842)."""
        try:
            return self.scheduler.step()
        except Exception as e:                      # noqa: BLE001
            events = self.abort_all(f"step failed: {e}")
            if not events:
                raise
            self.last_error = e
            return events

    def abort_all(self, message: str = "aborted") -> List[Event]:
        """End every running and waiting request now and give back what they hold."""
        events = self.scheduler.abort_all(message)
        for rid in list(self.runner.manager.requests):
            self.runner.manager.close(rid)
        return events

    def is_idle(self) -> bool:
        return self.scheduler.is_idle()

    def generate(self, prompts: Sequence[Sequence[int]], params: Optional[SamplingParams] = None,
                 max_new_tokens: int = 128, ignore_eos: bool = False) -> List[List[int]]:
        """Host token ids in, host token ids out, all prompts batched continuously."""
        rids = [self.add_request(p, params, max_new_tokens, ignore_eos=ignore_eos) for p in prompts]
        out: Dict[Hashable, List[int]] = {r: [] for r in rids}
        self.finish_reasons: Dict[Hashable, str] = {}
        while not self.is_idle():
            for ev in self.step():
                if ev.rid in out:
                    if ev.token is not None:
                        out[ev.rid].append(ev.token)
                    if ev.finished:
                        self.finish_reasons[ev.rid] = ev.reason if ev.message is None else f"{ev.reason}: {ev.message}"
        return [out[r] for r in rids]

    # ---- low level -----------------------------------------------------------------------------
    def forward(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        return self.runner.step(entries)

    def _launch(self, items: List[PlanItem]):
        """Run a planned batch and sample; returns at once with the tokens still on their way
        (``.result()`` waits).  The picks also stay on the device, per request slot, for a step
        launched before they are read."""
        entries = [StepEntry(it.run.req.rid, it.tokens, [len(it.tokens) - 1] if it.samples else [])
                   for it in items]
        for it in items:
            if it.run.rc.fresh:                          # its first step in this slot (new, or recomputed)
                self.runner.reset_history(it.run.rc.slot, it.run.generated)
        logits = self.runner.step(entries)
        rows = [it for it in items if it.samples]
        if not rows:
            return ReadyTokens([])
        return sample_rows_async(logits, [it.run.sampler for it in rows], [it.run.generated for it in rows],
                                 [it.run.rc.slot for it in rows], self.runner.device_tokens,
                                 self.runner.history, self.runner.history_len)

    def _execute(self, items: List[PlanItem]) -> List[int]:
        return self._launch(items).result()
