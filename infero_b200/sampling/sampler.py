"""Device sampling for the rows of a step.

The pipeline and its order are the reference's (crates/model/src/sampling.rs:108-235): the
uniform draw is taken on the host from the request's own generator and handed to the
kernel, so only the selection runs on the device (crates/server/src/scheduler.rs:1279-1299).
Greedy rows go through the argmax kernel; the repetition penalty is applied to the logits
in place first (once per distinct token for greedy, once per occurrence otherwise, exactly
as sampling.rs:240-310 does).
"""
from __future__ import annotations

from collections import Counter
from typing import List, Optional, Sequence

import numpy as np
import torch

from .. import kernels as K
from .params import SamplingParams


class RowSampler:
    """Host-side state of one request's sampler: parameters and generator."""

    def __init__(self, params: SamplingParams):
        self.params = params
        self.rng = np.random.Generator(np.random.PCG64(params.seed))

    def next_draw(self) -> float:
        return float(self.rng.random())

    def penalty_pairs(self, history: Sequence[int]):
        p = self.params
        if p.repetition_penalty == 1.0 or not history:
            return []
        recent = history[-p.repetition_window:] if p.repetition_window > 0 else []
        if p.is_greedy():
            return [(t, 1) for t in sorted(set(recent))]
        return sorted(Counter(recent).items())


class DeviceFault(RuntimeError):
    """A kernel of the step gave up on one of its bounded waits: its output is not to be trusted."""


class PendingTokens:
    """Tokens picked on the device, on their way to the host.  Behind the picks travels the device's
    fault flag; ``result`` raises ``DeviceFault`` (and clears the flag) when a kernel of this step, or
    of any step since the flag was last read, ran out of patience, so that the tokens of such a step
    are never handed on."""

    def __init__(self, host: torch.Tensor, ready: "torch.cuda.Event", n: int):
        self._host, self._ready, self._n = host, ready, n

    def result(self) -> List[int]:
        self._ready.synchronize()
        h = self._host.numpy()
        if h.size > self._n and h[self._n] != 0:
            from ..kernels import tc_gemm
            code = int(h[self._n])
            tc_gemm.clear_error_flag()
            raise DeviceFault(f"a kernel's bounded wait ran out (code {code}); the step's output is discarded")
        return [int(t) for t in h[:self._n]]


class ReadyTokens:
    def __init__(self, tokens: List[int]):
        self._tokens = list(tokens)

    def result(self) -> List[int]:
        return self._tokens


def sample_rows_async(logits: torch.Tensor, samplers: Sequence[RowSampler], histories: Sequence[Sequence[int]],
                      slots: Optional[Sequence[int]] = None,
                      device_tokens: Optional[torch.Tensor] = None,
                      ring: Optional[torch.Tensor] = None, ring_len: Optional[torch.Tensor] = None) -> PendingTokens:
    """As ``sample_rows``, without waiting: the picks go to pinned host memory by an asynchronous
    copy, and (when ``slots`` and ``device_tokens`` are given) stay on the device in
    ``device_tokens[slot]`` so that the next step can be launched before the host has them.
    With ``ring`` / ``ring_len`` (the requests' generated tokens kept on the device, per slot) the
    repetition penalty is worked out there too and the picks are appended to the histories, so not
    even the penalty needs the tokens on the host; ``histories`` is then only the fallback for a
    window longer than the ring."""
    R, V = logits.shape
    assert len(samplers) == R and len(histories) == R
    dev = logits.device
    greedy = [s.params.is_greedy() for s in samplers]
    sampling = not all(greedy)
    penalised = [s.params.repetition_penalty != 1.0 and s.params.repetition_window > 0 for s in samplers]
    on_ring = (ring is not None and slots is not None and any(penalised)
               and all(s.params.repetition_window <= ring.shape[1] for s, p in zip(samplers, penalised) if p))
    # everything the device needs from the host this step, in one pinned buffer and one copy:
    # draws (64-bit) | slot per row, use-the-sample flag per row | temperature, top_p, top_k | penalty, window
    n_bytes = 16 * R + (12 * R if sampling else 0) + (8 * R if on_ring else 0)
    staged = torch.empty(n_bytes, dtype=torch.uint8, pin_memory=(dev.type == "cuda"))
    h = staged.numpy()
    info = h[8 * R:16 * R].view(np.int32)
    info[:R] = -1 if slots is None or device_tokens is None else np.asarray(slots, dtype=np.int32)
    info[R:] = [0 if g else 1 for g in greedy]
    o = 16 * R
    if sampling:
        # a draw is taken for every row, greedy or not, as the reference does (sampling.rs:113-121)
        h[:8 * R].view(np.float64)[:] = [s.next_draw() for s in samplers]
        h[o:o + 4 * R].view(np.float32)[:] = [max(s.params.temperature, 0.0) for s in samplers]
        h[o + 4 * R:o + 8 * R].view(np.float32)[:] = [s.params.top_p for s in samplers]
        h[o + 8 * R:o + 12 * R].view(np.int32)[:] = [s.params.top_k for s in samplers]
        o_pen = o + 12 * R
    else:
        o_pen = o
    if on_ring:
        h[o_pen:o_pen + 4 * R].view(np.float32)[:] = [s.params.repetition_penalty if p else 1.0
                                                     for s, p in zip(samplers, penalised)]
        h[o_pen + 4 * R:o_pen + 8 * R].view(np.int32)[:] = [s.params.repetition_window for s in samplers]
    on_dev = staged.to(dev, non_blocking=True)
    d_info = on_dev[8 * R:16 * R].view(torch.int32)
    if on_ring:
        K.apply_penalty_ring(logits, d_info, on_dev[o_pen:o_pen + 4 * R].view(torch.float32),
                             on_dev[o_pen + 4 * R:o_pen + 8 * R].view(torch.int32), ring, ring_len)
    elif any(penalised):
        pairs = [s.penalty_pairs(hh) for s, hh in zip(samplers, histories)]
        width = max((len(p) for p in pairs), default=0)
        if width:
            toks = np.full((R, width), -1, dtype=np.int32)
            cnts = np.zeros((R, width), dtype=np.int32)
            for r, p in enumerate(pairs):
                for i, (t, c) in enumerate(p):
                    toks[r, i], cnts[r, i] = t, c
            pen = np.array([s.params.repetition_penalty for s in samplers], dtype=np.float32)
            K.apply_penalty(logits, torch.from_numpy(toks).to(dev), torch.from_numpy(cnts).to(dev),
                            torch.from_numpy(pen).to(dev))
    out = torch.empty(3 * R + 1, dtype=torch.int32, device=dev)  # argmax | sampled | final | the fault flag
    K.argmax(logits, out[:R])
    sampled = None
    if sampling:
        sampled = out[R:2 * R]
        K.sample(logits, on_dev[o:o + 4 * R].view(torch.float32), on_dev[o + 8 * R:o + 12 * R].view(torch.int32),
                 on_dev[o + 4 * R:o + 8 * R].view(torch.float32), on_dev[:8 * R].view(torch.float64), sampled)
    keep = device_tokens if device_tokens is not None else out[2 * R:3 * R]      # slot -1: nothing is kept
    use_ring = ring is not None and slots is not None and device_tokens is not None
    K.keep_tokens(out[:R], sampled, d_info, out[2 * R:], keep, ring if use_ring else None, ring_len if use_ring else None,
                  with_fault=True)
    host = torch.empty(R + 1, dtype=torch.int32, pin_memory=True)
    host.copy_(out[2 * R:], non_blocking=True)
    ready = torch.cuda.Event()
    ready.record()
    pending = PendingTokens(host, ready, R)
    pending._keep = (out, staged, on_dev)          # alive until the copies have run
    return pending


def sample_rows(logits: torch.Tensor, samplers: Sequence[RowSampler],
                histories: Sequence[Sequence[int]]) -> List[int]:
    """Pick one token per row of ``logits`` [R, vocab] (float32, device; modified in place
    when a repetition penalty applies).  Returns host ints (one device-to-host copy)."""
    return sample_rows_async(logits, samplers, histories).result()
