"""Sampling parameters, with the reference's names, meanings and defaults
(crates/model/src/sampling.rs:12-48)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional


@dataclass
class SamplingParams:
    temperature: float = 0.7          # <= 0 means greedy: always the argmax
    top_p: float = 0.8                # >= 1 disables the nucleus cut
    top_k: int = 20                   # 1 means greedy; 0 keeps as many as the device sampler can
    repetition_penalty: float = 1.05  # divides positive / multiplies negative logits of seen tokens
    repetition_window: int = 256      # how far back the penalty looks
    seed: Optional[int] = None

    @classmethod
    def greedy(cls) -> "SamplingParams":
        return cls(temperature=0.0)

    def is_greedy(self) -> bool:
        return self.temperature <= 0.0 or self.top_k == 1
