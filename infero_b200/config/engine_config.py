"""Run-time limits of one engine instance (not part of a model's config.json).

The reference spreads these over CLI flags and ``INFERO_*`` environment switches
(crates/server/src/main.rs:13-135; crates/model/src/lib.rs:1338-1371): context length
``--ctx``, ``--max-seqs``, ``--kv-slots``, the per-pass token budget ``batch_tokens``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional


@dataclass
class EngineConfig:
    dtype: str = "bfloat16"            # "bfloat16" | "float32"
    page_size: int = 16                # tokens per cache page (16, 32 or 64)
    num_pages: Optional[int] = None    # pages of a cache group that keeps every key (a window group gets
                                       # what its live requests can hold at once); None = from max_tokens
    max_tokens: Optional[int] = None   # tokens the cache can hold (rounded up to pages)
    max_seqs: int = 32                 # live requests (--max-seqs)
    ctx: int = 4096                    # longest sequence (--ctx)
    max_batch_tokens: int = 2048       # token budget of one step
    max_logit_rows: int = 256          # rows of logits one step may return
    seed: int = 0
    cuda_graphs: bool = True
    device: str = "cuda:0"

    def __post_init__(self):
        if self.dtype in ("bf16",):
            self.dtype = "bfloat16"
        if self.dtype in ("fp32", "f32"):
            self.dtype = "float32"
        if self.dtype not in ("bfloat16", "float32"):
            raise ValueError(f"dtype must be bfloat16 or float32, got {self.dtype!r}")
        if self.page_size not in (16, 32, 64):
            raise ValueError(f"page_size must be 16, 32 or 64, got {self.page_size}")
        if self.max_seqs <= 0 or self.ctx <= 0 or self.max_batch_tokens <= 0:
            raise ValueError("max_seqs, ctx and max_batch_tokens must be positive")

    def pages_for(self, tokens: int) -> int:
        return -(-tokens // self.page_size)

    def resolved_num_pages(self) -> int:
        if self.num_pages is not None:
            return self.num_pages
        if self.max_tokens is not None:
            return self.pages_for(self.max_tokens)
        return self.max_seqs * self.pages_for(self.ctx)
