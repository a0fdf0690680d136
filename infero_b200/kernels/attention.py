"""Choice of attention kernel for a step."""
from __future__ import annotations

from . import attention_generic


def paged_attention(ctx, qkv, out, kv, table, n_heads, n_kv, head_dim, window, scale) -> None:
    """qkv: [T, (H + 2 Hkv) D] with rotated queries in front; out [T, H*D]."""
    attention_generic(qkv, out, kv.k, kv.v, table, ctx.tok_entry, ctx.positions, n_heads, n_kv,
                      head_dim, kv.page_size, window, scale)
