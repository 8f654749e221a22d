"""Choice of differential-attention kernel for a step."""
from __future__ import annotations

from . import layer_ops as L


def paged_diff_attention(ctx, q, out, kv, table, H, G, D, V, window, scale, lam, eps, out_scale) -> None:
    """q [T, H*2*D] (normed, rotated), out [T, H*V]."""
    L.diff_attention_generic(q, out, kv.k, kv.v, table, ctx.tok_entry, ctx.positions, H, G, D, V, kv.page_size,
                             window, scale, lam, eps, out_scale)
