"""Choice of differential-attention kernel for a step.

The leading run of single-token requests (the scheduler puts decodes first) goes to the kernel that gives a
token a block of warps; what follows (prompt portions, and single tokens behind one) goes to the
tensor-core kernel when the step is bf16 and the sizes have an instance, else to the generic kernel (one
warp per token and head, any element type), which is the whole of prompt attention on the 32-bit path.
"""
from __future__ import annotations

from ctypes import c_float, c_int

import torch

from . import _check, _dt, _i32, _ptr, _stream, lib
from . import layer_ops as L
from .attention import _batch_shape

PREFILL_ROWS = 64


def prefill_supported(D: int, V: int, page_size: int) -> bool:
    return bool(lib().infero_diff_attn_prefill_supported(c_int(D), c_int(V), c_int(page_size)))


def decode(q, out, k_cache, v_cache, table, tok_entry, positions, n_tok, H, G, D, V, page_size, window, scale, lam,
           eps, out_scale) -> None:
    _check(lib().infero_diff_attn_decode(
        _ptr(q), c_int(q.stride(0)), _ptr(out), c_int(out.stride(0)), _ptr(k_cache), _ptr(v_cache), c_int(_dt(q)),
        _ptr(_i32(table, "block_table")), c_int(table.shape[1]), _ptr(_i32(tok_entry, "tok_entry")),
        _ptr(_i32(positions, "positions")), c_int(n_tok), c_int(H), c_int(G), c_int(D), c_int(V), c_int(page_size),
        c_int(window or 0), c_float(scale), c_float(lam), c_float(eps), c_float(out_scale), _stream()))


def prefill(q, out, k_cache, v_cache, table, entry_q_start, entry_q_len, entry_pos0, n_entries, first_entry, n_tiles,
            H, G, D, V, page_size, window, scale, lam, eps, out_scale) -> None:
    _check(lib().infero_diff_attn_prefill(
        _ptr(q), c_int(q.stride(0)), _ptr(out), c_int(out.stride(0)), _ptr(k_cache), _ptr(v_cache),
        _ptr(_i32(table, "block_table")), c_int(table.shape[1]), _ptr(_i32(entry_q_start, "entry_q_start")),
        _ptr(_i32(entry_q_len, "entry_q_len")), _ptr(_i32(entry_pos0, "entry_pos0")), c_int(n_entries),
        c_int(first_entry), c_int(n_tiles), c_int(H), c_int(G), c_int(D), c_int(V), c_int(page_size),
        c_int(window or 0), c_float(scale), c_float(lam), c_float(eps), c_float(out_scale), _stream()))


def as_plain_heads(dtype, D: int, V: int, page_size: int) -> bool:
    """Can the kernels for ordinary heads run this layer?  Where a value is as wide as a key row (V = 2 D), every map
    is an ordinary head of width V over the same cache once its query is padded with zeros in the other map's
    columns: bf16 steps then take the engine's split-context decode kernel and its tensor-core prompt kernels (2 H
    heads over G kv heads) and a small kernel that combines the maps."""
    from .attention import mma_supported
    return dtype == torch.bfloat16 and V == 2 * D and mma_supported(V, page_size)


def paged_diff_attention(ctx, q, out, kv, table, H, G, D, V, window, scale, lam, eps, out_scale, q_padded: bool = False) -> None:
    """q [T, H*2*D] (normed, rotated; [T, 2 H * 2 D] when ``q_padded``, see ``as_plain_heads``), out [T, H*V];
    keys [pages, G, page, 2 D], values [pages, G, page, V]."""
    if q_padded:
        from .attention import paged_attention
        maps = torch.empty((q.shape[0], 2 * H * V), dtype=q.dtype, device=q.device)
        paged_attention(ctx, q, maps, kv, table, 2 * H, G, V, window, scale)
        L.diff_combine(maps, out, H, V, lam, eps, out_scale)
        return
    n_dec, _, _, tiles_64 = _batch_shape(ctx)
    E, T = ctx.n_entries, q.shape[0]
    assert q.stride(1) == 1 and out.stride(1) == 1 and q.dtype == out.dtype == kv.k.dtype == kv.v.dtype
    if n_dec:
        decode(q, out, kv.k, kv.v, table, ctx.tok_entry, ctx.positions, n_dec, H, G, D, V, kv.page_size, window,
               scale, lam, eps, out_scale)
    if n_dec == E:
        return
    if q.dtype == torch.bfloat16 and prefill_supported(D, V, kv.page_size) and kv.k.is_contiguous() and kv.v.is_contiguous() \
            and q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0:
        prefill(q, out, kv.k, kv.v, table, ctx.entry_q_start, ctx.entry_q_len, ctx.entry_pos0, E, n_dec, tiles_64,
                H, G, D, V, kv.page_size, window, scale, lam, eps, out_scale)
        return
    L.diff_attention_generic(q[n_dec:], out[n_dec:], kv.k, kv.v, table, ctx.tok_entry[n_dec:], ctx.positions[n_dec:],
                             H, G, D, V, kv.page_size, window, scale, lam, eps, out_scale)
