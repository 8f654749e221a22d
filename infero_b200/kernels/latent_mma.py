"""The tensor-core kernel of latent attention (bf16 steps; ``csrc/latent_attention_mma.cu``).

The leading run of single-token requests (the scheduler puts them first) goes to the kernel's single-token form, with
long contexts cut into ranges of keys so that the grid fills the multiprocessors; what follows (prompt portions, and
single tokens behind one) to its tiled form, 64 / heads-per-CTA tokens a tile.  ``run`` returns False, with nothing
launched, where the kernel has no instance (sizes, element type) or the step gives no host copy of its lengths."""
from __future__ import annotations

import os
from ctypes import c_float, c_int, c_longlong

import torch

from . import _check, _i32, _ptr, _stream, lib

ENABLED = os.environ.get("INFERO_LATENT_MMA", "1") != "0"
MIN_CHUNK = int(os.environ.get("INFERO_LATENT_MIN_CHUNK", "64"))     # fewest keys per range of a cut context
launches = {"single": 0, "tiled": 0, "cut": 0}      # how often each form ran (tests look at it)


def supported(C: int, R: int) -> bool:
    return bool(lib().infero_latent_mma_supported(c_int(C), c_int(R)))


def plan_splits(n_tok: int, head_blocks: int, visible: int, sms: int):
    """(keys per range, ranges): about two CTAs per multiprocessor, ranges of whole key tiles, at least MIN_CHUNK keys."""
    want = max(1, (int(os.environ.get("INFERO_LATENT_CTAS_PER_SM", "2")) * sms) // max(1, n_tok * head_blocks))
    splits = max(1, min(want, visible // MIN_CHUNK, 64))
    chunk = -(-visible // splits)
    chunk = -(-chunk // 32) * 32
    return chunk, -(-visible // chunk)


def run(ctx, q_lat, q_rot, out, kv, table, n_tokens, H, C, R, scale) -> bool:
    cache = kv.k
    if not ENABLED or cache.dtype != torch.bfloat16 or not supported(C, R) or getattr(ctx, "h_q_len", None) is None:
        return False
    from .attention import _batch_shape
    from .tc_gemm import sm_count
    n_dec, vis_now, _, _ = _batch_shape(ctx)
    E = ctx.n_entries
    HC = int(lib().infero_latent_mma_heads(c_int(H)))
    rows = q_lat.shape[1]
    common = (_ptr(cache), _ptr(_i32(table, "block_table")), c_int(table.shape[1]), _ptr(_i32(ctx.entry_q_start, "entry_q_start")),
              _ptr(_i32(ctx.entry_q_len, "entry_q_len")), _ptr(_i32(ctx.entry_pos0, "entry_pos0")))
    if n_dec:
        vis = vis_now if getattr(ctx, "kv_bound", None) is None else int(ctx.kv_bound)
        chunk, splits = plan_splits(n_dec, -(-H // HC), max(vis, 1), sm_count(q_lat.device))
        part_o = part_ml = None
        launches["single"] += 1
        if splits > 1:
            launches["cut"] += 1
            part_o = torch.empty(n_dec * H * splits * C, dtype=torch.float32, device=q_lat.device)
            part_ml = torch.empty(n_dec * H * splits * 2, dtype=torch.float32, device=q_lat.device)
        _check(lib().infero_latent_attention_mma(_ptr(q_lat), _ptr(q_rot), c_longlong(rows), _ptr(out), _ptr(part_o), _ptr(part_ml),
                                                 *common, c_int(0), c_int(n_dec), c_int(n_dec), c_int(1), c_int(H), c_int(C),
                                                 c_int(R), c_int(kv.page_size), c_float(scale), c_int(chunk), c_int(splits),
                                                 _stream()))
    if n_dec < E:
        TQ = 64 // HC
        launches["tiled"] += 1
        tiles = sum(-(-int(n) // TQ) for n in ctx.h_q_len[n_dec:])
        _check(lib().infero_latent_attention_mma(_ptr(q_lat), _ptr(q_rot), c_longlong(rows), _ptr(out), _ptr(None), _ptr(None),
                                                 *common, c_int(n_dec), c_int(E), c_int(tiles), c_int(0), c_int(H), c_int(C),
                                                 c_int(R), c_int(kv.page_size), c_float(scale), c_int(0), c_int(1), _stream()))
    return True
