"""Choice of kernel for the experts of a mixture-of-experts feed-forward.

Few tokens: every (token, choice) streams the rows of its expert (bound by the bytes of the chosen experts).
Many tokens on the bf16 path: grouped tensor-core products over the pairs sorted by expert, so an expert's
matrices are read once per 64 rows.  The 32-bit path always streams."""
from __future__ import annotations

import os

import torch

from . import layer_ops as L

GROUPED_FROM = int(os.environ.get("INFERO_MOE_GROUPED_FROM", "5"))     # tokens from which the grouped path runs


def experts(h, gate_up, down, top_idx, top_w, shared, shared_gate, y) -> None:
    T, d = h.shape
    ff = gate_up.shape[1] // 2
    if (h.dtype == torch.bfloat16 and T >= GROUPED_FROM and d % 8 == 0 and ff % 8 == 0 and h.stride(0) % 8 == 0
            and h.data_ptr() % 16 == 0):
        L.moe_experts_grouped(h, gate_up, down, top_idx, top_w, shared, shared_gate, y)
        return
    # the streaming kernels index (token, choice) pairs by a grid dimension of at most 65,535
    step = max(1, 65535 // top_idx.shape[1])
    for a in range(0, T, step):
        b = min(T, a + step)
        L.moe_experts_streamed(h[a:b], gate_up, down, top_idx[a:b], top_w[a:b],
                               None if shared is None else shared[a:b], None if shared_gate is None else shared_gate[a:b],
                               y[a:b])
