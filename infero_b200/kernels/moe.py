"""Choice of kernel for the experts of a mixture-of-experts feed-forward."""
from __future__ import annotations

from . import layer_ops as L


def experts(h, gate_up, down, top_idx, top_w, shared, shared_gate, y) -> None:
    L.moe_experts_streamed(h, gate_up, down, top_idx, top_w, shared, shared_gate, y)
