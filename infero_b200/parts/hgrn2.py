"""HGRN2 mixer: a gated linear recurrence with a matrix state per head."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..config.spec import MixerSpec
from ..kernels import layer_ops as L
from .base import Mixer, StateSpec, TensorDecl
from .linear import Linear


class Hgrn2Mixer(Mixer):
    """Per head, with q_t = silu(Wq h_t) (D), v_t = Wv h_t (V) and the forget gate
    f_t = l + (1 - l) sigmoid(Wf h_t + b) (D, l a stored lower bound):

        S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T,   o_t = S_t^T q_t,

    o_t RMS-normed over V with a weight shared by the heads, heads concatenated, output product.  The state
    (float32 [heads, D, V], zero at a sequence's start) lives in the request's state slot.  q, f and v are
    one stacked product; gates, state and norm are 32-bit on both precisions."""

    def __init__(self, spec: MixerSpec, prefix: str):
        self.spec, self.prefix = spec, prefix
        self.H, self.D, self.V = spec.num_heads, spec.head_dim, spec.v_dim
        self.names = spec.tensor_names()
        self.qfv: Linear = None
        self.out: Linear = None

    def _n(self, role: str, matrix: bool = True) -> str:
        return f"{self.prefix}.{self.names[role]}" + (self.spec.weight_suffix if matrix else "")

    def state_spec(self) -> Optional[StateSpec]:
        return StateSpec((self.H, self.D, self.V), torch.float32)

    def declare(self) -> List[TensorDecl]:
        H, D, V, d = self.H, self.D, self.V, self.spec.hidden
        return [TensorDecl(self._n("q"), (H * D, d)), TensorDecl(self._n("f"), (H * D, d)),
                TensorDecl(self._n("f_bias", False), (H * D,), role="bias"),
                TensorDecl(self._n("lower", False), (H * D,), role="bias", init="uniform"),
                TensorDecl(self._n("v"), (H * V, d)),
                TensorDecl(self._n("out_norm", False), (V,), role="norm", init="ones"),
                TensorDecl(self._n("o"), (d, H * V))]

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        w = torch.cat([tensors[self._n(r)] for r in ("q", "f", "v")], dim=0)
        self._rows = w
        self.qfv = Linear(w, None, f"{self.prefix}.qfv")
        self.extra = None
        self.out = Linear(tensors[self._n("o")], None, self._n("o"))
        self.f_bias = tensors[self._n("f_bias", False)].float().contiguous()
        self.lower = tensors[self._n("lower", False)].float().contiguous()
        self.out_norm = tensors[self._n("out_norm", False)].float().contiguous()

    def append_rows(self, weight: torch.Tensor) -> None:
        """Stack more rows of the layer's input product behind q, f and v; their result is left in
        ``ctx.extra_product`` (float32 [T, rows]) by ``forward``."""
        self.qfv = Linear(torch.cat([self._rows, weight], dim=0), None, f"{self.prefix}.qfv")
        self.extra = (self._rows.shape[0], weight.shape[0])

    def forward(self, ctx, h, slot):
        H, D, V = self.H, self.D, self.V
        T = h.shape[0]
        proj = self.qfv.forward(h, out_dtype=torch.float32)              # [T, 2 H D + H V (+ stacked rows)]
        ctx.extra_product = proj[:, self.extra[0]:self.extra[0] + self.extra[1]] if self.extra else None
        o = torch.empty((T, H * V), dtype=h.dtype, device=h.device)
        L.hgrn2_scan(proj, 0, H * D, 2 * H * D, self.f_bias, self.lower, self.out_norm, self.spec.norm_eps,
                     ctx.state(slot.cache), ctx.entry_q_start, ctx.entry_q_len, ctx.entry_slot, o, ctx.n_entries,
                     H, D, V, q_lens=None if ctx.decode_only else ctx.h_q_len)
        return self.out.forward(o, residual=True, out_dtype=torch.float32)
