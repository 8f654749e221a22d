"""Differential attention over the paged cache."""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

from ..config.spec import MixerSpec
from ..kernels import layer_ops as L
from ..registry import part_class
from .base import KvCacheSpec, Mixer, StateSpec, TensorDecl
from .linear import Linear


class DiffAttention(Mixer):
    """H query heads over G key/value heads (query head h reads kv head h // (H/G)).  A head has two maps:
    q has H * 2 * D rows and k has G * 2 * D rows, laid out head by head as [map 1 | map 2]; both maps
    attend (causal softmax, 32-bit) over the same values of width V.  Behind the stacked q/k/v product come,
    in this order, an optional causal convolution over time on every channel (``conv_taps`` values ending at
    the token, zeros before the sequence; the last taps-1 product rows of a request are its state), an
    RMS norm with a shared weight on every map of every head of q and k, and rotary positions on adjacent
    pairs.  With a1, a2 the maps' results, o = a1 - lambda a2, lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff
    (one number per layer, worked out when the weights are bound), then o / sqrt(mean(o^2) + eps) over V
    and the factor 1 - diff; heads concatenated, output product.

    The cache holds a key row of width 2 D per kv head ([map 1 | map 2]) and a value row of width V."""

    def __init__(self, spec: MixerSpec, prefix: str):
        if spec.num_kv_heads <= 0 or spec.num_heads % spec.num_kv_heads:
            raise ValueError(f"{spec.num_heads} heads are not a multiple of {spec.num_kv_heads} kv heads")
        self.spec, self.prefix = spec, prefix
        self.H, self.G, self.D, self.V = spec.num_heads, spec.num_kv_heads, spec.head_dim, spec.v_dim
        self.Cq, self.Ck, self.Cv = 2 * self.H * self.D, 2 * self.G * self.D, self.G * self.V
        self.taps = int(spec.conv_taps)
        self.names = spec.tensor_names()
        self.rope = None
        if spec.position is not None and spec.position.rotary_dim > 0:
            self.rope = part_class("position", spec.position.kind)(spec.position)
            if getattr(self.rope, "amplitude", 1.0) != 1.0:
                raise ValueError("this mixer's rotary kernel has no amplitude; the position table needs one")
            if getattr(self.rope, "pairing", None) != "adjacent":
                raise ValueError("differential attention turns adjacent pairs; position kind "
                                 f"'{spec.position.kind}' pairs otherwise")
        self.qkv: Linear = None
        self.out: Linear = None
        self.lam = 0.0

    def _n(self, role: str, matrix: bool = True) -> str:
        return f"{self.prefix}.{self.names[role]}" + (self.spec.weight_suffix if matrix else "")

    def cache_spec(self) -> Optional[KvCacheSpec]:
        return KvCacheSpec(self.G, 2 * self.D, self.spec.window, v_head_dim=self.V)

    def state_spec(self) -> Optional[StateSpec]:
        if self.taps <= 1:
            return None
        return StateSpec((self.taps - 1, self.Cq + self.Ck + self.Cv), torch.float32)

    def declare(self) -> List[TensorDecl]:
        d, D = self.spec.hidden, self.D
        out = [TensorDecl(self._n("q"), (self.Cq, d)), TensorDecl(self._n("k"), (self.Ck, d)),
               TensorDecl(self._n("v"), (self.Cv, d)), TensorDecl(self._n("o"), (d, self.H * self.V))]
        if self.spec.qk_norm:
            out += [TensorDecl(self._n(r, False), (D,), role="norm", init="ones") for r in ("q_norm", "k_norm")]
        if self.taps > 0:
            out += [TensorDecl(self._n(r, False), (c, self.taps), role="bias", init="conv")
                    for r, c in (("q_conv", self.Cq), ("k_conv", self.Ck), ("v_conv", self.Cv))]
        out += [TensorDecl(self._n(r, False), (D,), role="bias") for r in ("lq1", "lk1", "lq2", "lk2")]
        return out

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        s = self.spec
        self._rows = torch.cat([tensors[self._n(r)] for r in ("q", "k", "v")], dim=0)
        self.qkv = Linear(self._rows, None, f"{self.prefix}.qkv")
        self.extra = None
        self.out = Linear(tensors[self._n("o")], None, self._n("o"))
        f32 = lambda r: tensors[self._n(r, False)].float().contiguous()          # noqa: E731
        self.q_norm = f32("q_norm") if s.qk_norm else None
        self.k_norm = f32("k_norm") if s.qk_norm else None
        # stored [channels, taps]; the kernel reads tap j of all channels side by side
        self.conv_w = torch.cat([f32("q_conv"), f32("k_conv"), f32("v_conv")], dim=0).t().contiguous() if self.taps > 0 else None
        v = {r: tensors[self._n(r, False)].double().cpu() for r in ("lq1", "lk1", "lq2", "lk2")}
        self.lam = math.exp(float((v["lq1"] * v["lk1"]).sum())) - math.exp(float((v["lq2"] * v["lk2"]).sum())) + s.diff

    def append_rows(self, weight: torch.Tensor) -> None:
        """Stack more rows of the layer's input product behind q, k and v; their result is left in
        ``ctx.extra_product`` (float32 [T, rows]) by ``forward``."""
        self.qkv = Linear(torch.cat([self._rows, weight], dim=0), None, f"{self.prefix}.qkv")
        self.extra = (self._rows.shape[0], weight.shape[0])

    def forward(self, ctx, h, slot):
        s = self.spec
        H, G, D, V = self.H, self.G, self.D, self.V
        T = h.shape[0]
        proj = self.qkv.forward(h, out_dtype=torch.float32)                # [T, Cq + Ck + Cv (+ stacked rows)]
        ctx.extra_product = proj[:, self.extra[0]:self.extra[0] + self.extra[1]] if self.extra else None
        kv = ctx.kv_cache(slot.cache)
        table = ctx.block_table(kv.group)
        state = ctx.state(slot.cache) if self.taps > 1 else None
        from ..kernels import diff_attention as A
        padded = A.as_plain_heads(h.dtype, D, V, kv.page_size) and kv.k.is_contiguous() and kv.v.is_contiguous()
        q = torch.empty((T, self.Cq * (2 if padded else 1)), dtype=h.dtype, device=h.device)
        inv = self.rope.inv_freq(h.device) if self.rope is not None else None
        L.qkv_prepare(proj, self.conv_w, self.taps, state, self.q_norm, self.k_norm, s.norm_eps, inv, ctx.positions,
                      ctx.tok_entry, ctx.entry_q_start, ctx.entry_slot, table, q, kv.k, kv.v, kv.page_size,
                      2 * H, 2 * G, G, D, V, write_cache=slot.write_cache, q_pad=padded)
        if state is not None:
            L.conv_state_update(proj, state, self.taps, ctx.entry_q_start, ctx.entry_q_len, ctx.entry_slot,
                                ctx.n_entries, self.Cq + self.Ck + self.Cv)
        attn = torch.empty((T, H * V), dtype=h.dtype, device=h.device)
        A.paged_diff_attention(ctx, q, attn, kv, table, H, G, D, V, s.window, s.scale, self.lam, s.norm_eps,
                               1.0 - s.diff, q_padded=padded)
        return self.out.forward(attn, residual=True, out_dtype=torch.float32)
