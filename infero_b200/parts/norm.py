"""RMSNorm with the residual add fused in front of it."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import kernels as K
from ..config.spec import NormSpec
from .base import Norm, TensorDecl


class RmsNorm(Norm):
    """h = v * rsqrt(mean(v^2) + eps) * w with v = x (+ delta), all in 32-bit
    (crates/kernels/src/cu/ops.cu:44-62; fused add as in cu/mmvq.cu:761)."""

    def __init__(self, spec: NormSpec, weight_name: str):
        self.spec = spec
        self.weight_name = weight_name
        self.weight: Optional[torch.Tensor] = None

    def declare(self) -> List[TensorDecl]:
        return [TensorDecl(self.weight_name, (self.spec.dim,), role="norm", init="ones")]

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors[self.weight_name].contiguous()

    def forward(self, ctx, x, delta, rows=None):
        n = x.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, self.spec.dim), dtype=ctx.act_dtype, device=x.device)
        K.add_rmsnorm(x, delta, self.weight, self.spec.eps, out, rows)
        return out


class ScalarRmsNorm(RmsNorm):
    """x * rsqrt(mean(x^2) + eps) * g with g a single stored number.  ``scalar`` is that number as a
    float32 tensor of one element (what kernels that normalise a sublayer's result take); ``weight`` is
    it repeated over the coordinates, which the shared norm kernel takes."""

    def __init__(self, spec: NormSpec, weight_name: str):
        super().__init__(spec, weight_name)
        self.scalar: Optional[torch.Tensor] = None

    def declare(self) -> List[TensorDecl]:
        return [TensorDecl(self.weight_name, (), role="norm", init="ones")]

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.scalar = tensors[self.weight_name].reshape(1).float().contiguous()
        self.weight = self.scalar.expand(self.spec.dim).contiguous()


class LayerNorm(Norm):
    """h = (v - mean(v)) * rsqrt(mean((v - mean(v))^2) + eps) * w with v = x (+ delta), no bias, all in 32-bit."""

    def __init__(self, spec: NormSpec, weight_name: str):
        self.spec = spec
        self.weight_name = weight_name
        self.weight: Optional[torch.Tensor] = None

    def declare(self) -> List[TensorDecl]:
        return [TensorDecl(self.weight_name, (self.spec.dim,), role="norm", init="ones")]

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors[self.weight_name].float().contiguous()

    def forward(self, ctx, x, delta, rows=None):
        from ..kernels import layer_ops as L
        n = x.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, self.spec.dim), dtype=ctx.act_dtype, device=x.device)
        if hasattr(delta, "as_partials"):
            delta = delta.as_partials()
        if isinstance(delta, K.Partials):
            delta = delta.materialize(torch.float32)
        elif delta is not None and delta.dtype != torch.float32:
            delta = delta.float()
        L.add_layernorm(x, delta, self.weight, self.spec.eps, out, rows)
        return out
