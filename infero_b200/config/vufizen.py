"""Typed configuration of the Vufizen decoder, read from its own config.json keys.

config.json: ``architecture`` "Vufizen", ``vocab``, ``width``, ``norm.eps`` and ``layers``, a list with
one entry per layer: ``type`` ("hgrn2" or "attention"), ``mixer`` (that mixer's sizes and constants),
``mlp`` (null, or ``kind`` "moe" with ``expert.ff``, ``router.experts``, ``router.top`` and optionally
``shared.ff``) and optionally ``weights_of``: the index of the layer whose tensors this layer runs on,
with a cache and state of its own.  Layer i's tensors start with ``l<i>.``.

Lowering: a layer is a "gated_postnorm" block (the sublayers read the residual stream itself, their
result is gated, RMS-normed with a single stored number and added); the mixers are "hgrn2" and
"diff_attention", the feed-forward "moe_swiglu"; a layer that names another's weights becomes a second
schedule entry of that layer's block with its own cache slot.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .qwen2 import ConfigError
from .spec import (BlockSpec, FeedForwardSpec, MixerSpec, ModelSpec, NormSpec, PositionSpec, ScheduleEntry)


def _pos_int(d: Dict[str, Any], key: str, where: str) -> int:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        raise ConfigError(f"config.json: {where}.{key} must be a positive integer, got {v!r}")
    return v


@dataclass(frozen=True)
class VufizenMlp:
    experts: int
    top: int
    expert_ff: int
    shared_ff: int = 0               # 0: no shared expert


@dataclass(frozen=True)
class VufizenLayer:
    type: str                        # "hgrn2" | "attention"
    heads: int
    dim: int
    vdim: int
    kv_heads: int = 0                # attention only
    conv: int = 0                    # taps of the convolution on q, k, v; 0: none
    diff: float = 0.0
    scale: float = 0.0
    rot_base: float = 10000.0
    rot_dims: int = 0                # 0: no rotation
    mlp: Optional[VufizenMlp] = None
    weights_of: Optional[int] = None
    raw: Tuple[Tuple[str, Any], ...] = ()


@dataclass(frozen=True)
class VufizenConfig:
    vocab: int
    width: int
    eps: float
    layers: Tuple[VufizenLayer, ...]
    raw_layers: Tuple[Any, ...] = ()
    max_positions: int = 1 << 20

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "VufizenConfig":
        vocab, width = _pos_int(raw, "vocab", "config"), _pos_int(raw, "width", "config")
        norm = raw.get("norm") or {}
        eps = float(norm.get("eps", 1e-6))
        if not (eps > 0 and math.isfinite(eps)):
            raise ConfigError(f"config.json: norm.eps {eps} must be positive")
        entries = raw.get("layers")
        if not isinstance(entries, list) or not entries:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, L in enumerate(entries):
            where = f"layers[{i}]"
            kind = L.get("type")
            if kind not in ("hgrn2", "attention"):
                raise ConfigError(f"config.json: {where}.type {kind!r} is neither 'hgrn2' nor 'attention'")
            m = L.get("mixer")
            if not isinstance(m, dict):
                raise ConfigError(f"config.json: {where}.mixer is missing")
            heads, dim = _pos_int(m, "heads", where + ".mixer"), _pos_int(m, "dim", where + ".mixer")
            vdim = _pos_int(m, "vdim", where + ".mixer") if m.get("vdim") is not None else dim
            kw: Dict[str, Any] = {}
            if kind == "attention":
                kv = m.get("kv_heads")
                kv = heads if kv is None else _pos_int(m, "kv_heads", where + ".mixer")
                if heads % kv:
                    raise ConfigError(f"config.json: {where}: {heads} heads are no multiple of {kv} kv heads")
                rot = m.get("rot") or {}
                rot_dims = int(rot.get("dims", 0) or 0)
                if rot_dims % 2 or rot_dims > dim or rot_dims < 0:
                    raise ConfigError(f"config.json: {where}.mixer.rot.dims {rot_dims} must be even and at most dim {dim}")
                conv = int(m.get("conv", 0) or 0)
                if conv < 0 or conv > 16:
                    raise ConfigError(f"config.json: {where}.mixer.conv {conv} outside 0..16")
                kw = dict(kv_heads=kv, conv=conv, diff=float(m.get("diff", 0.0)),
                          scale=float(m["scale"]) if m.get("scale") is not None else 1.0 / math.sqrt(dim),
                          rot_base=float(rot.get("base", 10000.0)), rot_dims=rot_dims)
            mlp = None
            ml = L.get("mlp")
            if ml is not None:
                if ml.get("kind", "moe") != "moe":
                    raise ConfigError(f"config.json: {where}.mlp.kind {ml.get('kind')!r} is not 'moe'")
                router, expert = ml.get("router") or {}, ml.get("expert") or {}
                E, top = _pos_int(router, "experts", where + ".mlp.router"), _pos_int(router, "top", where + ".mlp.router")
                if top > E:
                    raise ConfigError(f"config.json: {where}.mlp: top {top} of {E} experts")
                shared = ml.get("shared")
                mlp = VufizenMlp(E, top, _pos_int(expert, "ff", where + ".mlp.expert"),
                                 _pos_int(shared, "ff", where + ".mlp.shared") if shared else 0)
            wo = L.get("weights_of")
            if wo is not None and not (isinstance(wo, int) and 0 <= wo < len(entries) and wo != i):
                raise ConfigError(f"config.json: {where}.weights_of {wo!r} names no other layer")
            layers.append(VufizenLayer(type=kind, heads=heads, dim=dim, vdim=vdim, mlp=mlp, weights_of=wo, **kw))
        cfg = cls(vocab=vocab, width=width, eps=eps, layers=tuple(layers), raw_layers=tuple(entries),
                  max_positions=int(raw.get("max_positions", 1 << 20)))
        for i in range(len(layers)):
            j = cfg.owner(i)
            a, b = layers[i], layers[j]
            if (a.type, a.heads, a.dim, a.vdim, a.kv_heads, a.conv, a.mlp) != (b.type, b.heads, b.dim, b.vdim, b.kv_heads, b.conv, b.mlp):
                raise ConfigError(f"config.json: layers[{i}] names the weights of layers[{j}] but differs from it")
        return cfg

    def owner(self, i: int) -> int:
        """The layer whose tensors layer i runs on."""
        seen = set()
        while self.layers[i].weights_of is not None:
            if i in seen:
                raise ConfigError("config.json: 'weights_of' goes in a circle")
            seen.add(i)
            i = self.layers[i].weights_of
        return i

    def to_json_dict(self) -> Dict[str, Any]:
        return {"architecture": "Vufizen", "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
                "layers": list(self.raw_layers)}

    # ---- lowering to parts ---------------------------------------------------------------------
    def to_model_spec(self) -> ModelSpec:
        d = self.width
        norm = NormSpec(kind="rmsnorm_scalar", dim=d, eps=self.eps)
        blocks, block_of = [], {}
        for i, L in enumerate(self.layers):
            if L.weights_of is not None:
                continue
            if L.type == "hgrn2":
                mixer = MixerSpec(kind="hgrn2", hidden=d, num_heads=L.heads, head_dim=L.dim, value_dim=L.vdim,
                                  norm_eps=self.eps, weight_suffix="")
            else:
                pos = PositionSpec("rope_interleaved", L.rot_base, L.rot_dims) if L.rot_dims else None
                mixer = MixerSpec(kind="diff_attention", hidden=d, num_heads=L.heads, num_kv_heads=L.kv_heads,
                                  head_dim=L.dim, value_dim=L.vdim, scale=L.scale, position=pos,
                                  conv_taps=L.conv, qk_norm=True, norm_eps=self.eps, diff=L.diff, weight_suffix="")
            ffn = None
            if L.mlp is not None:
                ffn = FeedForwardSpec(kind="moe_swiglu", hidden=d, intermediate=L.mlp.expert_ff, experts=L.mlp.experts,
                                      top=L.mlp.top, shared_intermediate=L.mlp.shared_ff, weight_suffix="")
            block_of[i] = len(blocks)
            blocks.append(BlockSpec(kind="gated_postnorm", prefix=f"l{i}", mixer=mixer, ffn=ffn, mixer_norm=norm,
                                    ffn_norm=norm if ffn is not None else None, mixer_norm_name="norm1",
                                    ffn_norm_name="norm2", mixer_gate_name="rg1",
                                    ffn_gate_name="rg2" if ffn is not None else None, gate_bias_suffix=".b"))
        schedule = tuple(ScheduleEntry(block=block_of[self.owner(i)], cache=i) for i in range(len(self.layers)))
        return ModelSpec(architecture="Vufizen", vocab_size=self.vocab, hidden=d, blocks=tuple(blocks),
                         schedule=schedule, final_norm=norm, tie_embeddings=False, embed_name="embed",
                         final_norm_name="final.norm", head_name="head", max_positions=self.max_positions)
