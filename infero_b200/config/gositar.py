"""Typed configuration of the Gositar decoder, read from its own config.json keys.

config.json: ``architecture`` "Gositar", ``vocab``, ``width``, ``norm.eps``, optionally ``streams`` (the residual
kept as that many vectors per token, "hyper-connections"; absent: one plain residual) and ``layers``, a list with one
entry per layer: ``type`` "latent_attention" (rotation on adjacent pairs, a sigmoid gate per head on the result) or
"latent_attention_2" (rotation on pairs (i, i + dims/2), no gate), ``mixer`` (``heads``, ``dim``, ``rot_dim``, ``vdim``,
``kv_rank``, ``scale``, ``rot`` = {``base``, ``dims``, optionally ``scaling`` = {``factor``, ``original``, ``fast``,
``slow``}}) and ``mlp``: null, {``kind`` "dense", ``ff``} or {``kind`` "moe", ``expert`` {``ff``, ``limit``}, ``router``
{``experts``, ``top``, optionally ``groups`` {``count``, ``keep``}}, optionally ``shared`` {``ff``, ``limit``}}.
Layer i's tensors start with ``l<i>.``.

Lowering: layer norms (weight only); mixer "latent_attention" with the pairing as its position kind and the gate as a
flag; feed-forwards "relu2" and "moe_grouped" (clamped gated activation with the design's constant 1.702); blocks
"hyper_prenorm" with streams, "prenorm" without.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .qwen2 import ConfigError
from .spec import (BlockSpec, FeedForwardSpec, MixerSpec, ModelSpec, NormSpec, PositionSpec, ScheduleEntry)
from .vufizen import _pos_int

ACT_ALPHA = 1.702          # the slope inside the experts' sigmoid; fixed by the design
MIXER_TYPES = {"latent_attention": ("rope_interleaved", True), "latent_attention_2": ("rope_neox", False)}


def _number(d: Dict[str, Any], key: str, where: str, positive: bool = True) -> float:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, (int, float)) or not math.isfinite(v) or (positive and v <= 0):
        raise ConfigError(f"config.json: {where}.{key} must be a {'positive ' if positive else ''}number, got {v!r}")
    return float(v)


@dataclass(frozen=True)
class GositarMlp:
    kind: str                        # "dense" | "moe"
    ff: int                          # dense: the width; moe: an expert's width
    experts: int = 0
    top: int = 0
    limit: float = 0.0
    groups: int = 1
    keep: int = 1
    shared_ff: int = 0               # 0: no shared expert
    shared_limit: float = 0.0


@dataclass(frozen=True)
class GositarLayer:
    type: str
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    rot_base: float
    rot_dims: int
    yarn: Optional[Tuple[float, float, float, float]] = None
    mlp: Optional[GositarMlp] = None


@dataclass(frozen=True)
class GositarConfig:
    vocab: int
    width: int
    eps: float
    streams: int                     # 0: a plain residual
    layers: Tuple[GositarLayer, ...]
    raw: Tuple[Tuple[str, Any], ...] = ()
    max_positions: int = 1 << 20

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "GositarConfig":
        vocab, width = _pos_int(raw, "vocab", "config"), _pos_int(raw, "width", "config")
        eps = _number(raw.get("norm") or {}, "eps", "norm")
        streams = 0
        if raw.get("streams") is not None:
            streams = _pos_int(raw, "streams", "config")
            if streams > 8:
                raise ConfigError(f"config.json: {streams} streams, at most 8")
        entries = raw.get("layers")
        if not isinstance(entries, list) or not entries:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, L in enumerate(entries):
            where = f"layers[{i}]"
            if L.get("type") not in MIXER_TYPES:
                raise ConfigError(f"config.json: {where}.type {L.get('type')!r} is none of {sorted(MIXER_TYPES)}")
            m = L.get("mixer")
            if not isinstance(m, dict):
                raise ConfigError(f"config.json: {where}.mixer is missing")
            wm = where + ".mixer"
            heads, dim, rot_dim = _pos_int(m, "heads", wm), _pos_int(m, "dim", wm), _pos_int(m, "rot_dim", wm)
            vdim, rank = _pos_int(m, "vdim", wm), _pos_int(m, "kv_rank", wm)
            rot = m.get("rot") or {}
            rot_dims = int(rot.get("dims", rot_dim))
            if rot_dims % 2 or not 0 <= rot_dims <= rot_dim:
                raise ConfigError(f"config.json: {wm}.rot.dims {rot_dims} must be even and at most rot_dim {rot_dim}")
            base = _number(rot, "base", wm + ".rot") if rot_dims else 10000.0
            yarn = None
            sc = rot.get("scaling")
            if sc is not None and rot_dims:
                ws = wm + ".rot.scaling"
                yarn = (_number(sc, "factor", ws), _number(sc, "original", ws), _number(sc, "fast", ws), _number(sc, "slow", ws))
                if base == 1.0:
                    raise ConfigError(f"config.json: {ws} needs a base other than 1")
            mlp = None
            ml = L.get("mlp")
            if ml is not None:
                wl = where + ".mlp"
                if ml.get("kind") == "dense":
                    mlp = GositarMlp("dense", _pos_int(ml, "ff", wl))
                elif ml.get("kind") == "moe":
                    router, expert = ml.get("router") or {}, ml.get("expert") or {}
                    E, top = _pos_int(router, "experts", wl + ".router"), _pos_int(router, "top", wl + ".router")
                    if top > E:
                        raise ConfigError(f"config.json: {wl}: top {top} of {E} experts")
                    groups, keep = 1, 1
                    if router.get("groups") is not None:
                        groups = _pos_int(router["groups"], "count", wl + ".router.groups")
                        keep = _pos_int(router["groups"], "keep", wl + ".router.groups")
                        if E % groups or keep > groups or (E // groups) * keep < top:
                            raise ConfigError(f"config.json: {wl}.router: {groups} groups of {E} experts with {keep} kept "
                                              f"cannot give {top} choices")
                    shared = ml.get("shared")
                    mlp = GositarMlp("moe", _pos_int(expert, "ff", wl + ".expert"), E, top,
                                     _number(expert, "limit", wl + ".expert"), groups, keep,
                                     _pos_int(shared, "ff", wl + ".shared") if shared else 0,
                                     _number(shared, "limit", wl + ".shared") if shared else 0.0)
                else:
                    raise ConfigError(f"config.json: {wl}.kind {ml.get('kind')!r} is neither 'dense' nor 'moe'")
            layers.append(GositarLayer(L["type"], heads, dim, rot_dim, vdim, rank, _number(m, "scale", wm), base, rot_dims,
                                       yarn, mlp))
        return cls(vocab, width, eps, streams, tuple(layers), raw=tuple(raw.items()),
                   max_positions=int(raw.get("max_positions", 1 << 20)))

    def to_json_dict(self) -> Dict[str, Any]:
        keep = ("architecture", "vocab", "width", "norm", "streams", "layers", "max_positions")
        return {k: v for k, v in self.raw if k in keep}

    # ---- lowering to parts ---------------------------------------------------------------------
    def to_model_spec(self) -> ModelSpec:
        d = self.width
        norm = NormSpec(kind="layernorm", dim=d, eps=self.eps)
        blocks = []
        for i, L in enumerate(self.layers):
            pos_kind, gated = MIXER_TYPES[L.type]
            pos = PositionSpec(pos_kind, L.rot_base, L.rot_dims, yarn=L.yarn) if L.rot_dims else None
            mixer = MixerSpec(kind="latent_attention", hidden=d, num_heads=L.heads, num_kv_heads=1, head_dim=L.dim,
                              value_dim=L.vdim, rot_dim=L.rot_dim, latent_dim=L.kv_rank, out_gate=gated, scale=L.scale,
                              position=pos, norm_eps=self.eps, weight_suffix="")
            ffn = None
            if L.mlp is not None and L.mlp.kind == "dense":
                ffn = FeedForwardSpec(kind="relu2", hidden=d, intermediate=L.mlp.ff, weight_suffix="")
            elif L.mlp is not None:
                M = L.mlp
                ffn = FeedForwardSpec(kind="moe_grouped", hidden=d, intermediate=M.ff, experts=M.experts, top=M.top,
                                      shared_intermediate=M.shared_ff, activation="glu_clamped", limit=M.limit,
                                      act_alpha=ACT_ALPHA, shared_limit=M.shared_limit, route_groups=M.groups,
                                      route_keep=M.keep, route_correction=True, weight_suffix="")
            blocks.append(BlockSpec(kind="hyper_prenorm" if self.streams else "prenorm", prefix=f"l{i}", mixer=mixer,
                                    ffn=ffn, mixer_norm=norm, ffn_norm=norm if ffn is not None else None,
                                    mixer_norm_name="norm1", ffn_norm_name="norm2", streams=self.streams))
        schedule = tuple(ScheduleEntry(block=i, cache=i) for i in range(len(blocks)))
        return ModelSpec(architecture="Gositar", vocab_size=self.vocab, hidden=d, blocks=tuple(blocks),
                         schedule=schedule, final_norm=norm, tie_embeddings=False, embed_name="embed",
                         final_norm_name="final.norm", head_name="head", max_positions=self.max_positions,
                         streams=self.streams)
