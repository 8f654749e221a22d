"""Small Gositar configurations, random model folders and plain logits for the tests."""
from __future__ import annotations

import copy
import functools
import os
import random
import tempfile
from typing import Dict, List

import numpy as np
import torch

import plain_gositar as PG
import plain_qwen2

_TMP = tempfile.mkdtemp(prefix="infero_b200_gositar_")
# Largest |engine - plain| over a row of logits, relative to the request's largest |logit|.  bfloat16: measured over all
# cuts the worst row of these small, sharpened models is at 0.05 to 0.09 and the median near 0.02, the same for whole
# prompts, single tokens, portions and mixed batches (a wrong key, a lost page or a stream left out shows as 0.3 and more).
TOL = {"float32": 3e-5, "bfloat16": 0.12}


def _mix(heads, dim, rot_dim, vdim, rank, scale, base=5000.0, dims=None, yarn=None):
    rot = {"base": base, "dims": rot_dim if dims is None else dims}
    if yarn:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), yarn))
    return {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "scale": scale, "rot": rot}


def _moe(experts, top, ff, limit, groups=None, shared=None):
    m = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}
    if groups:
        m["router"]["groups"] = {"count": groups[0], "keep": groups[1]}
    if shared:
        m["shared"] = {"ff": shared[0], "limit": shared[1]}
    return m


# A: sizes the tensor-core products take; two streams; both mixer types; stretched and plain frequencies, more experts picked than groups kept (the stretch
#    begins inside a short test prompt: original 24); groups of experts; a layer without feed-forward
A = {"architecture": "Gositar", "vocab": 131, "width": 64, "norm": {"eps": 2e-5}, "streams": 2, "layers": [
    {"type": "latent_attention", "mixer": _mix(4, 16, 16, 24, 64, 0.3, yarn=(4.0, 24, 8.0, 1.0)), "mlp": _moe(8, 3, 24, 1.5, (4, 2), (40, 0.8))},
    {"type": "latent_attention_2", "mixer": _mix(2, 32, 8, 16, 32, 0.2, base=300.0), "mlp": {"kind": "dense", "ff": 96}},
    {"type": "latent_attention_2", "mixer": _mix(4, 16, 16, 24, 64, 0.3, yarn=(2.5, 16, 4.0, 0.5)), "mlp": None},
    {"type": "latent_attention", "mixer": _mix(2, 32, 8, 16, 32, 0.2, base=300.0), "mlp": _moe(8, 3, 24, 1.5, (4, 2), (40, 0.8))},
]}
# B: odd sizes (no tensor-core product takes them), three streams, three heads, fewer rotated coordinates than the
#    rotated part is wide, three groups of two, a shared expert with another limit
B = {"architecture": "Gositar", "vocab": 97, "width": 36, "norm": {"eps": 1e-6}, "streams": 3, "layers": [
    {"type": "latent_attention_2", "mixer": _mix(3, 6, 4, 10, 20, 0.4, base=77.0, dims=2), "mlp": _moe(6, 3, 10, 0.7, (3, 2), (6, 2.5))},
    {"type": "latent_attention", "mixer": _mix(3, 5, 6, 7, 12, 0.5, base=40.0, yarn=(3.0, 12, 6.0, 1.0)), "mlp": {"kind": "dense", "ff": 20}},
    {"type": "latent_attention", "mixer": _mix(1, 12, 2, 9, 11, 0.3, base=9.0), "mlp": _moe(4, 1, 8, 3.0)},
]}
# C: one plain residual (no streams key), no groups, as many choices as experts, no shared expert, one head
C = {"architecture": "Gositar", "vocab": 61, "width": 40, "norm": {"eps": 1e-5}, "layers": [
    {"type": "latent_attention", "mixer": _mix(1, 8, 8, 8, 16, 0.35), "mlp": _moe(3, 3, 16, 1.0)},
    {"type": "latent_attention_2", "mixer": _mix(5, 8, 2, 4, 8, 0.35), "mlp": None},
    {"type": "latent_attention_2", "mixer": _mix(2, 8, 8, 8, 24, 0.35, yarn=(8.0, 32, 16.0, 2.0)), "mlp": {"kind": "dense", "ff": 48}},
]}
# D: a single stream kept as streams (the small tensors are 1 x 1), one group that is kept
D = {"architecture": "Gositar", "vocab": 53, "width": 32, "norm": {"eps": 1e-6}, "streams": 1, "layers": [
    {"type": "latent_attention", "mixer": _mix(2, 8, 8, 8, 16, 0.35), "mlp": _moe(4, 2, 8, 2.0, (1, 1), (8, 2.0))},
    {"type": "latent_attention_2", "mixer": _mix(2, 8, 8, 8, 16, 0.35), "mlp": {"kind": "dense", "ff": 24}},
]}
# E: A with every expert chosen.  The choice of experts is a step function of the router's scores: in bf16 a near-tie
#    may fall the other way, which is no fault of either side and changes a token's result by far more than rounding.
#    Whole models in bf16 are therefore compared where the feed-forward is continuous (the weights still come from the
#    router); the choice itself is held to the plain statement by the routing test and by the 32-bit runs.
E = copy.deepcopy(A)
for _l in E["layers"]:
    if _l["mlp"] and _l["mlp"]["kind"] == "moe":
        _l["mlp"]["router"]["top"] = _l["mlp"]["router"]["experts"]
        _l["mlp"]["router"]["groups"]["keep"] = _l["mlp"]["router"]["groups"]["count"]
# F: sizes of the tensor-core attention kernel (latent 64 + 32 rotated; 128 + 64), every expert chosen, page size 64 runs
F = {"architecture": "Gositar", "vocab": 211, "width": 128, "norm": {"eps": 1e-6}, "streams": 4, "layers": [
    {"type": "latent_attention", "mixer": _mix(8, 32, 32, 32, 64, 0.15, yarn=(4.0, 64, 16.0, 1.0)), "mlp": {"kind": "dense", "ff": 256}},
    {"type": "latent_attention_2", "mixer": _mix(16, 64, 64, 64, 128, 0.1, base=1000.0), "mlp": _moe(4, 4, 64, 2.0, (2, 2), (64, 2.0))},
]}
CONFIGS = {"A": A, "B": B, "C": C, "D": D, "E": E, "F": F}


@functools.lru_cache(maxsize=None)
def model_dir(name: str, seed: int = 5, store: str = "bfloat16", sharp: float = 2.0) -> str:
    """A random model folder.  Random projections give an almost flat softmax, which hides a wrong key, so the query
    projection is multiplied by ``sharp``: scores then differ by several units."""
    from safetensors.torch import load_file, save_file
    from infero_b200.loading import write_random_model_dir
    d = os.path.join(_TMP, f"{name}_{seed}_{store}_{sharp}")
    write_random_model_dir(d, CONFIGS[name], seed=seed, dtype=store, std=0.15, norm_std=0.1)
    p = os.path.join(d, "model.safetensors")
    w = load_file(p)
    for k in list(w):
        if k.endswith("mix.q"):
            w[k] = (w[k].float() * sharp).to(w[k].dtype)
    save_file(w, p, metadata={"format": "pt"})
    return d


@functools.lru_cache(maxsize=None)
def plain_model(mdir: str):
    return plain_qwen2.read_model(mdir, torch.float64)


def plain_logits(mdir: str, reqs: Dict[str, List[int]]) -> Dict[str, np.ndarray]:
    cfg, w = plain_model(mdir)
    return {rid: PG.forward(cfg, w, toks).numpy() for rid, toks in reqs.items()}


def make_requests(name: str, lengths, seed: int = 0) -> Dict[str, List[int]]:
    rng = random.Random(seed)
    V = CONFIGS[name]["vocab"]
    return {f"r{i}": [rng.randrange(V) for _ in range(n)] for i, n in enumerate(lengths)}
