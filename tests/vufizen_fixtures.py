"""Small Vufizen configurations, random model folders and plain logits for the tests."""
from __future__ import annotations

import functools
import os
import random
import tempfile
from typing import Dict, List

import numpy as np
import torch

import plain_qwen2
import plain_vufizen as PV

_TMP = tempfile.mkdtemp(prefix="infero_b200_vufizen_")
# Largest |engine - plain| over a row of logits, relative to the request's largest |logit|.  bfloat16: in these
# small models the differential subtraction a1 - lambda a2 followed by a weightless norm amplifies the rounding of
# both maps; measured over all cuts the worst row is at 0.06 to 0.09 and the median at 0.02, the same for whole
# prompts, single tokens, portions and mixed batches (a wrong key, a lost state or a stale page shows as 0.3 and
# more); the recurrent-only model stays below 0.02.  The mechanisms' own tests hold the kernels to 2e-2 to 3e-2.
TOL = {"float32": 3e-5, "bfloat16": 0.12}


def _moe(experts, top, ff, shared=None):
    m = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def _att(heads, kv, dim, vdim, conv, diff, rot_dims, base=3000.0, scale=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "diff": diff}
    if conv:
        m["conv"] = conv
    if rot_dims:
        m["rot"] = {"base": base, "dims": rot_dims}
    if scale is not None:
        m["scale"] = scale
    return m


# A: sizes the tensor-core kernels take (map width 32 / 64, value width 48 / 32), two kv heads, partial rotation,
#    layers that run on another layer's tensors in another order, a layer without feed-forward
_A_ATT = _att(4, 2, 32, 48, 3, 0.3, 16, scale=0.25)
_A_HG = {"heads": 2, "dim": 16, "vdim": 32}
A = {"architecture": "Vufizen", "vocab": 131, "width": 64, "norm": {"eps": 2e-5}, "layers": [
    {"type": "attention", "mixer": _A_ATT, "mlp": _moe(5, 2, 24, shared=40)},
    {"type": "hgrn2", "mixer": _A_HG, "mlp": _moe(5, 2, 24)},
    {"type": "hgrn2", "mixer": _A_HG, "mlp": _moe(5, 2, 24), "weights_of": 1},
    {"type": "attention", "mixer": _A_ATT, "mlp": _moe(5, 2, 24, shared=40), "weights_of": 0},
    {"type": "attention", "mixer": _att(2, 2, 64, 32, 2, 0.55, 0), "mlp": None},
]}
# B: odd sizes (generic kernels), as many kv heads as heads, full rotation, five taps, one expert of three / all
#    three of three, one head
B = {"architecture": "Vufizen", "vocab": 97, "width": 40, "norm": {"eps": 1e-6}, "layers": [
    {"type": "hgrn2", "mixer": {"heads": 1, "dim": 12, "vdim": 20}, "mlp": _moe(3, 3, 12)},
    {"type": "attention", "mixer": _att(3, 3, 10, 14, 5, 0.8, 10), "mlp": _moe(3, 1, 12, shared=8)},
    {"type": "attention", "mixer": _att(2, 1, 12, 12, 0, 0.1, 4), "mlp": _moe(4, 2, 16)},
]}
# C: recurrent layers only: no paged cache at all
C = {"architecture": "Vufizen", "vocab": 61, "width": 32, "norm": {"eps": 1e-5}, "layers": [
    {"type": "hgrn2", "mixer": {"heads": 2, "dim": 24, "vdim": 16}, "mlp": _moe(2, 1, 16, shared=16)},
    {"type": "hgrn2", "mixer": {"heads": 4, "dim": 8, "vdim": 8}, "mlp": None},
]}
# D: A with every expert chosen.  The choice of experts is a step function of the router's logits: in bf16 a
#    near-tie may fall the other way, which is no fault of either side and changes a token's result by far more
#    than rounding.  Whole models in bf16 are therefore compared where the feed-forward is continuous (the
#    weights still come from the router); the choice itself is held to the plain statement by the routing
#    test and by the 32-bit runs of A and B.
import copy as _copy
D = _copy.deepcopy(A)
for _l in D["layers"]:
    if _l["mlp"]:
        _l["mlp"]["router"]["top"] = _l["mlp"]["router"]["experts"]
# E: a width that is no multiple of 8 (no tensor-core product takes it), prime sizes, one tap, one rotated pair, a
#    shared expert only where top = experts, kv_heads and scale left to their defaults
E = {"architecture": "Vufizen", "vocab": 53, "width": 36, "norm": {"eps": 3e-6}, "layers": [
    {"type": "attention", "mixer": {"heads": 3, "dim": 6, "vdim": 10, "conv": 1, "diff": 0.45, "rot": {"base": 77.0, "dims": 2}},
     "mlp": _moe(7, 7, 10, shared=6)},
    {"type": "hgrn2", "mixer": {"heads": 3, "dim": 5, "vdim": 7}, "mlp": _moe(7, 7, 10, shared=6)},
    {"type": "attention", "mixer": {"heads": 3, "dim": 6, "vdim": 10, "conv": 1, "diff": 0.45, "rot": {"base": 77.0, "dims": 2}},
     "mlp": _moe(7, 7, 10, shared=6), "weights_of": 0},
]}
CONFIGS = {"A": A, "B": B, "C": C, "D": D, "E": E}


@functools.lru_cache(maxsize=None)
def model_dir(name: str, seed: int = 5, store: str = "bfloat16", sharp: float = 2.5) -> str:
    """A random model folder.  Random projections give an almost flat softmax, which hides a wrong key, so the
    shared query-norm weight is multiplied by ``sharp``: scores then differ by several units."""
    from safetensors.torch import load_file, save_file
    from infero_b200.loading import write_random_model_dir
    d = os.path.join(_TMP, f"{name}_{seed}_{store}_{sharp}")
    write_random_model_dir(d, CONFIGS[name], seed=seed, dtype=store, std=0.15, norm_std=0.1)
    p = os.path.join(d, "model.safetensors")
    w = load_file(p)
    for k in list(w):
        if k.endswith("mix.q.norm"):
            w[k] = (w[k].float() * sharp).to(w[k].dtype)
        if k.endswith(("lq1", "lk1", "lq2", "lk2")):
            w[k] = (w[k].float() * 2.0).to(w[k].dtype)
    save_file(w, p, metadata={"format": "pt"})
    return d


@functools.lru_cache(maxsize=None)
def plain_model(mdir: str):
    return plain_qwen2.read_model(mdir, torch.float64)


def plain_logits(mdir: str, reqs: Dict[str, List[int]]) -> Dict[str, np.ndarray]:
    cfg, w = plain_model(mdir)
    return {rid: PV.forward(cfg, w, toks).numpy() for rid, toks in reqs.items()}


def make_requests(name: str, lengths, seed: int = 0) -> Dict[str, List[int]]:
    rng = random.Random(seed)
    V = CONFIGS[name]["vocab"]
    return {f"r{i}": [rng.randrange(V) for _ in range(n)] for i, n in enumerate(lengths)}
