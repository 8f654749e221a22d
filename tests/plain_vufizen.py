"""A plain, slow statement of the Vufizen decoder on whole sequences, one function per mechanism, in
64-bit torch on the CPU.  It is what the engine's kernels, cache and scheduler are held to; it shares
nothing with the package (it reads the model folder through the test suite's own safetensors reader).

Notation: x [T, d] is the residual stream of one sequence, positions are 0..T-1, matrices are stored
[out, in] and applied as y = x @ W.T.
"""
from __future__ import annotations

import math
from typing import Dict, List

import torch


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps)


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def gated_update(x, y, gate_w, gate_b, g, eps):
    """x + g * unit_rms(y * sigmoid(x G^T + b)): the residual update of one sublayer (g one number)."""
    return x + g * unit_rms(y * torch.sigmoid(x @ gate_w.T + gate_b), eps)


def hgrn2(h, wq, wf, bf, lower, wv, w_norm, wo, heads, dim, vdim, eps, state=None):
    """Token by token: S <- diag(f) S + (1 - f) v^T; o = S^T q; per head unit_rms(o) * w_norm; then wo."""
    T = h.shape[0]
    q = silu(h @ wq.T).view(T, heads, dim)
    f = (lower + (1 - lower) * torch.sigmoid(h @ wf.T + bf)).view(T, heads, dim)
    v = (h @ wv.T).view(T, heads, vdim)
    S = torch.zeros(heads, dim, vdim, dtype=h.dtype) if state is None else state
    rows = []
    for t in range(T):
        S = f[t].unsqueeze(-1) * S + (1 - f[t]).unsqueeze(-1) * v[t].unsqueeze(-2)
        o = (S * q[t].unsqueeze(-1)).sum(dim=1)                    # [heads, vdim]
        rows.append((unit_rms(o, eps) * w_norm).reshape(-1))
    return torch.stack(rows) @ wo.T, S


def causal_conv(u, w):
    """y[t, c] = sum_j w[c, j] * u[t - (taps - 1) + j, c], zeros before the start; u [T, C], w [C, taps]."""
    T, C = u.shape
    taps = w.shape[1]
    y = torch.zeros_like(u)
    for t in range(T):
        for j in range(taps):
            s = t - (taps - 1) + j
            if s >= 0:
                y[t] += w[:, j] * u[s]
    return y


def rotate_adjacent(x, positions, base, dims):
    """Pairs (2i, 2i+1), i < dims/2, of the last axis turn by positions * base^(-2i/dims); x [T, n, D]."""
    out = x.clone()
    for i in range(dims // 2):
        ang = positions.to(torch.float64) * base ** (-2.0 * i / dims)
        c, s = torch.cos(ang).unsqueeze(-1).to(x.dtype), torch.sin(ang).unsqueeze(-1).to(x.dtype)
        a, b = x[..., 2 * i], x[..., 2 * i + 1]
        out[..., 2 * i] = a * c - b * s
        out[..., 2 * i + 1] = b * c + a * s
    return out


def softmax_causal(scores):
    """scores [T, T]; row i sees columns j <= i."""
    T = scores.shape[0]
    keep = torch.ones(T, T, dtype=torch.bool).tril()
    return torch.softmax(scores.masked_fill(~keep, float("-inf")), dim=-1)


def differential_lambda(lq1, lk1, lq2, lk2, diff):
    return math.exp(float(lq1 @ lk1)) - math.exp(float(lq2 @ lk2)) + diff


def differential_combine(a1, a2, lam, diff, eps):
    return unit_rms(a1 - lam * a2, eps) * (1 - diff)


def diff_attention(h, w, m, eps):
    """w: dict of this mixer's tensors by leaf name ('q', 'k.conv', 'q.norm', 'lq1', ...); m: its sizes."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m.get("kv_heads", m["heads"]), m["dim"], m.get("vdim", m["dim"])
    q, k, v = h @ w["q"].T, h @ w["k"].T, h @ w["v"].T
    if m.get("conv"):
        q, k, v = causal_conv(q, w["q.conv"]), causal_conv(k, w["k.conv"]), causal_conv(v, w["v.conv"])
    q = unit_rms(q.view(T, H, 2, D), eps) * w["q.norm"]
    k = unit_rms(k.view(T, G, 2, D), eps) * w["k.norm"]
    rot = m.get("rot")
    if rot and rot.get("dims"):
        pos = torch.arange(T)
        q = rotate_adjacent(q.reshape(T, H * 2, D), pos, rot["base"], rot["dims"]).view(T, H, 2, D)
        k = rotate_adjacent(k.reshape(T, G * 2, D), pos, rot["base"], rot["dims"]).view(T, G, 2, D)
    v = v.view(T, G, V)
    scale = m["scale"] if m.get("scale") is not None else 1 / math.sqrt(D)
    lam = differential_lambda(w["lq1"], w["lk1"], w["lq2"], w["lk2"], m.get("diff", 0.0))
    heads = []
    for hh in range(H):
        g = hh // (H // G)
        a = [softmax_causal(q[:, hh, mp] @ k[:, g, mp].T * scale) @ v[:, g] for mp in range(2)]
        heads.append(differential_combine(a[0], a[1], lam, m.get("diff", 0.0), eps))
    return torch.cat(heads, dim=-1) @ w["o"].T


def swiglu_expert(h, gate, up, down):
    return (silu(h @ gate.T) * (h @ up.T)) @ down.T


def route(h, router, top):
    """(chosen experts [T, top], weights [T, top]): the largest logits, softmax over those alone."""
    z = h @ router.T
    val, idx = torch.sort(z, dim=-1, descending=True, stable=True)
    return idx[:, :top], torch.softmax(val[:, :top], dim=-1)


def moe(h, w, c):
    """w: this feed-forward's tensors by leaf name ('e3.gate', 'router', 'shared.up', 'shared.sg', ...)."""
    idx, wt = route(h, w["router"], c["router"]["top"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(idx.shape[1]):
            e = int(idx[t, j])
            out[t] += wt[t, j] * swiglu_expert(h[t], w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"])
    if c.get("shared"):
        out = out + torch.sigmoid(h @ w["shared.sg"].T) * swiglu_expert(h, w["shared.gate"], w["shared.up"], w["shared.down"])
    return out


def _sub(w: Dict[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v for k, v in w.items() if k.startswith(prefix)}


def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: List[int], residuals: list = None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence."""
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.tensor(tokens)]
    for i, layer in enumerate(cfg["layers"]):
        j = i
        while cfg["layers"][j].get("weights_of") is not None:
            j = cfg["layers"][j]["weights_of"]
        p = f"l{j}."
        m = layer["mixer"]
        if layer["type"] == "hgrn2":
            mw = _sub(w, p + "mix.")
            y, _ = hgrn2(x, mw["q"], mw["f"], mw["f.b"], mw["lower"], mw["v"], mw["norm"], mw["o"], m["heads"],
                         m["dim"], m.get("vdim", m["dim"]), eps)
        else:
            y = diff_attention(x, _sub(w, p + "mix."), m, eps)
        x = gated_update(x, y, w[p + "rg1"], w[p + "rg1.b"], w[p + "norm1"], eps)
        if layer.get("mlp") is not None:
            y = moe(x, _sub(w, p + "mlp."), layer["mlp"])
            x = gated_update(x, y, w[p + "rg2"], w[p + "rg2.b"], w[p + "norm2"], eps)
        if residuals is not None:
            residuals.append(x.clone())
    return (unit_rms(x, eps) * w["final.norm"]) @ w["head"].T
