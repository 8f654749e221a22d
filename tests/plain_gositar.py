"""A plain, slow statement of the Gositar decoder on whole sequences, one function per mechanism, in
64-bit torch on the CPU.  It is what the engine's kernels, cache and scheduler are held to; it shares
nothing with the package.

Notation: x [T, d] is one sequence (positions 0..T-1); matrices are stored [out, in] and applied as
y = x @ W.T; ``w`` maps tensor names to 64-bit tensors; ``cfg`` is the config.json dictionary.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


# ---- norms -----------------------------------------------------------------------------------------
def layer_norm(x, weight, eps):
    """(x - mean) / sqrt(var + eps) * weight, var the mean squared deviation; no bias."""
    mu = x.mean(dim=-1, keepdim=True)
    var = (x - mu).pow(2).mean(dim=-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * weight


def rms_norm(x, weight, eps):
    return x / torch.sqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps) * weight


# ---- rotary positions ------------------------------------------------------------------------------
def rotary_table(dims: int, base: float, scaling: Optional[dict]):
    """(frequencies [dims/2], amplitude).  Without scaling: base^(-2i/dims) and 1.  With a YaRN record
    {factor, original, fast, slow}: frequencies whose wavelength is long against ``original`` are divided by
    ``factor``, short ones stay, a linear ramp over the pair index in between; cos and sin grow by
    0.1 ln(factor) + 1."""
    half = dims // 2
    f = [base ** (-2.0 * i / dims) for i in range(half)]
    if not scaling:
        return torch.tensor(f, dtype=torch.float64), 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def index_of(turns):                                  # the pair index whose wave makes `turns` turns in `original`
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(index_of(float(scaling["fast"]))), 0)
    hi = min(math.ceil(index_of(float(scaling["slow"]))), dims - 1)
    out = []
    for i in range(half):
        ramp = min(1.0, max(0.0, (i - lo) / max(hi - lo, 0.001)))
        out.append(f[i] / factor * ramp + f[i] * (1.0 - ramp))
    return torch.tensor(out, dtype=torch.float64), 0.1 * math.log(factor) + 1.0


def rotate(x, positions, freqs, amp: float, pairing: str):
    """x [T, n, D]: the first 2 * len(freqs) coordinates turn, pair (a, b) -> (a cos - b sin, b cos + a sin) with
    cos and sin scaled by ``amp``; "adjacent": pairs (2i, 2i+1); "half": pairs (i, i + dims/2)."""
    half = freqs.numel()
    ang = positions.to(torch.float64).unsqueeze(-1) * freqs            # [T, half]
    c, s = (torch.cos(ang) * amp).unsqueeze(1), (torch.sin(ang) * amp).unsqueeze(1)
    out = x.clone()
    if pairing == "adjacent":
        a, b = x[..., 0:2 * half:2], x[..., 1:2 * half:2]
        out[..., 0:2 * half:2] = a * c - b * s
        out[..., 1:2 * half:2] = b * c + a * s
    else:
        a, b = x[..., :half], x[..., half:2 * half]
        out[..., :half] = a * c - b * s
        out[..., half:2 * half] = b * c + a * s
    return out


# ---- latent attention ------------------------------------------------------------------------------
def latent_attention(h, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float, pairing: str, gated: bool,
                     positions=None):
    """Keys and values are made from one small vector per token: c = rms_norm(first kv_rank rows of Wdkv h);
    head n's key is [Wuk_n c | rotated last rot_dim rows of Wdkv h] and its value Wuv_n c; the query is laid out
    per head as [dim | rot_dim] and its second part is rotated.  Causal softmax of q . k * scale."""
    T = h.shape[0]
    H, D, R, V, C = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    positions = torch.arange(T) if positions is None else positions
    rot = m.get("rot") or {}
    freqs, amp = rotary_table(int(rot.get("dims", R)), float(rot.get("base", 10000.0)), rot.get("scaling"))
    q = (h @ w[p + ".q"].T).view(T, H, D + R)
    q_plain, q_rot = q[..., :D], rotate(q[..., D:], positions, freqs, amp, pairing)
    down = h @ w[p + ".dkv"].T
    c = rms_norm(down[:, :C], w[p + ".dkv.norm"], eps)
    k_rot = rotate(down[:, C:].unsqueeze(1), positions, freqs, amp, pairing)[:, 0]           # [T, R], one for all heads
    k_plain = (c @ w[p + ".uk"].T).view(T, H, D)
    v = (c @ w[p + ".uv"].T).view(T, H, V)
    scores = (torch.einsum("thd,shd->hts", q_plain, k_plain) + torch.einsum("thr,sr->hts", q_rot, k_rot)) * m["scale"]
    mask = positions.unsqueeze(1) >= positions.unsqueeze(0)
    scores = scores.masked_fill(~mask, float("-inf"))
    o = torch.einsum("hts,shv->thv", torch.softmax(scores, dim=-1), v)
    if gated:
        o = o * torch.sigmoid(h @ w[p + ".g"].T).unsqueeze(-1)
    return o.reshape(T, H * V) @ w[p + ".o"].T


# ---- feed-forward ----------------------------------------------------------------------------------
def relu2_ff(h, up, down):
    return torch.relu(h @ up.T).pow(2) @ down.T


def clamped_glu(h, gate, up, down, limit: float):
    """g = min(gate h, limit), u = clamp(up h, -limit, limit); down (g sigmoid(1.702 g) (u + 1))."""
    g = torch.clamp(h @ gate.T, max=limit)
    u = torch.clamp(h @ up.T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ down.T


def route(z, correction, n_groups: int, keep: int, top: int):
    """z [T, E] router logits -> (index [T, top], weight [T, top]).  s = softmax(z); experts are picked by
    s + correction, among the ``keep`` groups (of E / n_groups neighbours) whose best pick score is largest;
    weights are s of the picked, normalised over the picked."""
    T, E = z.shape
    s = torch.softmax(z, dim=-1)
    pick = s + correction
    if n_groups > 1 and keep < n_groups:
        best = pick.view(T, n_groups, E // n_groups).max(dim=-1).values
        kept = torch.zeros(T, n_groups, dtype=torch.bool)
        kept.scatter_(1, best.topk(keep, dim=-1).indices, True)
        pick = pick.masked_fill(~kept.repeat_interleave(E // n_groups, dim=1), float("-inf"))
    idx = pick.topk(top, dim=-1).indices
    ws = s.gather(1, idx)
    return idx, ws / (ws.sum(dim=-1, keepdim=True) + 1e-20)


def moe_ff(h, w, p: str, ml: dict):
    r = ml["router"]
    E, top = r["experts"], r["top"]
    groups = r.get("groups") or {}
    z = h @ w[p + ".router"].T
    corr = w.get(p + ".correction")
    idx, ws = route(z, corr if corr is not None else torch.zeros(E, dtype=h.dtype), int(groups.get("count", 1)),
                    int(groups.get("keep", 1)), top)
    limit = float(ml["expert"]["limit"])
    y = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for c in range(top):
            e = int(idx[t, c])
            y[t] += ws[t, c] * clamped_glu(h[t:t + 1], w[f"{p}.e{e}.gate"], w[f"{p}.e{e}.up"], w[f"{p}.e{e}.down"], limit)[0]
    if ml.get("shared"):
        y = y + clamped_glu(h, w[p + ".shared.gate"], w[p + ".shared.up"], w[p + ".shared.down"], float(ml["shared"]["limit"]))
    return y


def feed_forward(h, w, p: str, ml: dict):
    if ml["kind"] == "dense":
        return relu2_ff(h, w[p + ".up"], w[p + ".down"])
    return moe_ff(h, w, p, ml)


# ---- residual streams ------------------------------------------------------------------------------
def hyper_sublayer(xs, w_in, w_mix, w_out, norm_w, eps, fn):
    """xs [S, T, d].  u = sum_s in[s] xs[s]; y = fn(layer_norm(u)); new xs[t] = sum_s mix[s, t] xs[s] + out[t] y."""
    u = torch.einsum("s,std->td", w_in, xs)
    y = fn(layer_norm(u, norm_w, eps))
    return torch.einsum("sr,std->rtd", w_mix, xs) + w_out.view(-1, 1, 1) * y.unsqueeze(0)


def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: List[int], per_layer: bool = False):
    """Logits [T, vocab] of one sequence (and, if asked, the residual stream after every layer)."""
    eps = float(cfg["norm"]["eps"])
    x = w["embed"][torch.tensor(tokens, dtype=torch.long)]
    S = cfg.get("streams")
    xs = x.unsqueeze(0).repeat(S, 1, 1) if S else None
    trail = []
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}"
        pairing = "adjacent" if L["type"] == "latent_attention" else "half"
        gated = L["type"] == "latent_attention"
        mixer = lambda h: latent_attention(h, w, p + ".mix", L["mixer"], eps, pairing, gated)          # noqa: E731
        ff = (lambda h: feed_forward(h, w, p + ".mlp", L["mlp"])) if L.get("mlp") else None          # noqa: E731
        if S:
            xs = hyper_sublayer(xs, w[p + ".hc1.in"], w[p + ".hc1.mix"], w[p + ".hc1.out"], w[p + ".norm1"], eps, mixer)
            if ff:
                xs = hyper_sublayer(xs, w[p + ".hc2.in"], w[p + ".hc2.mix"], w[p + ".hc2.out"], w[p + ".norm2"], eps, ff)
            trail.append(xs.sum(dim=0))
        else:
            x = x + mixer(layer_norm(x, w[p + ".norm1"], eps))
            if ff:
                x = x + ff(layer_norm(x, w[p + ".norm2"], eps))
            trail.append(x)
    if S:
        x = xs.sum(dim=0)
    logits = layer_norm(x, w["final.norm"], eps) @ w["head"].T
    return (logits, torch.stack(trail)) if per_layer else logits
