"""The Gositar decoder in the engine against the plain statement (tests/plain_gositar.py): each mechanism's
kernels alone, then whole models through the step function, the cache manager and the scheduler."""
import math
import types

import numpy as np
import pytest
import torch

import plain_gositar as PG
import replay_util as R
from engine_fixtures import make_runner
from gositar_fixtures import CONFIGS, TOL, make_requests, model_dir, plain_logits, plain_model

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _rel(got, ref):
    ref = ref.double()
    return float((got.double().cpu() - ref).abs().max() / ref.abs().max())


def _i32(a):
    return torch.tensor(list(a), dtype=torch.int32, device=DEV)


# ---- mechanisms alone --------------------------------------------------------------------------------------
@pytest.mark.parametrize("d", [36, 64, 1000])
def test_layer_norm_with_the_add_in_front(d):
    from infero_b200.kernels import layer_ops as L
    g = torch.Generator().manual_seed(d)
    x, delta, w = torch.randn(9, d, generator=g) * 3 + 1.5, torch.randn(9, d, generator=g), 1 + 0.2 * torch.randn(d, generator=g)
    xd = x.to(DEV)
    for dtype, tol in ((torch.float32, 3e-6), (torch.bfloat16, 6e-3)):
        xd = x.to(DEV)
        out = torch.empty(9, d, dtype=dtype, device=DEV)
        L.add_layernorm(xd, delta.to(DEV), w.to(DEV), 1e-5, out)
        assert _rel(xd, x.double() + delta.double()) < 1e-6
        assert _rel(out, PG.layer_norm(x.double() + delta.double(), w.double(), 1e-5)) < tol
    rows = _i32([7, 2, 2])
    out = torch.empty(3, d, device=DEV)
    before = xd.clone()
    L.add_layernorm(xd, None, w.to(DEV), 1e-5, out, rows)
    assert torch.equal(xd, before)
    assert _rel(out, PG.layer_norm(before.cpu().double()[[7, 2, 2]], w.double(), 1e-5)) < 3e-6


@pytest.mark.parametrize("S,d", [(1, 40), (2, 64), (3, 36), (5, 130), (8, 33)])
def test_streams_update_and_read_out_in_one_pass(S, d):
    """The update of one sublayer and the weighted sum and norm for the next, against the plain statement; a mix
    matrix that is not symmetric (from and to must not be swapped); the sum of the streams on chosen rows."""
    from infero_b200.kernels import layer_ops as L
    g = torch.Generator().manual_seed(S * 100 + d)
    T = 6
    xs = torch.randn(S, T, d, generator=g)
    y = torch.randn(T, d, generator=g)
    w_in, w_out = torch.randn(S, generator=g), torch.randn(S, generator=g)
    mix = torch.eye(S) + torch.randn(S, S, generator=g) * 0.4
    w_in2, norm_w = torch.randn(S, generator=g), 1 + 0.2 * torch.randn(d, generator=g)
    # the plain statement: a sublayer that returns y whatever it gets
    want_xs = PG.hyper_sublayer(xs.double(), w_in.double(), mix.double(), w_out.double(), norm_w.double(), 1e-5, lambda h: y.double())
    want_h = PG.layer_norm(torch.einsum("s,std->td", w_in2.double(), want_xs), norm_w.double(), 1e-5)
    xd = xs.permute(1, 0, 2).contiguous().to(DEV)                     # the engine keeps [T, S, d]
    h = torch.empty(T, d, device=DEV)
    L.hyper_step(xd, y.to(DEV), mix.to(DEV), w_out.to(DEV), w_in2.to(DEV), norm_w.to(DEV), 1e-5, h)
    assert _rel(xd.permute(1, 0, 2), want_xs) < 2e-6
    assert _rel(h, want_h) < 5e-6
    hb = torch.empty(T, d, dtype=torch.bfloat16, device=DEV)
    L.hyper_step(xd, None, None, None, w_in2.to(DEV), norm_w.to(DEV), 1e-5, hb)      # read-out alone changes nothing
    assert _rel(xd.permute(1, 0, 2), want_xs) < 2e-6 and _rel(hb, want_h) < 6e-3
    total = torch.empty(2, d, device=DEV)
    L.hyper_step(xd, None, None, None, None, None, 0.0, None, u_out=total, rows=_i32([4, 1]))
    assert _rel(total, want_xs.sum(dim=0)[[4, 1]]) < 2e-6
    fill = torch.empty(T, S, d, device=DEV)
    L.streams_fill(y.to(DEV), fill)
    assert all(torch.equal(fill[:, s].cpu(), y) for s in range(S))


def test_relu2_and_the_clamped_gated_activation():
    from infero_b200.kernels import layer_ops as L, Partials
    g = torch.Generator().manual_seed(1)
    v = torch.randn(5, 24, generator=g) * 3
    out = torch.empty(5, 24, device=DEV)
    L.relu2(v.to(DEV), out)
    assert _rel(out, torch.relu(v.double()).pow(2)) < 1e-6
    parts = torch.randn(3, 5, 24, generator=g)
    ob = torch.empty(5, 24, dtype=torch.bfloat16, device=DEV)
    L.relu2(Partials(parts.to(DEV)), ob)
    assert _rel(ob, torch.relu(parts.double().sum(0)).pow(2)) < 6e-3
    act = torch.empty(5, 12, device=DEV)
    L.glu_act(v.to(DEV), act, ("glu_clamped", 1.25, 1.702))
    gate, up = v.double()[:, 0::2], v.double()[:, 1::2]
    eye = torch.eye(12, dtype=torch.float64)
    # the plain expert with identity matrices is the activation itself
    want = PG.clamped_glu(torch.cat([gate, up], dim=1), torch.cat([eye, 0 * eye], dim=1), torch.cat([0 * eye, eye], dim=1), eye, 1.25)
    assert _rel(act, want) < 1e-6
    assert float((gate > 1.25).sum()) > 0 and float((up.abs() > 1.25).sum()) > 0      # the clamps were at work
    L.glu_act(v.to(DEV), act, None)
    assert _rel(act, gate * torch.sigmoid(gate) * up) < 1e-6


@pytest.mark.parametrize("M,N,K", [(300, 96, 64), (700, 256, 128), (1030, 520, 72)])
def test_activations_in_the_epilogue_of_the_many_row_product(M, N, K):
    """Squared relu and the clamped gated activation inside the tcgen05 product's epilogue against product-then-activation
    in 64-bit; 256 rows and fewer are refused (they take the split-K path and the activation kernel)."""
    from infero_b200.kernels import tc_gemm
    g = torch.Generator().manual_seed(M)
    a = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) * 0.3).to(torch.bfloat16)
    ref = a.double() @ w.double().T
    out = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    assert tc_gemm.gemm_act(a.to(DEV), w.to(DEV), out, "relu2")
    assert _rel(out, torch.relu(ref).pow(2)) < 1e-2
    out = torch.empty(M, N // 2, dtype=torch.bfloat16, device=DEV)
    assert tc_gemm.gemm_act(a.to(DEV), w.to(DEV), out, "glu_clamped", 1.5, 1.702)
    gate, up = ref[:, 0::2].clamp(max=1.5), ref[:, 1::2].clamp(-1.5, 1.5)
    assert _rel(out, gate * torch.sigmoid(1.702 * gate) * (up + 1)) < 1e-2
    assert float((ref[:, 0::2] > 1.5).float().mean()) > 0.05
    assert not tc_gemm.gemm_act(a[:200].to(DEV), w.to(DEV), out[:200], "glu_clamped", 1.5, 1.702)


def test_rotary_tables_on_the_device_and_both_pairings():
    """The prepare kernel's rotation against the plain one: stretched frequencies with their amplitude, both pairings,
    fewer rotated coordinates than the part is wide, positions far out."""
    from infero_b200.config.spec import PositionSpec
    from infero_b200.kernels import latent_attention as A
    from infero_b200.parts.rope import RopeInterleaved, RopeNeox
    g = torch.Generator().manual_seed(2)
    H, D, R, C, page = 3, 5, 12, 7, 16
    for cls, pairing, dims, yarn in ((RopeNeox, "half", 12, (4.0, 64.0, 8.0, 1.0)), (RopeInterleaved, "adjacent", 12, (4.0, 64.0, 8.0, 1.0)),
                                     (RopeNeox, "half", 8, None), (RopeInterleaved, "adjacent", 2, (1.7, 5.0, 2.0, 0.3))):
        rope = cls(PositionSpec("x", 123.0, dims, yarn=yarn))
        freqs, amp = PG.rotary_table(dims, 123.0, dict(zip(("factor", "original", "fast", "slow"), yarn)) if yarn else None)
        assert torch.allclose(rope.inv_freq("cpu").double(), freqs, rtol=1e-6) and abs(rope.amplitude - amp) < 1e-12
        pos = [0, 1, 17, 1000, 40000]
        T = len(pos)
        proj = torch.randn(T, H * (D + R) + C + R, generator=g)
        cache = torch.zeros(T, 1, page, C + R, device=DEV)                         # token t goes to page t, slot pos % page
        table = torch.full((T, 40000 // page + 1), -1, dtype=torch.int32)
        for t, p in enumerate(pos):
            table[t, p // page] = t
        q_plain, q_rot = torch.empty(H, T, D, device=DEV), torch.empty(H, T, R, device=DEV)
        w = 1 + 0.1 * torch.randn(C, generator=g)
        A.prepare(proj.to(DEV), 0, H * (D + R), w.to(DEV), 1e-5, rope.inv_freq64(DEV), pairing, rope.amplitude, _i32(pos),
                  _i32(range(T)), table.to(DEV), cache, page, q_plain, q_rot, T, H, D, R, C)
        q = proj[:, :H * (D + R)].double().view(T, H, D + R)
        assert _rel(q_plain.permute(1, 0, 2), q[..., :D]) < 1e-6
        # (the angle is formed in 64-bit and reduced before it is rounded: position 40,000 is as exact as position 1)
        assert torch.allclose(rope.inv_freq64("cpu"), freqs, rtol=1e-14, atol=0)
        assert _rel(q_rot.permute(1, 0, 2), PG.rotate(q[..., D:], torch.tensor(pos), freqs, amp, pairing)) < 2e-6
        row = proj[:, H * (D + R):].double()
        for t, p in enumerate(pos):
            got = cache[t, 0, p % page].cpu()
            assert _rel(got[:C], PG.rms_norm(row[t, :C], w.double(), 1e-5)) < 2e-6
            assert _rel(got[C:], PG.rotate(row[t:t + 1, C:].unsqueeze(1), torch.tensor([p]), freqs, amp, pairing)[0, 0]) < 2e-6


@pytest.mark.parametrize("E,top,groups,keep", [(8, 3, 4, 2), (6, 3, 3, 2), (16, 5, 4, 3), (5, 5, 1, 1), (12, 1, 6, 1), (9, 2, 3, 3), (64, 8, 8, 4), (8, 2, 4, 2)])
def test_routing_with_groups_and_a_correction(E, top, groups, keep):
    """Choice and weights against the plain statement.  The corrections are large and mostly negative, so pick scores
    are negative: a group that is shut out must count as minus infinity, not as 0."""
    from infero_b200.kernels import layer_ops as L
    g = torch.Generator().manual_seed(E * 7 + top)
    z = torch.randn(50, E, generator=g) * 2
    corr = torch.randn(E, generator=g) * 0.5 - 1.0
    idx, w = L.moe_select_grouped(z.to(DEV), corr.to(DEV), E, top, groups, keep)
    want_idx, want_w = PG.route(z.double(), corr.double(), groups, keep, top)
    assert torch.equal(idx.cpu().long(), want_idx)
    assert _rel(w, want_w) < 1e-5
    assert abs(float(w.sum(dim=1).mean()) - 1.0) < 1e-5
    if keep < groups and top > keep:
        # (the best `top` experts lie in at most `top` groups, so groups only bind where more are picked than kept)
        # the plain choice without groups differs: the groups were at work
        other, _ = PG.route(z.double(), corr.double(), 1, 1, top)
        assert not torch.equal(other, want_idx)
    idx0, w0 = L.moe_select_grouped(z.to(DEV), None, E, top, groups, keep)
    want_idx0, want_w0 = PG.route(z.double(), torch.zeros(E, dtype=torch.float64), groups, keep, top)
    assert torch.equal(idx0.cpu().long(), want_idx0) and _rel(w0, want_w0) < 1e-5


def test_the_lowest_index_wins_ties_between_experts_and_between_groups():
    from infero_b200.kernels import layer_ops as L
    z = torch.zeros(2, 8, device=DEV)                          # all scores equal: groups 0 and 1 are kept, experts 0 and 1 picked
    idx, w = L.moe_select_grouped(z, None, 8, 2, 4, 2)
    assert idx.cpu().tolist() == [[0, 1], [0, 1]]
    assert torch.allclose(w.cpu(), torch.full((2, 2), 0.5), atol=1e-6)
    corr = torch.tensor([0, 0, 0, 0, 0, 0, 0.5, 0], dtype=torch.float32, device=DEV)    # group 3 first, then group 0
    idx, _ = L.moe_select_grouped(z, corr, 8, 3, 4, 2)
    assert idx.cpu().tolist() == [[6, 0, 1], [6, 0, 1]]


@pytest.mark.parametrize("dtype,E,top,d,ff,T", [("float32", 6, 2, 40, 12, 9), ("bfloat16", 8, 3, 64, 24, 150), ("bfloat16", 4, 2, 64, 16, 2),
                                               ("bfloat16", 3, 2, 64, 24, 400)])
def test_experts_with_the_clamped_activation_on_all_three_kernels(dtype, E, top, d, ff, T):
    """Streamed (few tokens, 32-bit), warp-level grouped and tcgen05 grouped products, with a limit that clamps a good
    part of the gates and ups, and a shared expert added as it is."""
    from infero_b200.kernels import moe as M
    td = torch.float32 if dtype == "float32" else torch.bfloat16
    g = torch.Generator().manual_seed(E * 10 + top)
    rt = lambda *s, k=1.0: (torch.randn(*s, generator=g) * k).to(td)             # noqa: E731
    h = rt(T, d)
    gate, up, down = rt(E, ff, d, k=0.3), rt(E, ff, d, k=0.3), rt(E, d, ff, k=0.3)
    shared = torch.randn(T, d, generator=g)
    idx = torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(T)]).to(torch.int32)
    w = torch.rand(T, top, generator=g)
    gu = torch.stack([gate, up], dim=2).reshape(E, 2 * ff, d).contiguous().to(DEV)
    y = torch.empty(T, d, device=DEV)
    limit = 0.9
    M.experts(h.to(DEV), gu, down.to(DEV), idx.to(DEV), w.to(DEV), shared.to(DEV), None, y, ("glu_clamped", limit, 1.702))
    want = shared.double().clone()
    for t in range(T):
        for c in range(top):
            e = int(idx[t, c])
            want[t] += w[t, c].double() * PG.clamped_glu(h[t:t + 1].double(), gate[e].double(), up[e].double(), down[e].double(), limit)[0]
    assert _rel(y, want) < (2e-5 if dtype == "float32" else 2e-2)
    assert float(((h.double() @ gate[0].double().T) > limit).float().mean()) > 0.05


class _Latent:
    """One latent-attention mixer over a hand-made paged cache: requests get shuffled pages, portions are fed in
    steps of several requests, and the part runs as the model runs it (a stand-in for the step's context)."""

    def __init__(self, dtype, H, D, R, V, C, d=None, gated=True, pairing="adjacent", page=16, pages=80, seed=0, yarn=None, scale=0.3):
        from infero_b200.config.spec import MixerSpec, PositionSpec
        from infero_b200.parts.latent_attention import LatentAttention
        self.td = torch.float32 if dtype == "float32" else torch.bfloat16
        self.dims = (H, D, R, V, C)
        d = d or max(64, H * V)
        self.d, self.page, self.gated, self.pairing = d, page, gated, pairing
        pos = PositionSpec("rope_interleaved" if pairing == "adjacent" else "rope_neox", 700.0, R, yarn=yarn)
        self.m = {"heads": H, "dim": D, "rot_dim": R, "vdim": V, "kv_rank": C, "scale": scale,
                  "rot": {"base": 700.0, "dims": R, "scaling": dict(zip(("factor", "original", "fast", "slow"), yarn)) if yarn else None}}
        spec = MixerSpec(kind="latent_attention", hidden=d, num_heads=H, num_kv_heads=1, head_dim=D, value_dim=V, rot_dim=R,
                         latent_dim=C, out_gate=gated, scale=scale, position=pos, norm_eps=1e-5, weight_suffix="")
        self.part = LatentAttention(spec, "l0")
        g = torch.Generator().manual_seed(seed)
        self.w = {}
        for decl in self.part.declare():
            t = torch.randn(decl.shape, generator=g) * 0.25
            if decl.role == "norm":
                t = 1 + 0.4 * t
            self.w[decl.name] = t.to(self.td)
        self.w["l0.mix.o"] = torch.eye(d, H * V).to(self.td)            # the heads' results themselves
        self.part.bind({k: v.to(DEV) for k, v in self.w.items()})
        # rows that were never written hold large numbers: a key read from one shows at once
        self.cache = torch.full((pages, 1, page, C + R), 3.0e4, dtype=self.td, device=DEV)
        self.free = [int(p) for p in torch.randperm(pages, generator=g)]
        self.table, self.length = {}, {}

    def plain(self, h):
        return PG.latent_attention(h.double(), {k[3:]: v.double() for k, v in self.w.items()}, "mix", self.m, 1e-5, self.pairing, self.gated)

    def close(self, rid):
        self.free = self.table.pop(rid) + self.free                     # the pages given back are handed out next
        self.length.pop(rid)

    def step(self, entries):
        """entries: (request, rows of the mixer's input); returns request -> result rows."""
        from infero_b200.cache.storage import LayerKv
        E = len(entries)
        tok_entry, positions, q_start, q_len, pos0 = [], [], [], [], []
        for e, (rid, rows) in enumerate(entries):
            n0, n = self.length.get(rid, 0), rows.shape[0]
            pages = self.table.setdefault(rid, [])
            while len(pages) * self.page < n0 + n:
                pages.append(self.free.pop(0))
            q_start.append(len(tok_entry)), q_len.append(n), pos0.append(n0)
            tok_entry += [e] * n
            positions += list(range(n0, n0 + n))
            self.length[rid] = n0 + n
        width = max(len(self.table[rid]) for rid, _ in entries) + 1
        table = torch.full((E, width), -1, dtype=torch.int32)
        for e, (rid, _) in enumerate(entries):
            table[e, :len(self.table[rid])] = torch.tensor(self.table[rid], dtype=torch.int32)
        kv = LayerKv(k=self.cache, v=self.cache[..., :0], group=0, page_size=self.page)
        table = table.to(DEV)
        ctx = types.SimpleNamespace(
            act_dtype=self.td, device=DEV, n_tokens=len(tok_entry), n_entries=E, positions=_i32(positions), tok_entry=_i32(tok_entry),
            entry_q_start=_i32(q_start), entry_q_len=_i32(q_len), entry_pos0=_i32(pos0), h_q_start=np.array(q_start, dtype=np.int32),
            h_q_len=np.array(q_len, dtype=np.int32), h_pos0=np.array(pos0, dtype=np.int32), kv_bound=None,
            max_kv_len=max(p + n for p, n in zip(pos0, q_len)), kv_cache=lambda slot: kv, block_table=lambda group: table)
        h = torch.cat([rows for _, rows in entries]).to(self.td).to(DEV)
        out = self.part.forward(ctx, h, types.SimpleNamespace(cache=0, write_cache=True))
        if hasattr(out, "materialize"):                                   # a product of few rows left as partial sums
            out = out.materialize(torch.float32)
        out = out.float().cpu()
        return {rid: out[q_start[e]:q_start[e] + q_len[e]] for e, (rid, _) in enumerate(entries)}


LATENT_SHAPES = [(2, 8, 4, 6, 12), (3, 16, 16, 24, 64), (4, 32, 32, 32, 64), (2, 64, 64, 64, 128), (1, 5, 2, 7, 9), (16, 16, 8, 8, 32)]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,D,R,V,C", LATENT_SHAPES)
def test_latent_attention_in_portions_and_single_tokens(dtype, H, D, R, V, C):
    """Three requests cut differently (whole, portions down to two tokens, token by token) in shared steps, on shuffled
    pages; a fourth starts on the pages one of them gave back.  Gate on and off, both pairings."""
    for gated, pairing, yarn in ((True, "adjacent", (3.0, 32.0, 8.0, 1.0)), (False, "half", None)):
        # (scores with a spread of a few units: sharp enough to show a wrong key, not so sharp that the rounding of
        # bf16 scores moves the weights by more than the tolerance)
        a = _Latent(dtype, H, D, R, V, C, gated=gated, pairing=pairing, yarn=yarn, seed=H + D, scale=0.6 / math.sqrt(D + R))
        g = torch.Generator().manual_seed(D)
        hs = {r: torch.randn(n, a.d, generator=g) for r, n in (("a", 70), ("b", 37), ("c", 21), ("d", 50))}
        if dtype == "bfloat16":
            hs = {r: v.to(torch.bfloat16).float() for r, v in hs.items()}
        got = {r: [] for r in hs}
        cuts = {"a": [70], "b": [2, 15, 17, 1, 2], "c": [1] * 21}
        at = {r: 0 for r in cuts}
        while any(at[r] < hs[r].shape[0] for r in cuts):
            entries = []
            for r in ("c", "a", "b"):                                   # single tokens first, as the scheduler orders a step
                if at[r] < hs[r].shape[0]:
                    n = cuts[r].pop(0)
                    entries.append((r, hs[r][at[r]:at[r] + n]))
                    at[r] += n
            for r, rows in a.step(entries).items():
                got[r].append(rows)
        a.close("c"), a.close("a")
        got["d"].append(a.step([("d", hs["d"][:33])])["d"])
        got["d"].append(a.step([("d", hs["d"][33:])])["d"])
        tol = 2e-5 if dtype == "float32" else 2.5e-2
        for r in hs:
            assert _rel(torch.cat(got[r]), a.plain(hs[r])) < tol, (r, gated)


@pytest.mark.parametrize("H,D,R,V,C", [(16, 16, 32, 16, 64), (40, 8, 16, 8, 128), (70, 8, 16, 8, 64), (3, 16, 16, 16, 256), (2, 8, 64, 8, 512)])
def test_single_tokens_with_long_contexts_on_the_tensor_core_kernel(H, D, R, V, C):
    """Three requests of 40, 530 and 700 tokens, then single tokens of all three in shared steps: the contexts are cut
    into ranges of keys that are merged afterwards; head counts that fill one, several and not quite whole tiles of rows;
    all latent widths the kernel has instances for."""
    from infero_b200.kernels import latent_mma
    a = _Latent("bfloat16", H, D, R, V, C, gated=True, pairing="half", seed=C + H, scale=0.6 / math.sqrt(D + R), pages=100)
    g = torch.Generator().manual_seed(H)
    hs = {r: torch.randn(n + 6, a.d, generator=g).to(torch.bfloat16).float() for r, n in (("a", 40), ("b", 530), ("c", 700))}
    before = dict(latent_mma.launches)
    got = {r: [rows] for r, rows in a.step([(r, h[:-6]) for r, h in hs.items()]).items()}
    for i in range(6, 0, -1):
        for r, rows in a.step([(r, h[h.shape[0] - i:h.shape[0] - i + 1]) for r, h in hs.items()]).items():
            got[r].append(rows)
    assert latent_mma.launches["tiled"] > before["tiled"] and latent_mma.launches["cut"] >= before["cut"] + 6
    # (queries and softmax weights are bf16 operands of the tensor-core products here, and the maximum runs over up to
    # 560 columns: measured 0.02 to 0.045; a wrong or lost key shows as 0.3 and more)
    for r in hs:
        assert _rel(torch.cat(got[r]), a.plain(hs[r])) < 6e-2, r


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("far", [0, 1, 15, 16, 17, 63, 64, 65, 255, 256, 300, 310])
def test_a_far_key_is_found(dtype, far):
    """One key among hundreds matches the last queries of head 0 (the inputs of those tokens are solved so that the
    plain part of their query points along that key); its value then carries the result.  Keys at the sequence's
    start, on both sides of page and tile borders and far back, read from a prompt portion and from single tokens."""
    H, D, R, V, C = 4, 32, 32, 32, 64
    a = _Latent(dtype, H, D, R, V, C, d=128, gated=False, pairing="half", seed=3, scale=0.2)
    g = torch.Generator().manual_seed(far)
    n = 330
    h = torch.randn(n, a.d, generator=g)
    w = {k[3:]: v.double() for k, v in a.w.items()}
    down = h[far].double() @ w["mix.dkv"].T
    c = PG.rms_norm(down[:C], w["mix.dkv.norm"], 1e-5)
    k0 = (c @ w["mix.uk"].T)[:D]                                         # head 0's plain key at `far`
    wq0 = w["mix.q"][:D + R]                                             # the rows that make head 0's query
    # a score of about 14 for that key, a few units at most for the others; the rotated part of the query is zero
    target = torch.cat([14.0 / (float(k0 @ k0) * 0.2) * k0, torch.zeros(R, dtype=torch.float64)])
    for p in range(n - 12, n):
        if p != far:
            h[p] += (torch.linalg.pinv(wq0) @ (target - wq0 @ h[p].double())).float()
    h = h.to(a.td).float()
    want = a.plain(h)
    first = a.step([("r", h[:n - 8])])["r"]
    rest = [a.step([("r", h[p:p + 1])])["r"] for p in range(n - 8, n)]
    got = torch.cat([first] + rest)
    # (weights that follow exp of scores of 14: a rounding of the scores is passed on in full, and the tensor-core
    # kernel's queries are bf16)
    tol = 6e-5 if dtype == "float32" else 6e-2
    assert _rel(got, want) < tol
    if far < n - 12:
        # without that key the last rows differ by far more than the tolerance
        h2 = h.clone()
        h2[far] = 0.0
        b = _Latent(dtype, H, D, R, V, C, d=128, gated=False, pairing="half", seed=3, scale=0.2)
        assert _rel(b.plain(h2)[-8:, :V], want[-8:, :V]) > 0.4


# ---- whole models through the step function ---------------------------------------------------------------------
def _replay(name, dtype, steps_of, lengths, seed=0, page_size=16, max_seqs=3, tol=None):
    mdir = model_dir(name)
    reqs = make_requests(name, lengths, seed=seed)
    plain = plain_logits(mdir, reqs)
    steps = steps_of(reqs)
    runner = make_runner(mdir, dtype, R.max_live_tokens(steps, reqs), page_size=page_size, max_seqs=max_seqs)
    got = R.replay_inprocess(runner, steps)
    assert len(got) > 0
    worst, where = R.compare(got, plain)
    assert worst <= (tol or TOL[dtype]), f"{name} {dtype}: {worst:.3e} at {where}"
    assert not runner.manager.requests
    return runner


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("E", "bfloat16"), ("B", "float32"), ("C", "float32"), ("D", "float32"),
                                        ("F", "bfloat16"), ("F", "float32")])
def test_whole_prompts(name, dtype):
    _replay(name, dtype, R.steps_whole, [1, 2, 15, 16, 17, 33, 131])


def test_the_residual_after_every_layer():
    """The streams' sum after each layer of a short prompt against the plain statement, in 32-bit (the update a block
    leaves pending is applied first)."""
    from infero_b200.engine import StepEntry
    from infero_b200.parts.block import HyperPreNormBlock
    mdir = model_dir("A")
    toks = make_requests("A", [19], seed=3)["r0"]
    cfg, w = plain_model(mdir)
    _, trail = PG.forward(cfg, w, toks, per_layer=True)
    runner = make_runner(mdir, "float32", 64)
    seen = []
    orig = HyperPreNormBlock.forward

    def spy(self, ctx, x, delta, slot):
        pending = orig(self, ctx, x, delta, slot)
        now = x.clone()
        HyperPreNormBlock.flush(now, pending)
        seen.append(now.sum(dim=1).cpu())
        return pending
    HyperPreNormBlock.forward = spy
    try:
        runner.open("a")
        runner.step([StepEntry("a", toks, [len(toks) - 1])])
    finally:
        HyperPreNormBlock.forward = orig
    assert len(seen) == len(cfg["layers"])
    for i, got in enumerate(seen):
        assert _rel(got, trail[i]) < 1e-5, i


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("E", "bfloat16"), ("B", "float32"), ("C", "float32"), ("F", "bfloat16")])
def test_prompt_then_token_by_token(name, dtype):
    _replay(name, dtype, lambda r: R.steps_tail_decode(r, tail=40), [90, 41, 5])


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("E", "bfloat16"), ("B", "float32"), ("D", "float32"), ("F", "bfloat16")])
def test_portions_down_to_two_tokens(name, dtype):
    _replay(name, dtype, lambda r: R.steps_chunked(r, seed=2), [150, 64, 31])
    _replay(name, dtype, lambda r: R.steps_chunked(r, seed=5, sizes=(1, 2, 1, 3, 2, 16, 1, 15, 17)), [70])


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("E", "bfloat16"), ("B", "float32"), ("C", "float32"), ("F", "bfloat16")])
def test_mixed_batches_with_slots_and_pages_used_again(name, dtype):
    """Three live requests in exactly three request slots: every later request starts in a slot and on pages that an
    ended one gave back."""
    runner = _replay(name, dtype, lambda r: R.steps_mixed(r, seed=4, max_live=3), [120, 33, 80, 17, 64, 95, 2], max_seqs=3)
    assert runner.manager.pages_reused > 0


def test_a_batch_equals_each_request_alone_bitwise_in_32_bit():
    """On the 32-bit path what is computed for a token does not depend on what else is in the step."""
    mdir = model_dir("A")
    reqs = make_requests("A", [50, 21, 37], seed=9)
    together = R.replay_inprocess(make_runner(mdir, "float32", 256, max_seqs=3), [
        {"step": 0, "entries": [{"id": r, "tokens": t, "want": list(range(len(t)))} for r, t in reqs.items()], "end": list(reqs)}])
    alone = R.replay_inprocess(make_runner(mdir, "float32", 256, max_seqs=3), R.steps_whole(reqs))
    assert together.keys() == alone.keys()
    for k in alone:
        assert np.array_equal(together[k], alone[k]), k


def test_three_hundred_single_tokens():
    _replay("B", "float32", lambda r: R.steps_tail_decode(r, tail=300), [310], tol=6e-5)
    _replay("F", "bfloat16", lambda r: R.steps_tail_decode(r, tail=300), [305])


def test_long_prompts_in_large_portions():
    """Portions longer than the tiles of the product and attention kernels, cut beside their edges."""
    def steps(reqs):
        (a, ta), (b, tb) = list(reqs.items())[:2]
        return [{"step": 0, "entries": [{"id": a, "tokens": ta[:257], "want": [0, 127, 128, 129, 255, 256]},
                                        {"id": b, "tokens": tb[:40], "want": [39]}], "end": []},
                {"step": 1, "entries": [{"id": b, "tokens": tb[40:425], "want": [0, 87, 88, 384]},
                                        {"id": a, "tokens": ta[257:258], "want": [0]}], "end": []},
                {"step": 2, "entries": [{"id": a, "tokens": ta[258:], "want": list(range(len(ta) - 258))},
                                        {"id": b, "tokens": tb[425:], "want": list(range(len(tb) - 425))}], "end": [a, b]}]
    _replay("F", "bfloat16", steps, [300, 450], max_seqs=2)
    _replay("A", "float32", steps, [300, 450], max_seqs=2, tol=1e-4)


def test_page_size_64():
    _replay("F", "bfloat16", lambda r: R.steps_mixed(r, seed=1, max_live=2), [130, 70, 64], page_size=64)
    _replay("B", "float32", lambda r: R.steps_mixed(r, seed=1, max_live=2), [130, 70, 64], page_size=64)


# ---- the engine's own entry point --------------------------------------------------------------------------------
def _plain_greedy(cfg, w, prompt, n):
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(PG.forward(cfg, w, toks)[-1].argmax()))
    return toks[len(prompt):]


@pytest.mark.parametrize("name", ["A", "C"])
def test_greedy_generation_through_the_scheduler(name):
    """Several prompts queued at once, more than there are request slots, prompts cut into portions by the
    scheduler's budget, decode steps replayed from captured graphs."""
    from infero_b200.engine import Engine
    from infero_b200.sampling import SamplingParams
    mdir = model_dir(name)
    cfg, w = plain_model(mdir)
    prompts = list(make_requests(name, [19, 40, 3, 27], seed=21).values())
    eng = Engine(mdir, dtype="float32", ctx=128, max_seqs=2, kv_slots=2 * 128, max_batch_tokens=32, cuda_graphs=True)
    params = SamplingParams(temperature=0.0, repetition_penalty=1.0)
    got = eng.generate(prompts, params, max_new_tokens=10, ignore_eos=True)
    for p, g in zip(prompts, got):
        assert g == _plain_greedy(cfg, w, p, 10)
    assert eng.runner.graph_replays > 0


def test_generation_in_bf16_from_captured_graphs_equals_uncaptured_steps():
    from infero_b200.engine import Engine
    from infero_b200.sampling import SamplingParams
    mdir = model_dir("F")
    prompts = list(make_requests("F", [19, 40, 3], seed=22).values())
    params = SamplingParams(temperature=0.0, repetition_penalty=1.0)
    outs = []
    for graphs in (True, False):
        eng = Engine(mdir, dtype="bfloat16", ctx=128, max_seqs=4, kv_slots=4 * 128, max_batch_tokens=64, cuda_graphs=graphs)
        outs.append(eng.generate(prompts, params, max_new_tokens=12, ignore_eos=True))
        if graphs:
            assert eng.runner.graph_replays > 0
    assert outs[0] == outs[1]


def test_the_trace_runner_replays_a_gositar_folder(tmp_path):
    mdir = model_dir("A")
    reqs = make_requests("A", [70, 30], seed=2)
    steps = R.steps_mixed(reqs, seed=3, max_live=2)
    got = R.replay_subprocess(mdir, "float32", steps, R.max_live_tokens(steps, reqs), str(tmp_path), CONFIGS["A"]["vocab"])
    worst, where = R.compare(got, plain_logits(mdir, reqs))
    assert worst <= TOL["float32"], (worst, where)


def test_the_generate_command_line_on_a_gositar_folder():
    """``bin/generate`` as a user runs it: the model is chosen by the folder's config.json."""
    import os
    import subprocess
    import sys
    mdir = model_dir("B")
    cfg, w = plain_model(mdir)
    prompt = make_requests("B", [21], seed=8)["r0"]
    exe = os.path.join(R.ROOT, "bin", "generate")
    proc = subprocess.run([sys.executable, exe, mdir] + [str(t) for t in prompt] +
                          ["--greedy", "--repetition-penalty", "1.0", "-n", "7", "--dtype", "float32", "--ignore-eos",
                           "--max-seq-len", "128"], capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr
    lines = proc.stdout.splitlines()
    at = next(i for i, l in enumerate(lines) if l.startswith("kv cache"))
    toks = [int(t) for t in next(l for l in lines[at + 1:] if l.strip()).split()]
    assert toks == _plain_greedy(cfg, w, prompt, 7)
