"""Reading a Vufizen config.json, lowering it to parts, and the plain statement's own consistency (CPU)."""
import copy

import pytest
import torch

import plain_vufizen as PV
from vufizen_fixtures import A, B, C


def _spec(cfg):
    from infero_b200.registry import resolve_architecture
    arch = resolve_architecture(cfg)
    assert arch.name == "Vufizen"
    return arch.to_spec(arch.read_config(cfg))


def test_the_architecture_is_found_by_its_name_and_lowered_layer_by_layer():
    s = _spec(A)
    assert [b.mixer.kind for b in s.blocks] == ["diff_attention", "hgrn2", "diff_attention"]
    assert [(e.block, e.cache) for e in s.schedule] == [(0, 0), (1, 1), (1, 2), (0, 3), (2, 4)]
    m = s.blocks[0].mixer
    assert (m.num_heads, m.num_kv_heads, m.head_dim, m.v_dim, m.conv_taps, m.position.rotary_dim) == (4, 2, 32, 48, 3, 16)
    assert m.diff == 0.3 and m.scale == 0.25 and m.norm_eps == 2e-5
    assert s.blocks[2].ffn is None and s.blocks[2].mixer.position is None and s.blocks[2].mixer.scale == 1 / 8
    f = s.blocks[0].ffn
    assert (f.experts, f.top, f.intermediate, f.shared_intermediate) == (5, 2, 24, 40)
    assert s.blocks[1].ffn.shared_intermediate == 0
    assert s.final_norm.kind == "rmsnorm_scalar" and (s.embed_name, s.head_name) == ("embed", "head")


def test_declared_tensors_and_what_each_cache_slot_holds():
    from infero_b200.models.decoder import DecoderModel
    m = DecoderModel(_spec(A))
    names = {d.name: tuple(d.shape) for d in m.declare()}
    assert names["l0.mix.q"] == (2 * 4 * 32, 64) and names["l0.mix.k"] == (2 * 2 * 32, 64) and names["l0.mix.v"] == (96, 64)
    assert names["l0.mix.q.conv"] == (256, 3) and names["l0.mix.lq2"] == (32,) and names["l0.norm1"] == ()
    assert names["l1.mix.f.b"] == (32,) and names["l1.mix.norm"] == (32,) and names["l0.mlp.shared.sg"] == (1, 64)
    assert "l1.mlp.shared.gate" not in names and "l4.rg2" not in names and "l4.norm2" not in names and "l4.rg1.b" in names
    assert not any(n.startswith(("l2.", "l3.")) for n in names)         # layers that run on another layer's tensors
    assert sorted(m.kv_specs) == [0, 3, 4] and sorted(m.state_specs) == [0, 1, 2, 3, 4]
    assert m.kv_specs[0].head_dim == 64 and m.kv_specs[0].value_dim == 48 and m.kv_specs[0].num_kv_heads == 2
    assert m.state_specs[1].shape == (2, 16, 32) and m.state_specs[0].shape == (2, 256 + 128 + 96)
    only_recurrent = DecoderModel(_spec(C))
    assert not only_recurrent.kv_specs and len(only_recurrent.state_specs) == 2
    no_conv = DecoderModel(_spec(B))
    assert 2 not in no_conv.state_specs and 1 in no_conv.state_specs


@pytest.mark.parametrize("edit,word", [
    (lambda c: c["layers"][0].update(type="mamba"), "type"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "kv heads"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=34), "rot.dims"),
    (lambda c: c["layers"][2].update(weights_of=0), "differs"),
    (lambda c: c["layers"][2].update(weights_of=9), "weights_of"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=6), "top"),
    (lambda c: c.pop("width"), "width"),
])
def test_configurations_that_cannot_run_are_refused(edit, word):
    from infero_b200.config import ConfigError, VufizenConfig
    c = copy.deepcopy(A)
    edit(c)
    with pytest.raises(ConfigError) as e:
        VufizenConfig.from_dict(c)
    assert word in str(e.value)


def test_plain_recurrence_carries_its_state_and_the_convolution_its_zeros():
    g = torch.Generator().manual_seed(0)
    H, D, V, d, T = 2, 3, 4, 5, 9
    r = lambda *s: torch.randn(*s, generator=g, dtype=torch.float64)      # noqa: E731
    args = (r(H * D, d), r(H * D, d), r(H * D), torch.rand(H * D, generator=g, dtype=torch.float64), r(H * V, d), r(V),
            torch.eye(H * V, dtype=torch.float64), H, D, V, 1e-5)
    h = r(T, d)
    whole, S = PV.hgrn2(h, *args)
    a, Sa = PV.hgrn2(h[:4], *args)
    b, Sb = PV.hgrn2(h[4:], *args, state=Sa)
    assert torch.allclose(torch.cat([a, b]), whole) and torch.allclose(Sb, S)
    u, w = r(6, 3), r(3, 4)
    y = PV.causal_conv(u, w)
    assert torch.allclose(y[0], w[:, 3] * u[0]) and torch.allclose(y[4], (w.T * u[1:5]).sum(0))
    # the rotation turns pairs (0, 1), (2, 3) and leaves the rest
    x = r(2, 1, 6)
    z = PV.rotate_adjacent(x, torch.tensor([0, 3]), 100.0, 4)
    assert torch.equal(z[0], x[0]) and torch.equal(z[1, 0, 4:], x[1, 0, 4:])
    assert torch.allclose(z[1, 0, 0], x[1, 0, 0] * torch.cos(torch.tensor(3.0, dtype=torch.float64)) - x[1, 0, 1] * torch.sin(torch.tensor(3.0, dtype=torch.float64)))
