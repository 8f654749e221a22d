"""Reading a Gositar config.json, its refusals, and the lowering to parts (no GPU)."""
import copy
import math

import pytest
import torch

import plain_gositar as PG
from gositar_fixtures import CONFIGS
from infero_b200.config import ConfigError, GositarConfig
from infero_b200.config.spec import PositionSpec
from infero_b200.models.decoder import DecoderModel
from infero_b200.registry import resolve_architecture


def test_the_architecture_is_chosen_by_name_and_lowered():
    arch = resolve_architecture(CONFIGS["A"])
    assert arch.name == "Gositar"
    cfg = arch.read_config(CONFIGS["A"])
    spec = arch.to_spec(cfg)
    assert spec.streams == 2 and len(spec.blocks) == 4 and all(b.kind == "hyper_prenorm" for b in spec.blocks)
    m0, m1 = spec.blocks[0].mixer, spec.blocks[1].mixer
    assert (m0.kind, m0.out_gate, m0.position.kind, m0.position.yarn) == ("latent_attention", True, "rope_interleaved", (4.0, 24.0, 8.0, 1.0))
    assert (m1.out_gate, m1.position.kind, m1.position.yarn, m1.latent_dim, m1.rot_dim) == (False, "rope_neox", None, 32, 8)
    f0, f1 = spec.blocks[0].ffn, spec.blocks[1].ffn
    assert (f0.kind, f0.experts, f0.top, f0.route_groups, f0.route_keep, f0.limit, f0.shared_limit, f0.activation) == \
        ("moe_grouped", 8, 3, 4, 2, 1.5, 0.8, "glu_clamped")
    assert (f1.kind, f1.intermediate) == ("relu2", 96) and spec.blocks[2].ffn is None
    model = DecoderModel(spec)
    names = {d.name: tuple(d.shape) for d in model.declare()}
    assert names["l0.mix.q"] == (4 * 32, 64) and names["l0.mix.dkv"] == (80, 64) and names["l0.mix.g"] == (4, 64)
    assert "l1.mix.g" not in names and names["l0.hc2.mix"] == (2, 2) and "l2.hc2.in" not in names and "l2.norm2" not in names
    assert names["l0.mlp.correction"] == (8,) and names["l0.mlp.shared.down"] == (64, 40) and names["l1.mlp.up"] == (96, 64)
    # two kinds of cached rows: two groups of pages
    assert sorted({s.head_dim for s in model.kv_specs.values()}) == [40, 80]


def test_a_plain_residual_without_the_streams_key():
    spec = GositarConfig.from_dict(CONFIGS["C"]).to_model_spec()
    assert spec.streams == 0 and all(b.kind == "prenorm" and b.streams == 0 for b in spec.blocks)
    names = {d.name for d in DecoderModel(spec).declare()}
    assert not any(".hc" in n for n in names)
    f = spec.blocks[0].ffn
    assert (f.route_groups, f.route_keep, f.shared_intermediate) == (1, 1, 0)


@pytest.mark.parametrize("edit,word", [
    (lambda c: c["layers"][0].update(type="attention"), "type"),
    (lambda c: c["layers"][0]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=5), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=64), "rot.dims"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=9), "top"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(count=3), "groups"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(keep=1, count=8), "groups"),
    (lambda c: c["layers"][0]["mlp"]["expert"].pop("limit"), "limit"),
    (lambda c: c["layers"][1]["mlp"].update(kind="swiglu"), "kind"),
    (lambda c: c.update(streams=0), "streams"),
    (lambda c: c.update(streams=40), "streams"),
    (lambda c: c["norm"].update(eps=0), "eps"),
    (lambda c: c["layers"][0]["mixer"].update(scale="x"), "scale"),
])
def test_refusals(edit, word):
    c = copy.deepcopy(CONFIGS["A"])
    edit(c)
    with pytest.raises(ConfigError, match=word.replace(".", r"\.")):
        GositarConfig.from_dict(c)


@pytest.mark.parametrize("dims,base,yarn", [(16, 5000.0, (4.0, 24.0, 8.0, 1.0)), (64, 1e6, (8.0, 1024.0, 32.0, 1.0)), (32, 20000.0, (2.0, 1024.0, 32.0, 1.0)),
                                            (2, 9.0, (1.5, 4.0, 2.0, 0.2)), (8, 300.0, None), (12, 50.0, (40.0, 4096.0, 1.0, 1.0))])
def test_rotary_tables_with_stretched_frequencies(dims, base, yarn):
    from infero_b200.parts.rope import RopeNeox
    rope = RopeNeox(PositionSpec("rope_neox", base, dims, yarn=yarn))
    freqs, amp = PG.rotary_table(dims, base, dict(zip(("factor", "original", "fast", "slow"), yarn)) if yarn else None)
    assert torch.allclose(rope.inv_freq("cpu").double(), freqs, rtol=2e-7, atol=0)
    assert abs(rope.amplitude - amp) < 1e-12
    if yarn:
        assert amp == 0.1 * math.log(yarn[0]) + 1.0
        plain = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=torch.float64)
        assert (freqs <= plain + 1e-18).all() and (freqs >= plain / yarn[0] - 1e-18).all()


def test_mixers_without_an_amplitude_refuse_stretched_tables():
    from infero_b200.config.spec import MixerSpec
    from infero_b200.parts.attention import GqaAttention
    pos = PositionSpec("rope_neox", 1e4, 16, yarn=(4.0, 64.0, 8.0, 1.0))
    with pytest.raises(ValueError, match="amplitude"):
        GqaAttention(MixerSpec(kind="gqa_attention", hidden=32, num_heads=2, num_kv_heads=2, head_dim=16, scale=0.25, position=pos), "l0")


def test_a_model_folder_is_written_and_read_back(tmp_path):
    from infero_b200.loading import write_random_model_dir
    from infero_b200.registry import load_config
    write_random_model_dir(str(tmp_path), CONFIGS["B"], seed=1, std=0.1, norm_std=0.1)
    arch, cfg, spec = load_config(str(tmp_path))
    assert arch.name == "Gositar" and cfg.streams == 3 and spec.blocks[0].mixer.position.rotary_dim == 2
    import plain_qwen2
    raw, w = plain_qwen2.read_model(str(tmp_path))
    assert raw["streams"] == 3 and tuple(w["l0.hc1.mix"].shape) == (3, 3)
    # the mixing matrices start near the identity, the read-in and write-out weights near one
    assert float((w["l0.hc1.mix"] - torch.eye(3, dtype=torch.float64)).abs().max()) < 0.6
    logits = PG.forward(raw, w, [1, 2, 3, 4, 5])
    assert tuple(logits.shape) == (5, 97) and torch.isfinite(logits).all()
