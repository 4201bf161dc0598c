"""The Maferax configuration reader and definition, and the plain statement against itself (no device needed)."""
import copy

import pytest
import torch

import plain_maferax as plain
import tiny_maferax as tiny
from catena_models_b200.cache.spec import FixedStateSpec, KVStateSpec
from catena_models_b200.config.base import ConfigError
from catena_models_b200.config.registry import config_from_dict


def test_reads_every_size_and_constant():
    arch, cfg = config_from_dict(tiny.TINY_B)
    assert arch.name == "Maferax" and cfg.vocab == 77 and cfg.width == 36
    assert (cfg.norm_eps, cfg.postln_alpha, cfg.logit_scale) == (1e-6, 1.0, 1.0)
    att, lin = cfg.layers[0], cfg.layers[1]
    m = att.mixer
    assert att.type == "latent_attention"
    assert (m.heads, m.dim, m.rot_dim, m.vdim, m.kv_rank, m.q_rank, m.scale, m.rot_dims, m.rot_base) == (1, 12, 6, 20, 21, 10, 0.3, 4, 500.0)
    assert (att.mlp.kind, att.mlp.ff, att.mlp.experts, att.mlp.top, att.mlp.identity, att.mlp.scale, att.mlp.groups) == ("moe", 20, 3, 1, 0, 1.0, 0)
    assert lin.type == "gla" and lin.mlp is None and (lin.mixer.heads, lin.mixer.dim, lin.mixer.vdim, lin.mixer.tau) == (1, 12, 20, 1.0)
    _, cfg = config_from_dict(tiny.TINY_A)
    f = cfg.layers[1].mlp
    assert (f.experts, f.top, f.identity, f.scale, f.groups, f.keep) == (6, 3, 2, 1.5, 4, 2)
    assert cfg.postln_alpha == 2.0 and cfg.logit_scale == 0.5


def test_definition_states_tensors_and_depth():
    arch, cfg = config_from_dict(tiny.TINY_A)
    d = arch.define(cfg)
    specs = d.state_specs()
    assert specs[0] == FixedStateSpec((2 * 16 * 24,), "float32")
    assert specs[1] == KVStateSpec(1, 48, 0, planes=1)               # a latent of 40 and a turned part of 8 per token
    assert d.depth_entries == 5 and d.residual_float32 and d.logit_scale == 0.5
    shapes = {s.name: tuple(s.shape) for s in d.tensor_specs()}
    assert shapes["embed.norm"] == () and shapes["l2.norm2"] == () and shapes["l3.dwa"] == (5,) and shapes["l0.dwa"] == (2,)
    assert shapes["l1.mlp.router"] == (8, 64) and shapes["l1.mlp.correction"] == (8,)
    assert "l1.mlp.e5.down" in shapes and "l1.mlp.e6.down" not in shapes          # identity experts have no tensors
    assert shapes["l1.mix.dkv"] == (48, 64) and shapes["l1.mix.uk"] == (48, 40) and shapes["l1.mix.uv"] == (72, 40)
    assert shapes["l1.mix.g"] == (3, 64) and shapes["l0.mix.g"] == (48, 64) and shapes["l0.mix.a2.b"] == (32,)
    # a layer without feed-forward has no second norm unless its tensor is there
    arch, cfg = config_from_dict(tiny.TINY_B)
    names = {s.name for s in arch.define(cfg).tensor_specs()}
    assert "l1.norm2" not in names and "l1.norm1" in names
    names = {s.name for s in arch.define(cfg.with_tensor_shapes({"l1.norm2": (), "l1.mix.a1": (5, 36), "l2.mix.a1": (4, 36)})).tensor_specs()}
    assert "l1.norm2" in names


def test_rank_comes_from_the_tensors():
    cfg = copy.deepcopy(tiny.TINY_B)
    for layer in cfg["layers"]:
        layer["mixer"].pop("rank", None)
    arch, typed = config_from_dict(cfg)
    with pytest.raises(ValueError):
        arch.define(typed)
    typed = typed.with_tensor_shapes({"l1.mix.a1": (5, 36), "l2.mix.a1": (4, 36)})
    assert [l.mixer.rank for l in typed.layers[1:]] == [5, 4]
    arch.define(typed)


@pytest.mark.parametrize("change, words", [
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=10), "turned"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=3), "turned"),
    (lambda c: c["layers"][1]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=9), "top"),
    (lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(count=3), "groups"),
    (lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(keep=1), "groups"),
    (lambda c: c["layers"][0]["mixer"].update(tau=0.0), "tau"),
    (lambda c: c["layers"][2].update(type="other"), "known mixers"),
    (lambda c: c["layers"][0]["mlp"].update(kind="sparse"), "mlp.kind"),
    (lambda c: c.pop("width"), "width"),
])
def test_refuses_what_cannot_run(change, words):
    cfg = copy.deepcopy(tiny.TINY_A)
    change(cfg)
    with pytest.raises(ConfigError) as e:
        config_from_dict(cfg)
    assert words in str(e.value)


def test_paired_rates():
    from catena_models_b200.parts import build_part

    for dims, base in ((16, 20000.0), (4, 500.0), (2, 100.0)):
        part = build_part("position", "paired_rotary", dims=dims, theta=base)
        assert part.rates == pytest.approx([base ** (-2.0 * i / dims) for i in range(dims // 2)], rel=1e-12)
        assert part.pairing == "interleaved"


def test_plain_statement_in_portions_equals_whole():
    """The plain implementation carries its own states: a prompt in portions gives what the whole prompt gives."""
    import tempfile

    with tempfile.TemporaryDirectory() as tmp:
        cfg, P = tiny.load_plain(tiny.make_folder(tmp, "A", seed=3))
    tokens = tiny.prompt(40, cfg["vocab"], 5)
    whole, _, streams = plain.forward(tokens, P, cfg)
    assert streams.shape == (4, 40, 64)
    got, states, at = [], None, 0
    for n in (7, 1, 2, 30):
        logits, states, _ = plain.forward(tokens[at:at + n], P, cfg, p0=at, states=states)
        got.append(logits)
        at += n
    assert float((torch.cat(got) - whole).abs().max()) < 1e-9
    # the choice of experts honours groups: every chosen expert lies in one of the `keep` best groups
    h = torch.randn(50, 64, dtype=torch.float64, generator=torch.Generator().manual_seed(1))
    r = cfg["layers"][1]["mlp"]["router"]
    ids, w = plain.route(h, P, "l1.mlp.", r)
    assert all(len({i // 2 for i in row}) <= 2 for row in ids.tolist())
    assert torch.allclose(w.sum(-1), torch.full((50,), 1.5, dtype=torch.float64))
