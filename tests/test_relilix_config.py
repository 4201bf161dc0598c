"""Reading a Relilix config.json: every size and constant lands in the typed configuration, what may be left out gets
its neutral value, what the kernels cannot run or what contradicts itself is refused when the file is read, and the
definition names exactly the tensors that the layers need."""
import copy

import pytest

import tiny_relilix as tiny
from catena_models_b200.config.base import ConfigError
from catena_models_b200.config.registry import config_from_dict


def test_fields_of_every_layer():
    arch, cfg = config_from_dict(tiny.TINY_A)
    assert arch.name == "Relilix" and (cfg.vocab, cfg.width, cfg.norm_eps, cfg.embedding_scale) == (150, 64, 1e-5, 3.0)
    a, l, a2, l2 = cfg.layers
    assert (a.type, a.mixer.heads, a.mixer.kv_heads, a.mixer.dim, a.mixer.taps, a.mixer.window) == ("attention", 4, 2, 16, 3, 20)
    assert (a.mixer.scale, a.mixer.softcap, a.mixer.rot.dims, a.mixer.rot.base, a.mixer.rot.factor) == (0.3, 4.0, 8, 1000.0, None)
    assert (a.mlp.kind, a.mlp.ff) == ("dense", 96)
    m = l.mixer
    assert (l.type, m.heads, m.dim, m.rot_dim, m.vdim, m.kv_rank, m.q_rank, m.scale, m.kv_from) == ("latent_attention", 3, 16, 8, 24, 40, 24, 0.2, None)
    assert (m.rot.factor, m.rot.original, m.rot.fast, m.rot.slow) == tiny.YARN_A
    f = l.mlp
    assert (f.kind, f.ff, f.limit, f.experts, f.top, f.groups, f.keep) == ("moe", 32, 1.2, 6, 2, 3, 2)
    assert (f.shared.ff, f.shared.limit) == (48, 2.0)
    assert (a2.mlp.groups, a2.mlp.keep, a2.mlp.shared.ff) == (0, 0, 16)
    assert l2.mixer.kv_from == 1


def test_what_may_be_left_out():
    _, cfg = config_from_dict(tiny.TINY_C)
    a = cfg.layers[0].mixer
    assert (a.taps, a.window, a.softcap, a.rot) == (0, 0, 0.0, None)
    arch, d = config_from_dict(tiny.ONLY_DENSE)
    assert d.layers[0].mixer.taps == 1 and {s.name: tuple(s.shape) for s in arch.define(d).tensor_specs()}["l0.mix.k.conv"] == (8, 1)
    assert cfg.layers[2].mlp is None
    _, b = config_from_dict(tiny.TINY_B)
    assert b.layers[0].mlp.shared is None and b.layers[0].mlp.groups == 0


def test_the_definition_names_the_layers_tensors():
    arch, cfg = config_from_dict(tiny.TINY_A)
    names = {s.name: tuple(s.shape) for s in arch.define(cfg).tensor_specs()}
    assert names["l0.mix.q.conv"] == (64, 3) and names["l0.mix.k.conv"] == (32, 3) and "l0.mix.v" not in names
    assert names["l1.mix.dkv"] == (48, 64) and names["l1.mix.dkv.norm"] == (40,)
    assert "l3.mix.dkv" not in names and "l3.mix.dkv.norm" not in names and names["l3.mix.uk"] == (48, 40)
    assert names["l1.mlp.correction"] == (6,) and names["l1.mlp.shared.gate"] == (48, 64) and names["l1.mlp.e5.down"] == (64, 32)
    _, c = config_from_dict(tiny.TINY_C)
    assert not any(n.endswith(".conv") for n in (s.name for s in arch.define(c).tensor_specs() if s.name.startswith("l0.")))
    plan = arch.define(cfg).plan
    assert (plan[3].state, plan[3].owns_state) == (1, False) and all(e.owns_state for e in plan[:3])


def _with(path, value, base=None):
    cfg = copy.deepcopy(base or tiny.TINY_A)
    node = cfg
    for key in path[:-1]:
        node = node[key]
    node[path[-1]] = value
    return cfg


@pytest.mark.parametrize("path, value, text", [
    (("layers", 0, "mixer", "kv_heads"), 3, "kv_heads"),
    (("layers", 0, "mixer", "vdim"), 24, "values are the keys"),
    (("layers", 0, "mixer", "conv"), 99, "taps"),
    (("layers", 0, "mixer", "rot", "dims"), 18, "turned channels"),
    (("layers", 0, "mixer", "softcap"), -1.0, "softcap"),
    (("layers", 1, "mixer", "rot", "dims"), 10, "turned channels"),
    (("layers", 1, "mlp", "router", "top"), 7, "top"),
    (("layers", 1, "mlp", "router", "groups", "keep"), 4, "groups"),
    (("layers", 1, "mlp", "router", "groups", "count"), 4, "groups"),
    (("layers", 3, "mixer", "kv_from"), 0, "kv_from"),
    (("layers", 3, "mixer", "kv_from"), 3, "kv_from"),
    (("layers", 3, "mixer", "kv_rank"), 32, "differ"),
    (("layers", 0, "type"), "conv", "known mixers"),
    (("layers", 0, "mlp", "kind"), "sparse", "known"),
    (("width",), "wide", "integer"),
])
def test_refused_when_read(path, value, text):
    with pytest.raises(ConfigError) as e:
        config_from_dict(_with(path, value))
    assert text in str(e.value)


def test_rescaled_rates_follow_the_rule():
    """The rates of a rescaled rotation: unchanged below `lo`, divided by the factor above `hi`, a blend between."""
    import math

    from catena_models_b200.parts import build_part

    dims, base, factor, original, fast, slow = 16, 5000.0, 8.0, 128, 16.0, 1.0
    part = build_part("position", "paired_rotary", dims=dims, theta=base, factor=factor, original=original, fast=fast, slow=slow)
    where = lambda t: dims * math.log(original / (2.0 * math.pi * t)) / (2.0 * math.log(base))
    lo, hi = max(math.floor(where(fast)), 0), min(math.ceil(where(slow)), dims - 1)
    for i, rate in enumerate(part.rates):
        f = base ** (-2.0 * i / dims)
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        assert rate == pytest.approx(f / factor * ramp + f * (1.0 - ramp), rel=1e-12)
    assert part.magnitude == pytest.approx(0.1 * math.log(factor) + 1.0)
    plain_part = build_part("position", "paired_rotary", dims=dims, theta=base)
    assert plain_part.magnitude == 1.0 and plain_part.rates[3] == pytest.approx(base ** (-6.0 / dims))
