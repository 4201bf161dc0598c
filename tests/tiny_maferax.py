"""Small Maferax configurations for the tests, and weights for them that make a fault visible.

The configurations differ from each other in every size, in the order and kinds of layers and in the constants;
sizes that could hide a fault by being equal (key and value head sizes, the turned part and the channels that are
really turned, latent and query ranks) or by being 1 (heads, top, groups, tau, the factors) take both forms.
Weights are drawn so that activations are of order one: matrices N(0, 1/in), norms with one number near one, depth
coefficients that keep every earlier layer visible, corrections large enough to change the choice of experts.
Everything is stored in bfloat16, as a checkpoint is.
"""
import hashlib
import json
import os

import torch


def gla(heads, dim, vdim, tau, rank, mlp):
    return dict(type="gla", mlp=mlp, mixer=dict(heads=heads, dim=dim, vdim=vdim, tau=tau, rank=rank))


def latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, rot_dims=None, base=10000.0, mlp=None):
    return dict(type="latent_attention", mlp=mlp,
                mixer=dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=kv_rank, q_rank=q_rank, scale=scale,
                           rot=dict(dims=rot_dim if rot_dims is None else rot_dims, base=base)))


def dense(ff):
    return dict(kind="dense", ff=ff)


def moe(ff, experts, top, identity=0, scale=1.0, groups=None):
    router = dict(experts=experts, top=top, identity=identity, scale=scale)
    if groups:
        router["groups"] = dict(count=groups[0], keep=groups[1])
    return dict(kind="moe", expert=dict(ff=ff), router=router)


def model(vocab, width, eps, alpha, logit_scale, layers):
    return dict(architecture="Maferax", vocab=vocab, width=width, norm=dict(eps=eps), postln_alpha=alpha,
                logit_scale=logit_scale, layers=layers)


# A: both mixers twice, value heads larger than key heads, a router with groups, a correction and identity experts
TINY_A = model(150, 64, 1e-5, 2.0, 0.5, [
    gla(2, 16, 24, 8.0, 8, dense(96)),
    latent(3, 16, 8, 24, 40, 24, 0.2, mlp=moe(32, 6, 3, identity=2, scale=1.5, groups=(4, 2))),
    latent(3, 16, 8, 24, 40, 24, 0.2, mlp=dense(48)),
    gla(2, 16, 24, 8.0, 8, moe(24, 4, 2, identity=1, scale=0.5))])

# B: sizes that are multiples of nothing convenient; attention first; one head; only part of the turned part is turned;
# entries of the cache that need padding; one expert per token; tau 1, factor 1, scale 1; a layer without feed-forward
TINY_B = model(77, 36, 1e-6, 1.0, 1.0, [
    latent(1, 12, 6, 20, 21, 10, 0.3, rot_dims=4, base=500.0, mlp=moe(20, 3, 1)),
    gla(1, 12, 20, 1.0, 5, None),
    gla(3, 4, 12, 3.0, 4, dense(28))])

# C: key and value heads of one size, a turned part of one pair, one group that holds everything, more identity experts
# than real ones, a decay network wide enough for the runtime's products
TINY_C = model(96, 32, 1e-6, 3.0, 0.25, [
    latent(2, 8, 2, 8, 16, 16, 0.35, base=100.0, mlp=moe(16, 1, 2, identity=3, scale=2.0, groups=(1, 1))),
    gla(2, 8, 8, 4.0, 32, dense(64)),
    latent(4, 8, 4, 16, 24, 8, 0.25, base=100.0, mlp=None)])

# M: sizes that the tensor-core kernels take (multiples of 16, a width that is a multiple of 8)
TINY_M = model(210, 128, 1e-6, 2.5, 0.5, [
    gla(2, 32, 64, 16.0, 16, dense(256)),
    latent(4, 32, 16, 64, 64, 48, 0.15, base=5000.0, mlp=moe(64, 8, 2, groups=(2, 1))),
    latent(4, 32, 16, 64, 64, 48, 0.15, base=5000.0, mlp=dense(192)),
    gla(4, 16, 32, 2.0, 16, moe(64, 6, 4, identity=2, scale=2.0, groups=(4, 3)))])

# one mechanism at a time
ONLY_GLA = model(64, 40, 1e-6, 1.0, 1.0, [gla(2, 24, 40, 6.0, 6, None)])
ONLY_LATENT = model(64, 32, 1e-6, 1.0, 1.0, [latent(4, 16, 8, 24, 24, 12, 0.25, mlp=None)])
ONLY_MOE = model(64, 24, 1e-6, 1.5, 1.0, [gla(1, 8, 8, 2.0, 4, moe(16, 5, 2, identity=3, scale=1.2, groups=(4, 2)))])
ONLY_DENSE = model(64, 24, 1e-6, 0.8, 1.0, [gla(1, 8, 8, 2.0, 4, dense(56))])

ALL = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "M": TINY_M, "gla": ONLY_GLA, "latent": ONLY_LATENT, "moe": ONLY_MOE,
       "dense": ONLY_DENSE}


def _gen(seed, name):
    g = torch.Generator()
    g.manual_seed(int.from_bytes(hashlib.sha256(f"{seed}:{name}".encode()).digest()[:8], "little") & ((1 << 63) - 1))
    return g


def make_tensors(config, seed):
    """{name: bfloat16 tensor} for a configuration dict."""
    from catena_models_b200.config.registry import config_from_dict

    arch, typed = config_from_dict(config)
    out = {}
    for spec in arch.define(typed).tensor_specs():
        g, name, shape = _gen(seed, spec.name), spec.name, tuple(spec.shape)
        n = lambda std=1.0: torch.randn(shape, generator=g) * std
        tail = name.split(".")[-1]
        if tail in ("norm1", "norm2") or name in ("final.norm", "embed.norm"):
            t = 1.0 + 0.3 * torch.rand(shape, generator=g)
        elif tail == "norm":
            t = 1.0 + n(0.1)
        elif tail == "dwa":
            t = 0.2 + 0.5 * torch.rand(shape, generator=g)
            t[-1] = 1.0
        elif tail == "b":
            t = 1.5 + n(1.0)                     # decays spread between fast and slow
        elif tail == "correction":
            t = n(0.15)
        elif tail == "router":
            t = n(2.0 / shape[-1] ** 0.5)
        elif name == "embed":
            t = n(1.0)
        else:
            t = n(1.0 / shape[-1] ** 0.5)
        out[name] = t.to(torch.bfloat16)
    return out


def make_folder(tmp, name, seed=0, config=None, tensors=None):
    from catena_models_b200.weights.safetensors_io import write_safetensors

    config = config or ALL[name]
    folder = os.path.join(str(tmp), name)
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as fh:
        json.dump(config, fh)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors or make_tensors(config, seed))
    return folder


def load_plain(folder):
    """(config dict, {name: float64 tensor}) as the plain implementation takes them."""
    from catena_models_b200.weights.safetensors_io import SafetensorsFile

    with open(os.path.join(folder, "config.json")) as fh:
        cfg = json.load(fh)
    f = SafetensorsFile(os.path.join(folder, "model.safetensors"))
    tensors = {n: f.tensor(n).clone().to(torch.float64) for n in f.names()}
    f.close()
    return cfg, tensors


def prompt(n, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()
