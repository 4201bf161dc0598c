"""Small Relilix configurations for the tests, and weights for them that make a fault visible.

The configurations differ from each other in every size, in the order and kinds of layers and in the constants; sizes
that could hide a fault by being equal (query and key/value heads, latent and query ranks, value and key sizes of the
latent layers) or by being 1 (heads, key/value heads, top, taps, groups of one expert, a factor of 1) take both forms,
and what a configuration may leave out (the window, the cap, the taps, the rotation, its rescaling, the groups, the
shared expert, a feed-forward) is left out somewhere.  Weights are drawn so that activations are of order one and
scores reach the cap; corrections are large enough to change the choice of experts.  Everything is stored in bfloat16,
as a checkpoint is.
"""
import hashlib
import json
import os

import torch


def rot(dims, base, scaling=None):
    r = dict(dims=dims, base=base)
    if scaling:
        r["scaling"] = dict(factor=scaling[0], original=scaling[1], fast=scaling[2], slow=scaling[3])
    return r


def attention(heads, kv_heads, dim, conv, window, scale, softcap, rotation, mlp):
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=dim, scale=scale)
    if conv:
        m["conv"] = conv
    if window:
        m["mask"] = dict(size=window)
    if softcap:
        m["softcap"] = softcap
    if rotation:
        m["rot"] = rotation
    return dict(type="attention", mixer=m, mlp=mlp)


def latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, rotation, mlp, kv_from=None):
    m = dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=kv_rank, q_rank=q_rank, scale=scale, rot=rotation)
    if kv_from is not None:
        m["kv_from"] = kv_from
    return dict(type="latent_attention", mixer=m, mlp=mlp)


def dense(ff):
    return dict(kind="dense", ff=ff)


def moe(ff, limit, experts, top, groups=None, shared=None):
    router = dict(experts=experts, top=top)
    if groups:
        router["groups"] = dict(count=groups[0], keep=groups[1])
    f = dict(kind="moe", expert=dict(ff=ff, limit=limit), router=router)
    if shared:
        f["shared"] = dict(ff=shared[0], limit=shared[1])
    return f


def model(vocab, width, eps, emb_scale, layers):
    return dict(architecture="Relilix", vocab=vocab, width=width, norm=dict(eps=eps), embedding=dict(scale=emb_scale),
                layers=layers)


YARN_A = (4.0, 64, 16.0, 2.0)

# A: both mixers twice; fewer key/value heads than heads; a window shorter than a page; a latent layer that reads the
# latents of an earlier one; groups of two experts of which two of three stay open; a shared expert wider than the others
TINY_A = model(150, 64, 1e-5, 3.0, [
    attention(4, 2, 16, 3, 20, 0.3, 4.0, rot(8, 1000.0), dense(96)),
    latent(3, 16, 8, 24, 40, 24, 0.2, rot(8, 300.0, YARN_A), moe(32, 1.2, 6, 2, groups=(3, 2), shared=(48, 2.0))),
    attention(4, 2, 16, 3, 20, 0.3, 4.0, rot(8, 1000.0), moe(24, 0.8, 4, 3, shared=(16, 0.5))),
    latent(3, 16, 8, 24, 40, 24, 0.2, rot(8, 300.0, YARN_A), dense(48), kv_from=1)])

# B: sizes that are multiples of nothing convenient; a latent layer first; one head; heads that need padding; two taps; a
# window of seven; one expert per token, no groups, no shared expert; a layer without feed-forward; no rescaling
TINY_B = model(77, 36, 1e-6, 1.0, [
    latent(1, 12, 6, 20, 21, 10, 0.3, rot(6, 500.0), moe(20, 3.0, 3, 1)),
    attention(3, 3, 12, 2, 7, 0.4, 2.5, rot(4, 50.0), None),
    attention(2, 1, 20, 5, 70, 0.25, 6.0, rot(20, 10000.0), dense(28))])

# C: what may be left out is left out: no taps, no window, no cap, no rotation; one key/value head; groups of one expert,
# all groups open; a rescaling factor of 1; value and key heads of one size in the latent layer
TINY_C = model(96, 32, 1e-6, 0.5, [
    attention(2, 1, 8, 0, 0, 0.35, 0.0, None, moe(16, 1.0, 4, 2, groups=(4, 4), shared=(8, 1.0))),
    latent(2, 8, 4, 8, 16, 16, 0.35, rot(4, 100.0, (1.0, 32, 8.0, 1.0)), dense(64)),
    attention(4, 4, 8, 4, 64, 0.3, 3.0, rot(8, 100.0), None),
    latent(4, 8, 4, 16, 16, 8, 0.25, rot(4, 100.0, (1.0, 32, 8.0, 1.0)), None, kv_from=1)])

# M: sizes that the tensor-core kernels take (heads of 64 and 128, a width that is a multiple of 8); a window longer
# than a page and shorter than two
TINY_M = model(210, 128, 1e-6, 2.0, [
    attention(4, 2, 64, 4, 96, 0.125, 8.0, rot(32, 5000.0), dense(256)),
    latent(4, 32, 16, 64, 64, 48, 0.15, rot(16, 5000.0, (8.0, 128, 16.0, 1.0)), moe(64, 1.0, 8, 2, groups=(4, 2), shared=(128, 1.5))),
    attention(2, 1, 128, 3, 130, 0.09, 10.0, rot(64, 100000.0), moe(64, 2.0, 6, 3, groups=(2, 1))),
    latent(4, 32, 16, 64, 64, 48, 0.15, rot(16, 5000.0, (8.0, 128, 16.0, 1.0)), dense(192), kv_from=1)])

# L: a window of hundreds of tokens (the long-prompt attention kernels), with and without a window
TINY_L = model(120, 64, 1e-6, 1.5, [
    attention(2, 1, 64, 3, 800, 0.125, 6.0, rot(16, 10000.0), dense(64)),
    attention(2, 2, 64, 2, 0, 0.125, 5.0, rot(64, 10000.0), None)])

# one mechanism at a time
ONLY_ATTENTION = model(64, 32, 1e-6, 1.0, [attention(4, 2, 16, 4, 24, 0.3, 3.0, rot(16, 200.0), None)])
ONLY_LATENT = model(64, 32, 1e-6, 1.0, [latent(4, 16, 8, 24, 24, 12, 0.25, rot(8, 200.0, (2.0, 48, 8.0, 1.0)), None)])
ONLY_MOE = model(64, 24, 1e-6, 1.0, [attention(1, 1, 8, 0, 0, 0.3, 0.0, None, moe(16, 0.7, 8, 3, groups=(4, 2), shared=(24, 1.1)))])
# ... and a filter of one tap: a factor per channel, no state
ONLY_DENSE = model(64, 24, 1e-6, 2.0, [attention(1, 1, 8, 1, 0, 0.3, 0.0, None, dense(56))])

ALL = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "M": TINY_M, "L": TINY_L, "attention": ONLY_ATTENTION,
       "latent": ONLY_LATENT, "moe": ONLY_MOE, "dense": ONLY_DENSE}


def _gen(seed, name):
    g = torch.Generator()
    g.manual_seed(int.from_bytes(hashlib.sha256(f"{seed}:{name}".encode()).digest()[:8], "little") & ((1 << 63) - 1))
    return g


def make_tensors(config, seed):
    """{name: bfloat16 tensor} for a configuration dict."""
    from catena_models_b200.config.registry import config_from_dict

    arch, typed = config_from_dict(config)
    scale = (config.get("embedding") or {}).get("scale", 1.0)
    out = {}
    for spec in arch.define(typed).tensor_specs():
        g, name, shape = _gen(seed, spec.name), spec.name, tuple(spec.shape)
        n = lambda std=1.0: torch.randn(shape, generator=g) * std
        tail = name.split(".")[-1]
        if tail in ("norm1", "norm2") or name == "final.norm":
            t = 1.0 + 0.3 * torch.rand(shape, generator=g)
        elif tail == "norm":
            t = 1.0 + n(0.1)
        elif tail == "conv":
            t = n(0.6)
        elif tail == "correction":
            t = n(0.15)
        elif tail == "router":
            t = n(2.0 / shape[-1] ** 0.5)
        elif name == "embed":
            t = n(1.0 / scale)
        elif tail in ("q", "k", "uq"):
            t = n(1.6 / shape[-1] ** 0.5)              # scores that reach the cap
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
