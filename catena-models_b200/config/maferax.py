"""Configuration of the Maferax decoder.

config.json is nested: `vocab`, `width`, `norm.eps`, `postln_alpha` (the factor on the stream inside each sum that a
norm follows), `logit_scale`; `layers`, a list whose entries give `type` (which mixer the layer has), `mixer` (its
sizes and constants) and `mlp` (the feed-forward, or null for none).

Mixer types: `gla` (`heads`, `dim`, `vdim`, `tau`; the rank of its decay network is the first dimension of the tensor
`l<i>.mix.a1`, or `rank` for random weights) and `latent_attention` (`heads`, `dim`, `rot_dim`, `vdim`, `kv_rank`,
`q_rank`, `scale`, `rot.dims`, `rot.base`).

Feed-forward kinds: `dense` (`ff`) and `moe` (`expert.ff`; `router.experts`, `router.top`, `router.identity`: experts
without matrices that hand their input through, `router.scale`, `router.groups.count` and `router.groups.keep`).
"""
from __future__ import annotations

import dataclasses

from .base import ConfigError, Reader, base_type, section

MIXER_TYPES = ("gla", "latent_attention")
MLP_KINDS = ("dense", "moe")


@dataclasses.dataclass(frozen=True)
class GatedLinearConfig:
    heads: int
    dim: int
    vdim: int
    tau: float
    rank: int                # 0: taken from the tensors


@dataclasses.dataclass(frozen=True)
class LatentAttentionConfig:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    q_rank: int
    scale: float
    rot_dims: int            # leading channels of the rot_dim part that are turned
    rot_base: float


@dataclasses.dataclass(frozen=True)
class MlpConfig:
    kind: str                # dense | moe
    ff: int
    experts: int = 0         # experts with matrices
    top: int = 0
    identity: int = 0
    scale: float = 1.0
    groups: int = 0          # 0: no groups
    keep: int = 0


@dataclasses.dataclass(frozen=True)
class LayerConfig:
    type: str                # gla | latent_attention
    mixer: object
    mlp: object              # MlpConfig or None
    norm_alone: bool = False # no feed-forward, but the layer's second norm runs all the same (its tensor is there)


@dataclasses.dataclass(frozen=True)
class MaferaxConfig:
    architecture: str
    vocab: int
    width: int
    norm_eps: float
    postln_alpha: float
    logit_scale: float
    layers: tuple
    raw: dict = dataclasses.field(compare=False, default=None)

    @classmethod
    def from_dict(cls, data, where="config.json"):
        r = Reader(data, where)
        arch = r.string("architecture")
        vocab, width = r.integer("vocab", minimum=1), r.integer("width", minimum=1)
        norm = section(r, data, "norm", "")
        eps = norm.number("eps", positive=True) if norm else None
        alpha = r.number("postln_alpha", default=1.0)
        logit_scale = r.number("logit_scale", default=1.0)
        raw_layers = data.get("layers")
        if not isinstance(raw_layers, list) or not raw_layers:
            r.problem("'layers' must be a non-empty list")
            raw_layers = []
        layers = [cls._layer(r, entry, f"layers[{i}].") for i, entry in enumerate(raw_layers)]
        r.finish()
        cfg = cls(arch, vocab, width, eps, alpha, logit_scale, tuple(layers), data)
        cfg.validate(where)
        return cfg

    @staticmethod
    def _layer(r, entry, where):
        if not isinstance(entry, dict) or not isinstance(entry.get("type"), str):
            r.problem(f"'{where}type' must be a string")
            return None
        kind = base_type(entry["type"])
        if kind not in MIXER_TYPES:
            r.problem(f"'{where}type' is '{entry['type']}'; known mixers: {', '.join(MIXER_TYPES)}")
            return None
        m = section(r, entry, "mixer", where)
        mixer = None
        if m and kind == "gla":
            dim = m.integer("dim", minimum=1)
            mixer = GatedLinearConfig(m.integer("heads", minimum=1), dim, m.integer("vdim", default=dim, minimum=1),
                                      m.number("tau", positive=True), m.integer("rank", default=0, minimum=0))
        elif m:
            dim, rot_dim = m.integer("dim", minimum=1), m.integer("rot_dim", default=0, minimum=0)
            rot = section(r, m.data, "rot", where + "mixer.", required=bool(rot_dim))
            mixer = LatentAttentionConfig(m.integer("heads", minimum=1), dim, rot_dim, m.integer("vdim", default=dim, minimum=1),
                                          m.integer("kv_rank", minimum=1), m.integer("q_rank", minimum=1),
                                          m.number("scale", positive=True),
                                          rot.integer("dims", default=rot_dim, minimum=0) if rot else 0,
                                          rot.number("base", positive=True) if rot else 1.0)
        mlp = None
        if entry.get("mlp") is not None:
            f = section(r, entry, "mlp", where)
            kindf = f.string("kind") if f else None
            if kindf == "dense":
                mlp = MlpConfig("dense", f.integer("ff", minimum=1))
            elif kindf == "moe":
                ex, ro = section(r, f.data, "expert", where + "mlp."), section(r, f.data, "router", where + "mlp.")
                if ex and ro:
                    g = section(r, ro.data, "groups", where + "mlp.router.", required=False)
                    mlp = MlpConfig("moe", ex.integer("ff", minimum=1), ro.integer("experts", minimum=1),
                                    ro.integer("top", minimum=1), ro.integer("identity", default=0, minimum=0),
                                    ro.number("scale", default=1.0),
                                    g.integer("count", minimum=1) if g else 0, g.integer("keep", minimum=1) if g else 0)
            elif kindf is not None:
                r.problem(f"'{where}mlp.kind' is '{kindf}'; known: {', '.join(MLP_KINDS)}")
        return LayerConfig(kind, mixer, mlp)

    def validate(self, where="config"):
        from ..parts.recurrent import scan_fits

        problems = []
        for i, layer in enumerate(self.layers):
            if layer is None or layer.mixer is None:
                continue
            m = layer.mixer
            if layer.type == "gla":
                if not scan_fits(m.dim, m.vdim):
                    problems.append(f"layers[{i}]: heads of {m.dim} key channels: the scan kernel takes up to 1024")
            else:
                if m.rot_dims % 2 or m.rot_dims > m.rot_dim:
                    problems.append(f"layers[{i}]: {m.rot_dims} turned channels in a part of {m.rot_dim}")
                if m.kv_rank > 512:
                    problems.append(f"layers[{i}]: latents of {m.kv_rank} channels: the kernels take up to 512")
            f = layer.mlp
            if f is not None and f.kind == "moe":
                outputs = f.experts + f.identity
                if f.top > outputs:
                    problems.append(f"layers[{i}]: top {f.top} of {outputs} router outputs")
                if f.groups and (outputs % f.groups or not 1 <= f.keep <= f.groups or f.keep * (outputs // f.groups) < f.top):
                    problems.append(f"layers[{i}]: {f.groups} groups over {outputs} router outputs, {f.keep} kept, top {f.top}")
        if problems:
            raise ConfigError(f"{where}: " + "; ".join(problems))

    def with_tensor_shapes(self, shapes):
        """The same configuration with what only the tensors give: the decay network's rank, and whether a layer without
        a feed-forward has a second norm (`l<i>.norm2`)."""
        layers = []
        for i, layer in enumerate(self.layers):
            if layer.mlp is None and f"l{i}.norm2" in shapes:
                layer = dataclasses.replace(layer, norm_alone=True)
            if layer.type == "gla" and layer.mixer.rank == 0:
                shape = shapes.get(f"l{i}.mix.a1")
                if shape is None or len(shape) != 2:
                    raise ConfigError(f"layer {i}: the tensor 'l{i}.mix.a1' that gives the decay network's rank is missing")
                layer = dataclasses.replace(layer, mixer=dataclasses.replace(layer.mixer, rank=int(shape[0])))
            layers.append(layer)
        return dataclasses.replace(self, layers=tuple(layers))

    def to_dict(self):
        return self.raw
