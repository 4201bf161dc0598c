"""Configuration of the Relilix decoder.

config.json is nested: `vocab`, `width`, `norm.eps`, `embedding.scale` (the factor on every embedding row); `layers`,
a list whose entries give `type` (which mixer the layer has), `mixer` (its sizes and constants) and `mlp` (the
feed-forward, or null for none).

Mixer types: `attention` (`heads`, `kv_heads`, `dim`, `vdim`, `conv`: taps of the short filter behind the query and
key projections, `scale`, `softcap`, `mask.size`: the sliding window, `rot.dims`, `rot.base`; the values are the keys
before their rotation, so `vdim` equals `dim`) and `latent_attention` (`heads`, `dim`, `rot_dim`, `vdim`, `kv_rank`,
`q_rank`, `scale`, `rot.dims`, `rot.base`, `rot.scaling.{factor, original, fast, slow}`, and optionally `kv_from`: the
layer whose cached latents this layer reads instead of making its own).

Feed-forward kinds: `dense` (`ff`) and `moe` (`expert.ff`, `expert.limit`; `router.experts`, `router.top`,
`router.groups.count`, `router.groups.keep`; `shared.ff`, `shared.limit`: an expert that every token runs, or absent).
"""
from __future__ import annotations

import dataclasses

from ..csrc import limits
from .base import ConfigError, Reader, base_type, section

MIXER_TYPES = ("attention", "latent_attention")
MLP_KINDS = ("dense", "moe")


@dataclasses.dataclass(frozen=True)
class RotationConfig:
    dims: int
    base: float
    factor: object           # None: the rates are not rescaled
    original: float
    fast: float
    slow: float


@dataclasses.dataclass(frozen=True)
class AttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    taps: int                # 0: no filter and no filter tensors; 1: one tap, a factor per channel
    scale: float
    softcap: float           # 0: none
    window: int              # 0: every earlier position is seen
    rot: object              # RotationConfig or None


@dataclasses.dataclass(frozen=True)
class LatentAttentionConfig:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    q_rank: int
    scale: float
    rot: object              # RotationConfig or None
    kv_from: object          # a layer index, or None


@dataclasses.dataclass(frozen=True)
class ExpertConfig:
    ff: int
    limit: float


@dataclasses.dataclass(frozen=True)
class MlpConfig:
    kind: str                # dense | moe
    ff: int                  # dense: the inner width; moe: an expert's
    limit: float = 0.0       # moe: where an expert's gate and up halves are clamped
    experts: int = 0
    top: int = 0
    groups: int = 0          # 0: no groups
    keep: int = 0
    shared: object = None    # ExpertConfig or None


@dataclasses.dataclass(frozen=True)
class LayerConfig:
    type: str
    mixer: object
    mlp: object              # MlpConfig or None


def _rotation(r, m, where):
    rot = section(r, m.data, "rot", where + "mixer.", required=False)
    if not rot:
        return None
    sc = section(r, rot.data, "scaling", where + "mixer.rot.", required=False)
    return RotationConfig(rot.integer("dims", minimum=2), rot.number("base", positive=True),
                          sc.number("factor", positive=True) if sc else None,
                          sc.number("original", positive=True) if sc else 0.0,
                          sc.number("fast", positive=True) if sc else 0.0,
                          sc.number("slow", positive=True) if sc else 0.0)


@dataclasses.dataclass(frozen=True)
class RelilixConfig:
    architecture: str
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    layers: tuple
    raw: dict = dataclasses.field(compare=False, default=None)

    @classmethod
    def from_dict(cls, data, where="config.json"):
        r = Reader(data, where)
        arch = r.string("architecture")
        vocab, width = r.integer("vocab", minimum=1), r.integer("width", minimum=1)
        norm = section(r, data, "norm", "")
        eps = norm.number("eps", positive=True) if norm else None
        emb = section(r, data, "embedding", "", required=False)
        emb_scale = emb.number("scale", default=1.0) if emb else 1.0
        raw_layers = data.get("layers")
        if not isinstance(raw_layers, list) or not raw_layers:
            r.problem("'layers' must be a non-empty list")
            raw_layers = []
        layers = [cls._layer(r, entry, f"layers[{i}].") for i, entry in enumerate(raw_layers)]
        r.finish()
        cfg = cls(arch, vocab, width, eps, emb_scale, tuple(layers), data)
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
        if m and kind == "attention":
            heads, dim = m.integer("heads", minimum=1), m.integer("dim", minimum=1)
            mask = section(r, m.data, "mask", where + "mixer.", required=False)
            mixer = AttentionConfig(heads, m.integer("kv_heads", default=heads, minimum=1), dim,
                                    m.integer("vdim", default=dim, minimum=1), m.integer("conv", default=0, minimum=0),
                                    m.number("scale", positive=True), m.number("softcap", default=0.0),
                                    mask.integer("size", default=0, minimum=0) if mask else 0, _rotation(r, m, where))
        elif m:
            dim, rot_dim = m.integer("dim", minimum=1), m.integer("rot_dim", default=0, minimum=0)
            mixer = LatentAttentionConfig(m.integer("heads", minimum=1), dim, rot_dim,
                                          m.integer("vdim", default=dim, minimum=1), m.integer("kv_rank", minimum=1),
                                          m.integer("q_rank", minimum=1), m.number("scale", positive=True),
                                          _rotation(r, m, where), m.integer("kv_from", default=None, minimum=0))
        mlp = None
        if entry.get("mlp") is not None:
            f = section(r, entry, "mlp", where)
            kindf = f.string("kind") if f else None
            if kindf == "dense":
                mlp = MlpConfig("dense", f.integer("ff", minimum=1))
            elif kindf == "moe":
                ex, ro = section(r, f.data, "expert", where + "mlp."), section(r, f.data, "router", where + "mlp.")
                sh = section(r, f.data, "shared", where + "mlp.", required=False)
                if ex and ro:
                    g = section(r, ro.data, "groups", where + "mlp.router.", required=False)
                    shared = ExpertConfig(sh.integer("ff", minimum=1), sh.number("limit", positive=True)) if sh else None
                    mlp = MlpConfig("moe", ex.integer("ff", minimum=1), ex.number("limit", positive=True),
                                    ro.integer("experts", minimum=1), ro.integer("top", minimum=1),
                                    g.integer("count", minimum=1) if g else 0, g.integer("keep", minimum=1) if g else 0,
                                    shared)
            elif kindf is not None:
                r.problem(f"'{where}mlp.kind' is '{kindf}'; known: {', '.join(MLP_KINDS)}")
        return LayerConfig(kind, mixer, mlp)

    def validate(self, where="config"):
        problems = []
        for i, layer in enumerate(self.layers):
            if layer is None or layer.mixer is None:
                continue
            m = layer.mixer
            if layer.type == "attention":
                if m.heads % m.kv_heads:
                    problems.append(f"layers[{i}]: {m.heads} heads over {m.kv_heads} kv_heads")
                if m.vdim != m.dim:
                    problems.append(f"layers[{i}]: values of {m.vdim} channels, but the values are the keys ({m.dim} channels)")
                if m.dim > limits.MAX_HEAD_DIM:
                    problems.append(f"layers[{i}]: heads of {m.dim} channels: the kernels take up to {limits.MAX_HEAD_DIM}")
                if m.taps > limits.MAX_CONV_TAPS:
                    problems.append(f"layers[{i}]: {m.taps} taps: the kernels take up to {limits.MAX_CONV_TAPS}")
                if m.softcap < 0.0:
                    problems.append(f"layers[{i}]: a softcap of {m.softcap}")
                if m.rot is not None and (m.rot.dims % 2 or m.rot.dims > m.dim):
                    problems.append(f"layers[{i}]: {m.rot.dims} turned channels in heads of {m.dim}")
            else:
                if m.rot is not None and (m.rot.dims % 2 or m.rot.dims > m.rot_dim):
                    problems.append(f"layers[{i}]: {m.rot.dims} turned channels in a part of {m.rot_dim}")
                if m.kv_rank > 512:
                    problems.append(f"layers[{i}]: latents of {m.kv_rank} channels: the kernels take up to 512")
                if m.kv_from is not None:
                    src = self.layers[m.kv_from] if m.kv_from < i else None
                    if src is None or src.type != "latent_attention" or src.mixer is None or src.mixer.kv_from is not None:
                        problems.append(f"layers[{i}]: kv_from {m.kv_from} is no earlier latent attention layer with latents of its own")
                    elif (src.mixer.kv_rank, src.mixer.rot_dim, src.mixer.rot) != (m.kv_rank, m.rot_dim, m.rot):
                        problems.append(f"layers[{i}]: latent size or rotation differ from layer {m.kv_from}, whose latents it reads")
            f = layer.mlp
            if f is not None and f.kind == "moe":
                if f.top > f.experts:
                    problems.append(f"layers[{i}]: top {f.top} of {f.experts} experts")
                if f.experts > 4096:
                    problems.append(f"layers[{i}]: {f.experts} experts: the router kernel takes up to 4096")
                if f.groups > 64 or (f.groups and f.experts // f.groups > 64):
                    problems.append(f"layers[{i}]: {f.groups} groups of {f.experts // f.groups} experts: the router kernel takes up to "
                                    f"64 groups of up to 64")
                if f.groups and (f.experts % f.groups or not 1 <= f.keep <= f.groups or f.keep * (f.experts // f.groups) < f.top):
                    problems.append(f"layers[{i}]: {f.groups} groups over {f.experts} experts, {f.keep} kept, top {f.top}")
        if problems:
            raise ConfigError(f"{where}: " + "; ".join(problems))

    def to_dict(self):
        return self.raw
