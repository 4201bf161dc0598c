"""The Relilix decoder as parts.

The embedding rows are multiplied by `embedding.scale`.  A layer is a `PreNormBlock` on a float32 stream: an RMS norm
and a mixer, then (if the layer has one) an RMS norm and a feed-forward.  The mixer is a grouped-query attention behind
short causal taps on its query and key projections, whose values are the keys before their rotation, with capped
scores and a sliding window (`gqa_attention` with `taps`, `softcap` and `value_from_key`), or an attention over cached
latents with a turned key part whose rates are rescaled for long contexts (`latent_attention`).  A latent layer with
`kv_from` makes no latents: the plan hands it the state unit of the layer it names.  The feed-forward is a dense gated
one (silu), or a routed one (sigmoid scores, a correction for the choice only, groups whose score is the sum of their
two best, weights renormalised and applied to the experts' outputs, a clamped gate) plus an expert that every token
runs.

Tensor names: `embed`, `l<i>.norm1`, `l<i>.norm2`, `l<i>.mix.{q,k,q.conv,k.conv,o}` or
`l<i>.mix.{dq,dq.norm,uq,dkv,dkv.norm,uk,uv,g,o}`, `l<i>.mlp.{gate,up,down}` or
`l<i>.mlp.{router,correction,e<j>.{gate,up,down},shared.{gate,up,down}}`, `final.norm`, `head`.
"""
from __future__ import annotations

from ..config.registry import register_architecture
from ..config.relilix import RelilixConfig
from ..engine.definition import ModelDefinition, PlanEntry
from ..parts import build_part
from ..parts.linear import Linear


def _position(rot):
    if rot is None:
        return build_part("position", "none")
    return build_part("position", "paired_rotary", dims=rot.dims, theta=rot.base, factor=rot.factor, original=rot.original,
                      fast=rot.fast, slow=rot.slow)


def _mixer(cfg, i, layer):
    W, m, p = cfg.width, layer.mixer, f"l{i}.mix."
    if layer.type == "attention":
        return build_part("mixer", "gqa_attention", prefix=p, hidden=W, heads=m.heads, kv_heads=m.kv_heads, head_dim=m.dim,
                          window=m.window, position=_position(m.rot), qk_norm_eps=None, output_gate=False, scale=m.scale,
                          softcap=m.softcap, taps=m.taps, value_from_key=True,
                          names={"q": "q", "k": "k", "out": "o", "q_taps": "q.conv", "k_taps": "k.conv"}, out_dtype="float32")
    return build_part("mixer", "latent_attention", prefix=p, hidden=W, heads=m.heads, dim=m.dim, rot_dim=m.rot_dim,
                      value_dim=m.vdim, kv_rank=m.kv_rank, q_rank=m.q_rank, position=_position(m.rot), scale=m.scale,
                      eps=cfg.norm_eps, output_gate=True, shares_latents=m.kv_from is not None, out_dtype="float32")


def _feed_forward(cfg, i, mlp):
    if mlp is None:
        return None
    p, W = f"l{i}.mlp.", cfg.width
    names = {"gate": "gate", "up": "up", "down": "down"}
    if mlp.kind == "dense":
        return build_part("feed_forward", "swiglu", prefix=p, hidden=W, intermediate=mlp.ff, names=names, out_dtype="float32")
    routed = build_part("feed_forward", "routed_swiglu", prefix=p, hidden=W, intermediate=mlp.ff, experts=mlp.experts,
                        top=mlp.top, gate="sigmoid", renormalize=True, weight_on="output", activation="clamped_swish",
                        limit=mlp.limit, correction_name="correction", groups=mlp.groups, keep=mlp.keep, group_best=2,
                        renorm_eps=1e-20)
    if mlp.shared is None:
        return routed
    shared = build_part("feed_forward", "swiglu", prefix=p + "shared.", hidden=W, intermediate=mlp.shared.ff, names=names,
                        out_dtype="float32", activation="clamped_swish", limit=mlp.shared.limit)
    return build_part("feed_forward", "sum", members=[routed, shared])


def define(cfg: RelilixConfig) -> ModelDefinition:
    W = cfg.width
    norm = lambda name: build_part("norm", "rms", name=name, width=W, eps=cfg.norm_eps)
    blocks, plan = [], []
    for i, layer in enumerate(cfg.layers):
        ff = _feed_forward(cfg, i, layer.mlp)
        blocks.append(build_part("block", "prenorm", mixer=_mixer(cfg, i, layer), feed_forward=ff,
                                 input_norm=norm(f"l{i}.norm1"), ffn_norm=norm(f"l{i}.norm2") if ff is not None else None))
        lender = layer.mixer.kv_from if layer.type == "latent_attention" else None
        plan.append(PlanEntry(block=i, state=i) if lender is None else PlanEntry(block=i, state=lender, owns_state=False))
    return ModelDefinition(architecture=cfg.architecture, vocab_size=cfg.vocab, hidden_size=W, embedding_name="embed",
                           blocks=blocks, plan=plan, final_norm=norm("final.norm"), head=Linear("head", cfg.vocab, W),
                           embedding_scale=cfg.embedding_scale, residual_float32=True)


register_architecture("Relilix", RelilixConfig, define)
